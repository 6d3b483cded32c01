// Pre-pass of the split-operand tensor-core kernels for fp32 callers: every fp32 tensor is scaled by a power of two
// (chosen from its largest magnitude) and written as rows [hi (64 fp16, HD used) | lo (64 fp16, HD used)] -- for
// 128-wide heads (forward only) [hi (128) | lo (128)] -- with
// hi = fp16(x), lo = fp16(x - hi): 22 mantissa bits per element, both halves inside the normal range of fp16 for
// every element that matters.
//
// Workspace (one per attention handle or caller):
//   bytes [0,16)     amax[4]   largest |x| of q, k, v, dY as float bit patterns (integer order = float order)
//   bytes [64,128)   fac[16]   scale factors derived from them (all powers of two), see SplitFac
//   bytes [1024,...) four tensors of rows x 128 fp16 (256 for 128-wide heads): q, k, v, dY
#pragma once
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"

namespace split {

enum SplitFac : int {
  FAC_INV_QK = 0,    // 1 / (s_q s_k): logits = (Q' K'^T) x this
  FAC_INV_V = 1,     // 1 / s_v: output = (P V') x this
  FAC_DYV = 2,       // s_dy s_v: delta in the units of dP' = dY' V'^T
  FAC_INV_DYVK = 3,  // 1 / (s_dy s_v s_k): dQ
  FAC_INV_DYVQ = 4,  // 1 / (s_dy s_v s_q): dK
  FAC_INV_DY = 5,    // 1 / s_dy: dV
};

constexpr int TENSOR_Q = 0, TENSOR_K = 1, TENSOR_V = 2, TENSOR_DY = 3;

struct Workspace {
  unsigned int* amax;
  float* fac;
  __half* tensor[4];
};

// fp16 values per row of a split tensor: two halves of 64 (head sizes up to 64) or of 128
__host__ __device__ constexpr int row_halves(int HD) { return HD > 64 ? 256 : 128; }

inline int64_t workspace_bytes(int64_t rows, int HD = 64) { return 1024 + 4 * rows * row_halves(HD) * 2; }

inline Workspace carve(void* base, int64_t rows, int HD = 64) {
  Workspace w;
  w.amax = static_cast<unsigned int*>(base);
  w.fac = reinterpret_cast<float*>(static_cast<char*>(base) + 64);
  __half* t = reinterpret_cast<__half*>(static_cast<char*>(base) + 1024);
  for (int i = 0; i < 4; ++i) w.tensor[i] = t + (size_t)i * rows * row_halves(HD);
  return w;
}

struct Job {
  const float* src[3];   // up to three fp32 tensors with the same element strides
  __half* dst[3];
  int slot[3];           // which amax entry each one owns
};

// Where the i-th 16-byte piece of a (B, H, T, HD) view starts.  A contiguous tensor needs no index arithmetic; otherwise
// the row index (below 2^31) is taken apart with 32-bit divisions.
template <int HD>
__device__ __forceinline__ const float* piece_ptr(const float* x, const McaStrides& st, bool contiguous, int H, int T, int64_t i) {
  if (contiguous) return x + i * 4;
  constexpr int V4 = HD / 4;
  const unsigned row = (unsigned)(i / V4);
  const int c = (int)(i - (int64_t)row * V4);
  const unsigned bh = row / (unsigned)T, t = row - bh * (unsigned)T;
  const unsigned b = bh / (unsigned)H, h = bh - b * (unsigned)H;
  return x + (int64_t)b * st.b + (int64_t)h * st.h + (int64_t)t * st.t + c * 4;
}
__host__ __device__ inline bool is_contiguous(const McaStrides& st, int H, int T, int HD) {
  return st.t == HD && st.h == (int64_t)T * HD && st.b == (int64_t)H * T * HD;
}

// 16-byte load that asks L2 to keep (or to give up first) the line: the reduction reads each tensor once and the row
// kernel reads it again right behind it; three tensors of a layer fit in L2, so the second pass need not go to HBM.
__device__ __forceinline__ uint64_t l2_policy_keep() {
  uint64_t pol;
  asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_drop() {
  uint64_t pol;
  asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ float4 ld_f4_hint(const float* ptr, uint64_t pol) {
  float4 v;
  asm volatile("ld.global.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(ptr), "l"(pol));
  return v;
}

// amax[slot] = max |x| of each tensor
template <int HD>
__global__ void __launch_bounds__(256) amax_kernel(const Job job, McaStrides st, int H, int T, int64_t rows,
                                                   unsigned int* __restrict__ amax) {
  mca_pdl_launch_dependents();
  mca_pdl_wait();   // the tensors are earlier kernels' output
  const float* x = job.src[blockIdx.y];
  constexpr int V4 = HD / 4;
  const bool contiguous = is_contiguous(st, H, T, HD);
  const int64_t n = rows * V4, stride = (int64_t)gridDim.x * blockDim.x;
  float m = 0.f;
  const uint64_t keep = l2_policy_keep();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n; i += 4 * stride) {   // four independent loads in flight
    const float4 v0 = ld_f4_hint(piece_ptr<HD>(x, st, contiguous, H, T, i), keep);
    const float4 v1 = ld_f4_hint(piece_ptr<HD>(x, st, contiguous, H, T, i + stride), keep);
    const float4 v2 = ld_f4_hint(piece_ptr<HD>(x, st, contiguous, H, T, i + 2 * stride), keep);
    const float4 v3 = ld_f4_hint(piece_ptr<HD>(x, st, contiguous, H, T, i + 3 * stride), keep);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))));
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v2.x), fabsf(v2.y)), fmaxf(fabsf(v2.z), fabsf(v2.w))));
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v3.x), fabsf(v3.y)), fmaxf(fabsf(v3.z), fabsf(v3.w))));
  }
  for (; i < n; i += stride) {
    const float4 v = ld_f4_hint(piece_ptr<HD>(x, st, contiguous, H, T, i), keep);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
  // one atomic per block: thousands of warps updating the same three words serialise in L2
  __shared__ float s_m[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) s_m[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < 8 ? s_m[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (threadIdx.x == 0 && m > 0.f) atomicMax(amax + job.slot[blockIdx.y], __float_as_uint(m));
  }
}

// The power of two that brings max |x| into [2^12, 2^13): the largest fp16 is 65504 and the low half of an element
// is about 2^-11 of it, so both halves of everything within 2^-14 of the maximum are normal fp16 numbers.
__device__ __forceinline__ float pow2_scale(unsigned int amax_bits) {
  const float a = __uint_as_float(amax_bits);
  if (!(a > 0.f) || !(a < 3.0e38f)) return 1.0f;
  int e;
  frexpf(a, &e);                    // a = f * 2^e, f in [0.5, 1)
  return ldexpf(1.0f, 13 - e);
}

// backward with ydot / delta given: also delta[row] = sum_c x[row][c] * ydot[row][c] (ydot contiguous rows), the
// softmax backward's row term, from the elements this kernel holds anyway.
template <int HD>
__global__ void __launch_bounds__(256) rows_kernel(const Job job, McaStrides st, int H, int T, int64_t rows,
                                                   const unsigned int* __restrict__ amax, float* __restrict__ fac,
                                                   int backward, const float* __restrict__ ydot, float* __restrict__ delta) {
  mca_pdl_launch_dependents();
  mca_pdl_wait();   // the magnitudes are the reduction's output
  const int which = blockIdx.y;
  const float* x = job.src[which];
  __half* dst = job.dst[which];
  const float sc = pow2_scale(amax[job.slot[which]]);
  if (which == 0 && blockIdx.x == 0 && threadIdx.x == 0) {
    const float sq = pow2_scale(amax[TENSOR_Q]), sk = pow2_scale(amax[TENSOR_K]), sv = pow2_scale(amax[TENSOR_V]);
    if (!backward) {
      fac[FAC_INV_QK] = 1.0f / (sq * sk);   // powers of two: every product and quotient here is exact
      fac[FAC_INV_V] = 1.0f / sv;
    } else {
      const float sdy = pow2_scale(amax[TENSOR_DY]);
      fac[FAC_DYV] = sdy * sv;
      fac[FAC_INV_DYVK] = 1.0f / (sdy * sv * sk);
      fac[FAC_INV_DYVQ] = 1.0f / (sdy * sv * sq);
      fac[FAC_INV_DY] = 1.0f / sdy;
    }
  }
  // eight elements per thread and step: two 16-byte loads (adjacent pieces of one row), one 16-byte store per half
  constexpr int V8 = HD / 8;
  const bool contiguous = is_contiguous(st, H, T, HD);
  const uint64_t drop = l2_policy_drop();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * V8; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / V8;          // V8 is a power of two
    const int c = (int)(i - row * V8);
    const float* src = piece_ptr<HD>(x, st, contiguous, H, T, 2 * i);
    const float4 v0 = ld_f4_hint(src, drop), v1 = ld_f4_hint(src + 4, drop);
    if (delta != nullptr) {   // uniform: the HD / 8 consecutive lanes of a row are all in this iteration
      const float4 y0 = *reinterpret_cast<const float4*>(ydot + i * 8), y1 = *reinterpret_cast<const float4*>(ydot + i * 8 + 4);
      float acc = fmaf(v0.x, y0.x, fmaf(v0.y, y0.y, fmaf(v0.z, y0.z, v0.w * y0.w)));
      acc += fmaf(v1.x, y1.x, fmaf(v1.y, y1.y, fmaf(v1.z, y1.z, v1.w * y1.w)));
      const unsigned active = __activemask();
#pragma unroll
      for (int o = V8 / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(active, acc, o);
      if (c == 0) delta[row] = acc;
    }
    const float e[8] = {v0.x * sc, v0.y * sc, v0.z * sc, v0.w * sc, v1.x * sc, v1.y * sc, v1.z * sc, v1.w * sc};
    __align__(16) __half hi[8];
    __align__(16) __half lo[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      hi[j] = __float2half_rn(e[j]);
      lo[j] = __float2half_rn(e[j] - __half2float(hi[j]));
    }
    constexpr int RH = row_halves(HD);
    __half* o = dst + row * RH + c * 8;
    *reinterpret_cast<uint4*>(o) = *reinterpret_cast<const uint4*>(hi);
    *reinterpret_cast<uint4*>(o + RH / 2) = *reinterpret_cast<const uint4*>(lo);
  }
}

// Split `count` tensors (q, k, v for the forward; dY for the backward) into the workspace.
template <int HD>
inline int run(const Job& job, int count, const McaStrides& st, int H, int T, int64_t rows, const Workspace& w, bool backward,
               cudaStream_t stream, const float* ydot = nullptr, float* delta = nullptr) {
  // the slots of this call's tensors are consecutive (q, k, v or dY alone): one clear
  int lo = job.slot[0], hi = job.slot[0];
  for (int i = 1; i < count; ++i) { lo = std::min(lo, job.slot[i]); hi = std::max(hi, job.slot[i]); }
  MCA_CUDA_TRY(cudaMemsetAsync(w.amax + lo, 0, sizeof(unsigned int) * (size_t)(hi - lo + 1), stream));
  // the reduction as one wave of resident blocks over all its tensors (eight blocks of 256 threads per SM)
  const int blocks_amax = (int)std::min<int64_t>((148 * 8) / count, (rows * (HD / 4) + 4 * 256 - 1) / (4 * 256));
  int e = mca_launch_pdl(amax_kernel<HD>, dim3(std::max(1, blocks_amax), count), dim3(256), 0, stream, job, st, H, T, rows, w.amax);
  if (e) return e;
  const int blocks_rows = (int)std::min<int64_t>(148 * 8, (rows * (HD / 8) + 255) / 256);
  return mca_launch_pdl(rows_kernel<HD>, dim3(blocks_rows, count), dim3(256), 0, stream, job, st, H, T, rows, w.amax, w.fac,
                        backward ? 1 : 0, ydot, delta);
}

}  // namespace split

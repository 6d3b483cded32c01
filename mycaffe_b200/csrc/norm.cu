// Row normalisations that sit either side of the attention block in every transformer layer,
// each as ONE pass over the tensor (read x once, write y once), bound by HBM bandwidth:
//   * LayerNorm forward / backward -- replaces LayerNormData<T>::Forward / Backward
//     (CudaDnnDLL/Cuda Files/layernorm.cu:291-333, :340-384), which issue 10 and 9 elementwise or
//     reduction kernels over seven full-size scratch tensors; their row means are computed by one
//     thread per row walking the row serially (channel_mean_kernel, math.cu:6817-6831).
//   * RMSNorm layer forward / backward -- replaces the 8 (forward) and 14 (backward) CudaDnn calls of
//     RMSNormLayer<T>.forward / backward (MyCaffe.layers.gpt/layers.gpt/RMSNormLayer.cs:156-179, :190-231).
// A row is held in the registers of a group of G threads (a warp for short rows, a whole CTA for
// long ones); sums are reduced with shuffles (and one pass through shared memory for G > 32) in a
// fixed order, so results do not depend on timing.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int NORM_MAX_PARTIALS = 296;   // CTAs of the RMSNorm backward (two per SM): one dW partial each

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the G threads that share a row.  G == 32: the warp.  G > 32: the CTA (G == blockDim.x).
template <int G>
__device__ __forceinline__ float group_sum(float v, float* sred) {
  v = warp_sum(v);
  if (G == 32) return v;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sred[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < G / 32; ++w) t += sred[w];
  __syncthreads();
  return t;
}

// The part of a row one thread holds: MAXV pieces of VEC floats, piece i at element (i*G + g)*VEC.
template <int G, int MAXV, int VEC>
struct RowPart {
  float v[MAXV][VEC];
  __device__ __forceinline__ void load(const float* row, int inner, int g) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int e = (i * G + g) * VEC;
      if (e < inner) {
        if (VEC == 4) {
          const float4 t = *reinterpret_cast<const float4*>(row + e);
          v[i][0] = t.x; v[i][1 % VEC] = t.y; v[i][2 % VEC] = t.z; v[i][3 % VEC] = t.w;
        } else {
          v[i][0] = row[e];
        }
      } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) v[i][j] = 0.f;
      }
    }
  }
  __device__ __forceinline__ void store(float* row, int inner, int g) const {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int e = (i * G + g) * VEC;
      if (e < inner) {
        if (VEC == 4) *reinterpret_cast<float4*>(row + e) = make_float4(v[i][0], v[i][1 % VEC], v[i][2 % VEC], v[i][3 % VEC]);
        else row[e] = v[i][0];
      }
    }
  }
};

// which: 0 LayerNorm forward, 1 LayerNorm backward, 2 RMSNorm forward, 3 RMSNorm backward
struct NormParams {
  const float* a;      // LN fwd: x.  LN bwd: y.  RMS fwd: x.  RMS bwd: x
  const float* b;      // LN bwd: dy.  RMS bwd: dy
  const float* w;      // RMS: weights or null
  const float* stat;   // LN bwd: stdev (rows).  RMS bwd: 1/rms (rows)
  float* out;          // y or dx
  float* stat_out;     // LN fwd: stdev.  RMS fwd: 1/rms (may be null)
  float* dw_partial;   // RMS bwd: (gridDim.x, inner) or null
  int64_t rows;
  int inner;
  float eps;
};

template <int WHICH, int G, int MAXV, int VEC>
__global__ void __launch_bounds__(G == 32 ? 256 : G) norm_rows_kernel(const NormParams p) {
  __shared__ float sred[32];
  extern __shared__ float dw_smem[];   // RMS bwd with G == 32: (inner) floats, the CTA's dW partial
  constexpr int GROUPS = G == 32 ? 8 : 1;   // rows in flight per CTA
  const int g = threadIdx.x % G, grp = threadIdx.x / G;
  const int inner = p.inner;
  const float inv_n = 1.0f / (float)inner;
  RowPart<G, MAXV, VEC> dw;
  if (WHICH == 3) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i)
#pragma unroll
      for (int j = 0; j < VEC; ++j) dw.v[i][j] = 0.f;
  }
  // every group walks the same number of rows so that the CTA-wide barriers of G > 32 stay uniform
  for (int64_t row0 = (int64_t)blockIdx.x * GROUPS; row0 < p.rows; row0 += (int64_t)gridDim.x * GROUPS) {
    const int64_t row = row0 + grp;
    const bool live = row < p.rows;
    const int64_t off = (live ? row : 0) * inner;
    RowPart<G, MAXV, VEC> x;
    x.load(p.a + off, inner, g);
    if (WHICH == 0) {
      // mean, centred squares, stdev = sqrt(var + eps), y = (x - mean) / stdev   (layernorm.cu:296-330)
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < MAXV; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) s += x.v[i][j];
      const float mean = group_sum<G>(s, sred) * inv_n;
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < MAXV; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const bool in = (i * G + g) * VEC + j < inner;
          x.v[i][j] = in ? x.v[i][j] - mean : 0.f;
          q += x.v[i][j] * x.v[i][j];
        }
      const float sd = sqrtf(group_sum<G>(q, sred) * inv_n + p.eps);
#pragma unroll
      for (int i = 0; i < MAXV; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) x.v[i][j] = x.v[i][j] / sd;
      if (live) {
        x.store(p.out + off, inner, g);
        if (g == 0) p.stat_out[row] = sd;
      }
    } else if (WHICH == 1) {
      // dx = (dy - (y * mean(y*dy) + mean(dy))) / stdev   (layernorm.cu:345-381).  The reference adds eps
      // to the first `rows` ELEMENTS of its row-broadcast stdev tensor before the division
      // (add_scalar over outer*channels items of a count-sized buffer, :377): reproduced here.
      RowPart<G, MAXV, VEC> dy;
      dy.load(p.b + off, inner, g);
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < MAXV; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) { s1 = fmaf(x.v[i][j], dy.v[i][j], s1); s2 += dy.v[i][j]; }
      const float m1 = group_sum<G>(s1, sred) * inv_n;
      const float m2 = group_sum<G>(s2, sred) * inv_n;
      const float sd = p.stat[live ? row : 0];
#pragma unroll
      for (int i = 0; i < MAXV; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const int64_t flat = off + (i * G + g) * VEC + j;
          const float denom = flat < p.rows ? sd + p.eps : sd;
          x.v[i][j] = (dy.v[i][j] - (x.v[i][j] * m1 + m2)) / denom;
        }
      if (live) x.store(p.out + off, inner, g);
    } else if (WHICH == 2) {
      // rms = sqrt(mean(x^2) + eps); y = w * (x * (1 / rms))   (RMSNormLayer.cs:158-173)
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < MAXV; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) q = fmaf(x.v[i][j], x.v[i][j], q);
      const float rms = sqrtf(group_sum<G>(q, sred) * inv_n + p.eps);
      const float inv = rms == 0.f ? 0.f : 1.0f / rms;   // invert_kernel maps 0 to 0, math.cu:6018-6024
      if (p.w != nullptr) {
        RowPart<G, MAXV, VEC> w;
        w.load(p.w, inner, g);
#pragma unroll
        for (int i = 0; i < MAXV; ++i)
#pragma unroll
          for (int j = 0; j < VEC; ++j) x.v[i][j] = w.v[i][j] * (x.v[i][j] * inv);
      } else {
#pragma unroll
        for (int i = 0; i < MAXV; ++i)
#pragma unroll
          for (int j = 0; j < VEC; ++j) x.v[i][j] = x.v[i][j] * inv;
      }
      if (live) {
        x.store(p.out + off, inner, g);
        if (g == 0 && p.stat_out != nullptr) p.stat_out[row] = inv;
      }
    } else {
      // g = dy * w; dW += dy * (x * inv); dx = g * inv - x * sum(g * x) * inv^3 / n   (RMSNormLayer.cs:194-229:
      // dinv = sum(g x), drms = -dinv / rms^2, dmean = drms / (2 rms), dx += 2 x dmean / n)
      RowPart<G, MAXV, VEC> dy;
      dy.load(p.b + off, inner, g);
      const float inv = live ? p.stat[row] : 0.f;
      if (p.w != nullptr) {
        RowPart<G, MAXV, VEC> w;
        w.load(p.w, inner, g);
#pragma unroll
        for (int i = 0; i < MAXV; ++i)
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            dw.v[i][j] = fmaf(dy.v[i][j], x.v[i][j] * inv, dw.v[i][j]);
            dy.v[i][j] *= w.v[i][j];
          }
      }
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < MAXV; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) s = fmaf(dy.v[i][j], x.v[i][j], s);
      const float dinv = group_sum<G>(s, sred);
      const float drms = -dinv * (inv * inv);
      const float dmean = drms * (0.5f * inv);
      const float c = 2.0f * dmean * inv_n;
#pragma unroll
      for (int i = 0; i < MAXV; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) x.v[i][j] = fmaf(x.v[i][j], c, dy.v[i][j] * inv);
      if (live) x.store(p.out + off, inner, g);
    }
  }
  if (WHICH == 3 && p.dw_partial != nullptr) {
    float* dst = p.dw_partial + (int64_t)blockIdx.x * inner;
    if (G == 32) {   // the CTA's eight row groups add their partials in group order
      for (int e = threadIdx.x; e < inner; e += blockDim.x) dw_smem[e] = 0.f;
      __syncthreads();
      for (int turn = 0; turn < GROUPS; ++turn) {
        if (grp == turn) {
#pragma unroll
          for (int i = 0; i < MAXV; ++i)
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
              const int e = (i * G + g) * VEC + j;
              if (e < inner) dw_smem[e] += dw.v[i][j];
            }
        }
        __syncthreads();
      }
      for (int e = threadIdx.x; e < inner; e += blockDim.x) dst[e] = dw_smem[e];
    } else {
      dw.store(dst, inner, g);
    }
  }
}

// dW[e] = sum over the CTAs' partials, in CTA order
__global__ void norm_dw_reduce_kernel(const float* __restrict__ partial, int n_partials, int inner, float* __restrict__ dw) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= inner) return;
  float s = 0.f;
  for (int c = 0; c < n_partials; ++c) s += partial[(int64_t)c * inner + e];
  dw[e] = s;
}

struct Shape { int G, MAXV, VEC; };

// the narrowest group that holds a row; vector loads need inner % 4 == 0 and 16-byte aligned tensors
bool pick(int inner, bool aligned, Shape* s) {
  if (aligned && inner % 4 == 0) {
    if (inner <= 32 * 8 * 4) { *s = {32, 8, 4}; return true; }
    if (inner <= 256 * 4 * 4) { *s = {256, 4, 4}; return true; }
    if (inner <= 1024 * 4 * 4) { *s = {1024, 4, 4}; return true; }
    return false;
  }
  if (inner <= 32 * 16) { *s = {32, 16, 1}; return true; }
  if (inner <= 1024 * 16) { *s = {1024, 16, 1}; return true; }
  return false;
}

template <int WHICH, int G, int MAXV, int VEC>
int launch_norm(NormParams p, int grid_cap, cudaStream_t st) {
  constexpr int GROUPS = G == 32 ? 8 : 1;
  constexpr int THREADS = G == 32 ? 256 : G;
  const int64_t want = (p.rows + GROUPS - 1) / GROUPS;
  const int grid = (int)std::min<int64_t>(want, grid_cap);
  const size_t smem = (WHICH == 3 && G == 32 && p.dw_partial) ? sizeof(float) * (size_t)p.inner : 0;
  norm_rows_kernel<WHICH, G, MAXV, VEC><<<grid, THREADS, smem, st>>>(p);
  return mca_launch_status();
}

template <int WHICH>
int dispatch_norm(const NormParams& p, bool aligned, int grid_cap, cudaStream_t st) {
  Shape s;
  if (!pick(p.inner, aligned, &s)) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  if (s.VEC == 4) {
    if (s.G == 32) return launch_norm<WHICH, 32, 8, 4>(p, grid_cap, st);
    if (s.G == 256) return launch_norm<WHICH, 256, 4, 4>(p, grid_cap, st);
    return launch_norm<WHICH, 1024, 4, 4>(p, grid_cap, st);
  }
  if (s.G == 32) return launch_norm<WHICH, 32, 16, 1>(p, grid_cap, st);
  return launch_norm<WHICH, 1024, 16, 1>(p, grid_cap, st);
}

bool a16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
constexpr int NORM_GRID_CAP = 148 * 16;

}  // namespace

int mca_layernorm_forward_f32(const float* x, float* y, float* stdev, int64_t rows, int inner, float eps, void* stream) {
  if (!x || !y || !stdev) return ERROR_PARAM_NULL;
  if (rows <= 0 || inner <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  NormParams p = {};
  p.a = x; p.out = y; p.stat_out = stdev; p.rows = rows; p.inner = inner; p.eps = eps;
  return dispatch_norm<0>(p, a16(x) && a16(y), NORM_GRID_CAP, (cudaStream_t)stream);
}

int mca_layernorm_backward_f32(const float* y, const float* dy, const float* stdev, float* dx, int64_t rows, int inner,
                               float eps, void* stream) {
  if (!y || !dy || !stdev || !dx) return ERROR_PARAM_NULL;
  if (rows <= 0 || inner <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  NormParams p = {};
  p.a = y; p.b = dy; p.stat = stdev; p.out = dx; p.rows = rows; p.inner = inner; p.eps = eps;
  return dispatch_norm<1>(p, a16(y) && a16(dy) && a16(dx), NORM_GRID_CAP, (cudaStream_t)stream);
}

int mca_rmsnorm_forward_f32(const float* x, const float* w, float* y, float* inv_rms, int64_t rows, int inner, float eps,
                            void* stream) {
  if (!x || !y) return ERROR_PARAM_NULL;
  if (rows <= 0 || inner <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  NormParams p = {};
  p.a = x; p.w = w; p.out = y; p.stat_out = inv_rms; p.rows = rows; p.inner = inner; p.eps = eps;
  return dispatch_norm<2>(p, a16(x) && a16(y) && a16(w), NORM_GRID_CAP, (cudaStream_t)stream);
}

int64_t mca_rmsnorm_backward_scratch_floats(int inner) { return (int64_t)NORM_MAX_PARTIALS * inner; }

int mca_rmsnorm_backward_f32(const float* x, const float* w, const float* dy, const float* inv_rms, float* dx, float* dw,
                             float* scratch, int64_t scratch_floats, int64_t rows, int inner, void* stream) {
  if (!x || !dy || !inv_rms || !dx) return ERROR_PARAM_NULL;
  if (rows <= 0 || inner <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (dw != nullptr && (w == nullptr || scratch == nullptr)) return ERROR_PARAM_NULL;
  if (dw != nullptr && scratch_floats < mca_rmsnorm_backward_scratch_floats(inner)) return ERROR_ATTN_SCRATCH_TOO_SMALL;
  NormParams p = {};
  p.a = x; p.b = dy; p.w = w; p.stat = inv_rms; p.out = dx; p.dw_partial = dw ? scratch : nullptr;
  p.rows = rows; p.inner = inner;
  Shape s;
  const bool aligned = a16(x) && a16(dy) && a16(dx) && a16(w) && a16(scratch);
  if (!pick(inner, aligned, &s)) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  const int groups = s.G == 32 ? 8 : 1;
  const int grid = (int)std::min<int64_t>((rows + groups - 1) / groups, NORM_MAX_PARTIALS);
  int e = dispatch_norm<3>(p, aligned, NORM_MAX_PARTIALS, (cudaStream_t)stream);
  if (e || dw == nullptr) return e;
  norm_dw_reduce_kernel<<<mca_ceil_div(inner, 256), 256, 0, (cudaStream_t)stream>>>(scratch, grid, inner, dw);
  return mca_launch_status();
}

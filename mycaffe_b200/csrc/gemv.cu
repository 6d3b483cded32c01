// Weight-streaming projections of the llama2 decode attention block, fused with what surrounds them:
//   * RMSNorm + Wq/Wk/Wv:  q,k,v = W · (w_rms ∘ x / sqrt(mean(x²) + eps))
//   * Wo + residual:       x += Wo · attn
//   * RMSNorm + W1/W3 + SwiGLU:  h = silu(W1 · xn) ∘ (W3 · xn)   (llama2_gpu.cpp:84-91, llama2_cpu.cpp:352-368)
//   * W2 + residual:       x += W2 · h                           (llama2_gpu.cpp:94-97)
//   * final RMSNorm + classifier: logits = Wcls · xn             (llama2_gpu.cpp:101-105)
// Replaces, for one new token, Primitives::rmsnorm (a square kernel, a thrust::reduce with a
// device-to-host round trip and a scale kernel; CudaExtension.llm32.llama2/Files/
// primitives.cu:281-303) followed by three cublasSgemv calls (primitives.cu:322-340;
// llama2_gpu.cpp:56-61), and the Wo cublasSgemv plus the residual add kernel
// (llama2_gpu.cpp:78-81).  The arithmetic follows the CPU twin (rmsnorm llama2_cpu.cpp:189-202,
// matmul :224-237): o[j] = w[j] * (s * x[j]) with s = 1/sqrt(sum(x²)/n + eps).
//
// These are GEMVs: the weights (dim x dim floats, 67 MB at dim 4096) are read exactly once and
// nothing else matters, so the kernel is bound by HBM bandwidth and is built around keeping
// enough weight bytes in flight.  Every warp streams its part of the matrix through a ring in
// shared memory filled by cp.async: each lane copies the 16-byte vectors it will itself consume,
// DEPTH-1 steps ahead, so no synchronisation other than its own wait_group is needed and the
// bytes in flight do not depend on registers or occupancy.  The first steps of the ring leave
// for HBM before the CTA stages (and RMS-normalises) the activations in shared memory.
// Rows are dealt to groups of S warps of one CTA in contiguous, balanced ranges; with S > 1 (few,
// long rows, as Wo and W2 have) the warps of a group split every row along K and their partial
// sums are added in a fixed order through shared memory, so results do not depend on timing.
// Up to 8 sequences share one pass over the weights (then two rows at a time per warp share the
// activation reads); larger batches take several passes.
#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "proj_tc.cuh"

namespace {

constexpr int GV_SPLIT_STEPS = 16;   // row steps a K-split group may own (their sums wait in registers)
constexpr size_t GV_SMEM_LIMIT = 226 * 1024;

template <typename WT> struct WLoad;
template <> struct WLoad<float> {
  static constexpr int VEC = 4;
  static __device__ __forceinline__ void unpack(const uint4& t, float (&w)[4]) {
    w[0] = __uint_as_float(t.x); w[1] = __uint_as_float(t.y); w[2] = __uint_as_float(t.z); w[3] = __uint_as_float(t.w);
  }
};
template <> struct WLoad<__nv_bfloat16> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ void unpack(const uint4& t, float (&w)[8]) {
    const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { w[2 * i] = __uint_as_float(u[i] << 16); w[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
  }
};

struct GemvParams {
  const float* x;        // (B, n) input activations
  const float* norm_w;   // (n) RMSNorm weights or null (no normalisation)
  const void* w[3];      // up to three stacked matrices, each (rows[i], n) row-major
  float* out[3];         // (B, rows[i]) each
  int rows[3];
  int n_mats, B, n, accumulate;  // accumulate: out += result (residual connection)
  int swiglu;                    // out[0][r] = silu(w[0] row r . x) * (w[1] row r . x); rows[1] == rows[0]
  int split;                     // S: warps of a CTA that share a row along K (1, 2, 4 or 8)
  float eps;
};

// NB sequences per pass, R weight rows per step per warp (they share the activation reads from
// shared memory), THREADS per CTA, DEPTH ring steps per warp, each of U warp-wide vectors per row.  GLU: the two rows of a step are
// row r of w[0] and row r of w[1], combined by SwiGLU (R must be 2); otherwise they are
// consecutive rows of the stacked matrix.
template <typename WT, int NB, int R, int THREADS, bool GLU, int DEPTH, int U>
__global__ void __launch_bounds__(THREADS) gemv_stream_kernel(const GemvParams p, int b0) {
  static_assert(!GLU || R == 2, "the gated form pairs one row of each matrix");
  constexpr int STEP = GLU ? 1 : R;   // output rows finished per step
  constexpr int WARPS = THREADS / 32;
  constexpr int VEC = WLoad<WT>::VEC;
  extern __shared__ __align__(16) unsigned char gv_smem[];
  __shared__ float red[WARPS][NB];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = p.n;
  float* xs = reinterpret_cast<float*>(gv_smem);                                    // [NB][n] activations
  uint4* ring = reinterpret_cast<uint4*>(gv_smem + sizeof(float) * (size_t)NB * n); // [WARPS][DEPTH][R][U][32]
  uint4* my_ring = ring + (size_t)warp * DEPTH * R * U * 32;
  const uint32_t my_ring_s = (uint32_t)__cvta_generic_to_shared(my_ring);

  const int total_rows = GLU ? p.rows[0] : p.rows[0] + (p.n_mats > 1 ? p.rows[1] : 0) + (p.n_mats > 2 ? p.rows[2] : 0);
  const int total_steps = (total_rows + STEP - 1) / STEP;
  const int S = p.split;
  const int groups = gridDim.x * (WARPS / S);
  auto group_begin = [&](int g) { return (int)(((int64_t)g * total_steps) / groups); };
  const int gid = blockIdx.x * (WARPS / S) + warp / S;
  const int step_lo = group_begin(gid);
  const int n_steps = group_begin(gid + 1) - step_lo;
  const int chunks = (n + 32 * VEC * U - 1) / (32 * VEC * U);    // ring steps per row
  const int seg = warp % S;
  const int c_lo = (seg * chunks) / S, c_hi = ((seg + 1) * chunks) / S;   // this warp's part of every row

  // operand q of the step that starts at output row r: which matrix, which of its rows
  auto row_ptr = [&](int r, int q, int& m, int& rr) -> const WT* {
    if (GLU) {
      m = q; rr = min(r, total_rows - 1);
    } else {
      m = 0; rr = min(r + q, total_rows - 1);
      if (rr >= p.rows[0]) { rr -= p.rows[0]; m = 1; if (rr >= p.rows[1]) { rr -= p.rows[1]; m = 2; } }
    }
    const void* base = m == 0 ? p.w[0] : (m == 1 ? p.w[1] : p.w[2]);  // no dynamic indexing of the parameter block
    return reinterpret_cast<const WT*>(base) + (int64_t)rr * n;
  };
  // ---- producer side of the ring
  const WT* i_ptr[R];
  int i_step = 0, i_c = c_lo, i_slot = 0;
  auto set_issue_rows = [&]() {
#pragma unroll
    for (int q = 0; q < R; ++q) { int m, rr; i_ptr[q] = row_ptr((step_lo + i_step) * STEP, q, m, rr); }
  };
  set_issue_rows();
  auto issue = [&]() {
    if (i_step < n_steps && c_lo < c_hi) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = ((i_c * U + u) * 32 + lane) * VEC;
        if (k < n) {
#pragma unroll
          for (int q = 0; q < R; ++q)
            mca_cp_async16(my_ring_s + (uint32_t)((((i_slot * R + q) * U + u) * 32 + lane) * sizeof(uint4)), i_ptr[q] + k);
        }
      }
      if (++i_c == c_hi) { i_c = c_lo; ++i_step; set_issue_rows(); }
    }
    mca_cp_async_commit();   // one group per step, also when it is empty, so that the group count is the step count
    i_slot = (i_slot + 1 == DEPTH) ? 0 : i_slot + 1;
  };
  // The first weight vectors leave for HBM before anything else -- also before the kernel that
  // produces the activations has finished (programmatic dependent launch): weights depend on nothing.
  mca_pdl_launch_dependents();
#pragma unroll
  for (int t = 0; t < DEPTH - 1; ++t) issue();
  mca_pdl_wait();   // from here on the previous kernel's results are complete and visible

  // ---- phase 1: activations of this pass's sequences -> shared memory, RMS-normalised
  float ss[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) ss[b] = 0.f;
  for (int k = tid * 4; k < n; k += THREADS * 4) {
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      const float4 v = *reinterpret_cast<const float4*>(p.x + (int64_t)(b0 + b) * n + k);
      *reinterpret_cast<float4*>(xs + b * n + k) = v;
      ss[b] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
  if (p.norm_w != nullptr) {
#pragma unroll
    for (int b = 0; b < NB; ++b) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss[b] += __shfl_xor_sync(0xffffffffu, ss[b], o);
      if (lane == 0) red[warp][b] = ss[b];
    }
    __syncthreads();
    float scale[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) t += red[w][b];
      t = t / (float)n + p.eps;
      scale[b] = 1.0f / sqrtf(t);
    }
    for (int k = tid * 4; k < n; k += THREADS * 4) {
      const float4 g = *reinterpret_cast<const float4*>(p.norm_w + k);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float4 v = *reinterpret_cast<float4*>(xs + b * n + k);
        v.x = g.x * (scale[b] * v.x); v.y = g.y * (scale[b] * v.y); v.z = g.z * (scale[b] * v.z); v.w = g.w * (scale[b] * v.w);
        *reinterpret_cast<float4*>(xs + b * n + k) = v;
      }
    }
  }
  __syncthreads();

  // finished sums of output step `step` (values of rows r .. r+R-1, or the gate pair) -> memory
  auto emit = [&](int step, const float (&v)[R][NB]) {
    const int r = step * STEP;
    if (GLU) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        // val = hb * (1 / (1 + exp(-hb))) * hb2, llama2_cpu.cpp:359-367
        float val = v[0][b];
        val *= (1.0f / (1.0f + expf(-val)));
        val *= v[R - 1][b];
        p.out[0][(int64_t)(b0 + b) * p.rows[0] + r] = val;
      }
    } else {
#pragma unroll
      for (int q = 0; q < R; ++q) {
        if (r + q >= total_rows) continue;
        int m, rr;
        row_ptr(r, q, m, rr);
        float* ob = m == 0 ? p.out[0] : (m == 1 ? p.out[1] : p.out[2]);
        const int orows = m == 0 ? p.rows[0] : (m == 1 ? p.rows[1] : p.rows[2]);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float* dst = ob + (int64_t)(b0 + b) * orows + rr;
          *dst = p.accumulate ? (*dst + v[q][b]) : v[q][b];
        }
      }
    }
  };

  // ---- phase 2: consume the ring
  float acc[R][NB], keep[R][NB];
#pragma unroll
  for (int q = 0; q < R; ++q)
#pragma unroll
    for (int b = 0; b < NB; ++b) { acc[q][b] = 0.f; keep[q][b] = 0.f; }
  const int T = (c_lo < c_hi) ? n_steps * (c_hi - c_lo) : 0;
  int c = c_lo, step = 0, slot = 0;
  for (int t = 0; t < T; ++t) {
    issue();
    mca_cp_async_wait<DEPTH - 1>();
#pragma unroll
    for (int u = 0; u < U; ++u) {
    const int k = ((c * U + u) * 32 + lane) * VEC;
    if (k < n) {
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const uint4 raw = my_ring[((slot * R + q) * U + u) * 32 + lane];
        float w[VEC];
        WLoad<WT>::unpack(raw, w);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const float* xv = xs + b * n + k;
#pragma unroll
          for (int i = 0; i < VEC; i += 4) {
            const float4 xx = *reinterpret_cast<const float4*>(xv + i);
            acc[q][b] = fmaf(w[i], xx.x, acc[q][b]); acc[q][b] = fmaf(w[i + 1], xx.y, acc[q][b]);
            acc[q][b] = fmaf(w[i + 2], xx.z, acc[q][b]); acc[q][b] = fmaf(w[i + 3], xx.w, acc[q][b]);
          }
        }
      }
    }
    }
    slot = (slot + 1 == DEPTH) ? 0 : slot + 1;
    if (++c == c_hi) {   // this warp's part of the step is complete
#pragma unroll
      for (int q = 0; q < R; ++q)
#pragma unroll
        for (int b = 0; b < NB; ++b) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) acc[q][b] += __shfl_xor_sync(0xffffffffu, acc[q][b], o);
        }
      if (S == 1) {
        if (lane == 0) emit(step_lo + step, acc);
      } else if (lane == step) {   // lane i keeps the sums of the group's step i until the group adds them
#pragma unroll
        for (int q = 0; q < R; ++q)
#pragma unroll
          for (int b = 0; b < NB; ++b) keep[q][b] = acc[q][b];
      }
#pragma unroll
      for (int q = 0; q < R; ++q)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[q][b] = 0.f;
      c = c_lo; ++step;
    }
  }
  mca_cp_async_wait<0>();
  if (S == 1) return;   // uniform over the CTA

  // ---- K-split groups: partial sums -> this warp's (now idle) ring -> added in warp order
  float* my_part = reinterpret_cast<float*>(my_ring);   // [GV_SPLIT_STEPS][R][NB]
  if (lane < n_steps && lane < GV_SPLIT_STEPS) {
#pragma unroll
    for (int q = 0; q < R; ++q)
#pragma unroll
      for (int b = 0; b < NB; ++b) my_part[(lane * R + q) * NB + b] = keep[q][b];
  }
  __syncthreads();
  if (seg == 0 && lane < n_steps && lane < GV_SPLIT_STEPS) {
    float v[R][NB];
#pragma unroll
    for (int q = 0; q < R; ++q)
#pragma unroll
      for (int b = 0; b < NB; ++b) v[q][b] = 0.f;
    for (int s2 = 0; s2 < S; ++s2) {
      const float* part = reinterpret_cast<const float*>(ring + (size_t)(warp + s2) * DEPTH * R * U * 32);
#pragma unroll
      for (int q = 0; q < R; ++q)
#pragma unroll
        for (int b = 0; b < NB; ++b) v[q][b] += part[(lane * R + q) * NB + b];
    }
    emit(step_lo + lane, v);
  }
}

template <int R, int THREADS, int DEPTH, int U = 1>
constexpr size_t ring_bytes() { return (size_t)(THREADS / 32) * DEPTH * R * U * 32 * sizeof(uint4); }

template <typename WT, int NB, int R, int THREADS, bool GLU, int DEPTH, int U = 1>
int launch_pass(GemvParams p, int b0, cudaStream_t st) {
  constexpr int STEP = GLU ? 1 : R;
  constexpr int WARPS = THREADS / 32;
  static_assert(ring_bytes<R, THREADS, DEPTH, U>() / WARPS >= sizeof(float) * GV_SPLIT_STEPS * R * NB, "partials fit the ring");
  const size_t smem = sizeof(float) * (size_t)NB * p.n + ring_bytes<R, THREADS, DEPTH, U>();
  if (smem > GV_SMEM_LIMIT) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  auto kern = gemv_stream_kernel<WT, NB, R, THREADS, GLU, DEPTH, U>;
  const int total_rows = GLU ? p.rows[0] : p.rows[0] + (p.n_mats > 1 ? p.rows[1] : 0) + (p.n_mats > 2 ? p.rows[2] : 0);
  const int total_steps = mca_ceil_div(total_rows, STEP);
  // every CTA resident at once; rows dealt evenly to groups of S warps.  The attribute and the
  // occupancy of this instantiation are looked up once per (device, shared-memory size).
  int ctas_per_sm = 1, dev = 0, sms = 148;
  MCA_CUDA_TRY(cudaGetDevice(&dev));
  {
    static std::mutex lock;
    static int c_dev = -1, c_ctas = 0, c_sms = 0;
    static size_t c_smem = 0;
    std::lock_guard<std::mutex> g(lock);
    if (c_dev != dev || c_smem != smem) {
      MCA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      MCA_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&c_ctas, kern, THREADS, smem));
      MCA_CUDA_TRY(cudaDeviceGetAttribute(&c_sms, cudaDevAttrMultiProcessorCount, dev));
      c_dev = dev; c_smem = smem;
    }
    ctas_per_sm = c_ctas; sms = c_sms;
  }
  int grid = sms * std::max(1, ctas_per_sm);
  int S = 1;
  while (S < WARPS && total_steps / (grid * WARPS / S) < 8) S *= 2;
  if (S > 1 && mca_ceil_div(total_steps, grid * WARPS / S) > GV_SPLIT_STEPS) S = 1;   // cannot happen by construction
  if (grid * (WARPS / S) > total_steps) grid = mca_ceil_div(total_steps, WARPS / S);
  p.split = S;
  return mca_launch_pdl(kern, dim3(grid), dim3(THREADS), smem, st, p, b0);
}

// More than eight sequences: one pass over the weights on the tensor cores (proj_tc.cuh).  Returns -1 when the shape
// is outside that kernel (the caller then takes the streaming passes).
template <typename WT>
int run_proj_tc(const GemvParams& p, cudaStream_t st) {
  using PL = proj::Plan<WT>;
  constexpr bool BF = !PL::CONVERT;
  if (!proj::enabled() || p.B <= 8 || p.B > proj::MAX_B || p.n > proj::MAX_N || p.n % 8 != 0) return -1;
  const int Bp = (p.B + 15) & ~15;
  proj::Params q = {};
  int tiles = 0;
  for (int m = 0; m < 3; ++m) { q.out[m] = p.out[m]; q.rows[m] = p.rows[m]; }
  if (p.swiglu) {
    tiles = mca_ceil_div(p.rows[0], proj::ROWS);
    q.tile0[0] = 0; q.tile0[1] = q.tile0[2] = q.tile0[3] = tiles;
  } else {
    for (int m = 0; m < 3; ++m) {
      q.tile0[m] = tiles;
      if (m < p.n_mats) tiles += mca_ceil_div(p.rows[m], proj::ROWS);
    }
    q.tile0[3] = tiles;
  }
  if (tiles > proj::MAX_TILES) return -1;
  int dev = 0, sms = 148;
  MCA_CUDA_TRY(cudaGetDevice(&dev));
  MCA_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  uint16_t* pieces = nullptr;
  float* xscale = nullptr;
  MCA_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&pieces), proj::g_x_pieces));
  MCA_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&xscale), proj::g_x_scale));
  q.n_mats = p.n_mats; q.B = p.B; q.Bp = Bp; q.n = p.n; q.accumulate = p.accumulate; q.swiglu = p.swiglu;
  q.tiles = tiles; q.kchunks = mca_ceil_div(p.n, proj::KC);
  q.slices = proj::pick_slices(tiles, q.kchunks, sms);
  CUtensorMap mw[3], mx;
  int e;
  for (int m = 0; m < 3; ++m) {
    const int mm = m < p.n_mats ? m : 0;
    if ((e = proj::make_map_2d(&mw[m], p.w[mm], BF ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                               (int)sizeof(WT), p.rows[mm], p.n, proj::KC, proj::ROWS,
                               BF ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE)))
      return e;
  }
  if ((e = proj::make_map_2d(&mx, pieces, BF ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                             (int64_t)PL::PIECES * Bp, p.n, proj::KC, Bp, CU_TENSOR_MAP_SWIZZLE_128B)))
    return e;
  auto pre = proj::x_pieces_kernel<BF>;
  MCA_CUDA_TRY(cudaFuncSetAttribute(pre, cudaFuncAttributeMaxDynamicSharedMemorySize, proj::MAX_N * 4));
  // both kernels are launched programmatically dependent: the pre-pass's launch overlaps the tail of whatever runs
  // before it (it waits for that before it reads or writes anything), the contraction's set-up overlaps the pre-pass
  if ((e = mca_launch_pdl(pre, dim3(Bp), dim3(256), sizeof(float) * (size_t)p.n, st, p.x, p.norm_w, p.eps, p.n, p.B, Bp, pieces, xscale)))
    return e;
  const size_t smem = proj::smem_bytes<WT>();
  auto kern = proj::proj_tc_kernel<WT>;
  MCA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int items = tiles * q.slices;
  // programmatic dependent launch: set-up and the first weight tiles overlap the pre-pass
  return mca_launch_pdl(kern, dim3(std::min(items, sms)), dim3(proj::THREADS), smem, st, mw[0], mw[1], mw[2], mx, q);
}

template <typename WT>
int run_gemv(const GemvParams& p, cudaStream_t st) {
  int e = run_proj_tc<WT>(p, st);
  if (e >= 0) return e;
  e = 0;
  const size_t xbytes = sizeof(float) * (size_t)p.n;
  auto fits = [&](int nb, size_t ring) { return nb * xbytes + ring <= GV_SMEM_LIMIT; };
  constexpr size_t RING_512 = ring_bytes<2, 512, 6>(), RING_256 = ring_bytes<2, 256, 6>();
  constexpr size_t RING_1 = ring_bytes<1, 256, 4, 4>();   // = ring_bytes<2, 256, 4, 2>(), the one- and two-sequence kernels
  if (!fits(1, RING_1)) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  const bool deep = xbytes + ring_bytes<1, 256, 6, 4>() <= 112 * 1024;   // half an SM's shared memory, less the per-CTA reserve
  for (int b0 = 0; b0 < p.B && !e;) {
    const int left = p.B - b0;
    if (p.swiglu) {
      if (left >= 8 && fits(8, RING_512)) { e = launch_pass<WT, 8, 2, 512, true, 6>(p, b0, st); b0 += 8; }
      else if (left >= 4 && fits(4, RING_512)) { e = launch_pass<WT, 4, 2, 512, true, 6>(p, b0, st); b0 += 4; }
      else if (left >= 4 && fits(4, RING_256)) { e = launch_pass<WT, 4, 2, 256, true, 6>(p, b0, st); b0 += 4; }
      else if (left >= 2 && fits(2, RING_1)) { e = launch_pass<WT, 2, 2, 256, true, 4, 2>(p, b0, st); b0 += 2; }
      else {   // a deeper ring while two CTAs per SM still fit
        e = deep ? launch_pass<WT, 1, 2, 256, true, 6, 2>(p, b0, st) : launch_pass<WT, 1, 2, 256, true, 4, 2>(p, b0, st);
        b0 += 1;
      }
    } else {
      if (left >= 8 && fits(8, RING_512)) { e = launch_pass<WT, 8, 2, 512, false, 6>(p, b0, st); b0 += 8; }
      else if (left >= 4 && fits(4, RING_512)) { e = launch_pass<WT, 4, 2, 512, false, 6>(p, b0, st); b0 += 4; }
      else if (left >= 4 && fits(4, RING_256)) { e = launch_pass<WT, 4, 2, 256, false, 6>(p, b0, st); b0 += 4; }
      else if (left >= 2 && fits(2, RING_1)) { e = launch_pass<WT, 2, 1, 256, false, 4, 4>(p, b0, st); b0 += 2; }
      else {
        e = deep ? launch_pass<WT, 1, 1, 256, false, 6, 4>(p, b0, st) : launch_pass<WT, 1, 1, 256, false, 4, 4>(p, b0, st);
        b0 += 1;
      }
    }
  }
  return e;
}

// one sequence's activations and the smallest ring fit in shared memory
bool gemv_supported(int n) { return sizeof(float) * (size_t)n + ring_bytes<1, 256, 4, 4>() <= GV_SMEM_LIMIT; }

bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int mca_decode_qkv_rmsnorm(const float* x, const float* rms_weight, float eps, const void* wq, const void* wk,
                           const void* wv, int weights_bf16, int B, int dim, int kv_dim, float* q_out, float* k_out,
                           float* v_out, void* stream) {
  if (!x || !rms_weight || !wq || !wk || !wv || !q_out || !k_out || !v_out) return ERROR_PARAM_NULL;
  if (B <= 0 || dim <= 0 || kv_dim <= 0 || dim % 8 != 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (!al16(x) || !al16(rms_weight) || !al16(wq) || !al16(wk) || !al16(wv)) return ERROR_PARAM_OUT_OF_RANGE;
  GemvParams p;
  p.swiglu = 0;
  p.x = x; p.norm_w = rms_weight; p.eps = eps; p.n = dim; p.B = B; p.accumulate = 0; p.n_mats = 3;
  p.w[0] = wq; p.w[1] = wk; p.w[2] = wv;
  p.out[0] = q_out; p.out[1] = k_out; p.out[2] = v_out;
  p.rows[0] = dim; p.rows[1] = kv_dim; p.rows[2] = kv_dim;
  return weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
}

int mca_decode_out_proj(const float* attn, const void* wo, int weights_bf16, int B, int dim, float* x_inout,
                        void* stream) {
  if (!attn || !wo || !x_inout) return ERROR_PARAM_NULL;
  if (B <= 0 || dim <= 0 || dim % 8 != 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (!al16(attn) || !al16(wo)) return ERROR_PARAM_OUT_OF_RANGE;
  GemvParams p;
  p.swiglu = 0;
  p.x = attn; p.norm_w = nullptr; p.eps = 0.f; p.n = dim; p.B = B; p.accumulate = 1; p.n_mats = 1;
  p.w[0] = wo; p.w[1] = p.w[2] = nullptr;
  p.out[0] = x_inout; p.out[1] = p.out[2] = nullptr;
  p.rows[0] = dim; p.rows[1] = p.rows[2] = 0;
  return weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
}

int mca_decode_ffn(const float* rms_weight, float eps, const void* w1, const void* w2, const void* w3, int weights_bf16,
                   int B, int dim, int hidden_dim, float* hidden_scratch, float* x_inout, void* stream) {
  if (!rms_weight || !w1 || !w2 || !w3 || !hidden_scratch || !x_inout) return ERROR_PARAM_NULL;
  if (B <= 0 || dim <= 0 || hidden_dim <= 0 || dim % 8 != 0 || hidden_dim % 8 != 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (!al16(x_inout) || !al16(rms_weight) || !al16(w1) || !al16(w2) || !al16(w3) || !al16(hidden_scratch))
    return ERROR_PARAM_OUT_OF_RANGE;
  if (!gemv_supported(hidden_dim) || !gemv_supported(dim)) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  GemvParams p;
  // h = silu(W1 xn) * (W3 xn)
  p.swiglu = 1;
  p.x = x_inout; p.norm_w = rms_weight; p.eps = eps; p.n = dim; p.B = B; p.accumulate = 0; p.n_mats = 2;
  p.w[0] = w1; p.w[1] = w3; p.w[2] = nullptr;
  p.out[0] = hidden_scratch; p.out[1] = p.out[2] = nullptr;
  p.rows[0] = hidden_dim; p.rows[1] = hidden_dim; p.rows[2] = 0;
  int e = weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
  if (e) return e;
  // x += W2 h
  p.swiglu = 0;
  p.x = hidden_scratch; p.norm_w = nullptr; p.eps = 0.f; p.n = hidden_dim; p.accumulate = 1; p.n_mats = 1;
  p.w[0] = w2; p.w[1] = nullptr;
  p.out[0] = x_inout;
  p.rows[0] = dim; p.rows[1] = 0;
  return weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
}

int mca_decode_logits(const float* x, const float* rms_weight, float eps, const void* wcls, int weights_bf16, int B,
                      int dim, int vocab_size, float* logits, void* stream) {
  if (!x || !rms_weight || !wcls || !logits) return ERROR_PARAM_NULL;
  if (B <= 0 || dim <= 0 || vocab_size <= 0 || dim % 8 != 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (!al16(x) || !al16(rms_weight) || !al16(wcls)) return ERROR_PARAM_OUT_OF_RANGE;
  GemvParams p;
  p.swiglu = 0;
  p.x = x; p.norm_w = rms_weight; p.eps = eps; p.n = dim; p.B = B; p.accumulate = 0; p.n_mats = 1;
  p.w[0] = wcls; p.w[1] = p.w[2] = nullptr;
  p.out[0] = logits; p.out[1] = p.out[2] = nullptr;
  p.rows[0] = vocab_size; p.rows[1] = p.rows[2] = 0;
  return weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
}

int mca_proj_tc_enable(int on) {
  const int was = proj::enabled() ? 1 : 0;
  proj::enabled() = on != 0;
  return was;
}

int mca_proj_tc_status(int* status4) {
  if (!status4) return ERROR_PARAM_NULL;
  void* sp = nullptr;
  MCA_CUDA_TRY(cudaGetSymbolAddress(&sp, proj::g_status));
  MCA_CUDA_TRY(cudaMemcpy(status4, sp, 4 * sizeof(int), cudaMemcpyDeviceToHost));
  if (status4[0] != 0) {   // a bounded wait gave up: the tickets of that launch may be left half-counted
    void* tp = nullptr;
    MCA_CUDA_TRY(cudaGetSymbolAddress(&tp, proj::g_tickets));
    MCA_CUDA_TRY(cudaMemset(tp, 0, sizeof(unsigned int) * proj::MAX_TILES * proj::EPI_WARPS));
    MCA_CUDA_TRY(cudaMemset(sp, 0, 4 * sizeof(int)));
  }
  return 0;
}

// Interpretable multi-head attention of the Temporal Fusion Transformer: per-head Q/K, one V
// shared by all heads, and the head-means of both the probabilities and the outputs.
//
// Replaces the attention block of MultiHeadAttentionInterpLayer<T>.forward
// (MyCaffe.layers.tft/layers.tft/MultiHeadAttentionInterpLayer.cs:728-759), which the
// reference runs as ~30 launches: V tiled H times in memory (:706-710), K transposed, two
// batched matmuls, scale, mask_batch, softmax and two per-head channel_copy+add loops for the
// means (:244-264).  Because V is shared, mean_h(P_h V) = (mean_h P_h) V, so one CTA computes
// the mean probabilities for a few query rows and multiplies V once.  The problem is tiny
// (tens of MB): the kernel is launch/latency bound, not roofline bound.
#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int TFT_ROWS = 8;        // query rows per CTA, one per warp
constexpr int TFT_THREADS = 256;

// (Nk, d) tile -> shared memory rows of d + 4 floats with asynchronous 16-byte copies: all of a thread's copies are
// in flight at once (a load-then-store loop serialises on the round trip of each one).
__device__ __forceinline__ void tile_to_smem_async(float* dst, const float* __restrict__ src, int Nk, int d, int tid) {
  const int d4 = d / 4, ld = d + 4;
  for (int idx = tid; idx < Nk * d4; idx += TFT_THREADS) {
    const int j = idx / d4, c4 = idx - j * d4;
    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(dst + (size_t)j * ld + c4 * 4);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(src + (size_t)idx * 4) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tile_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// smem: KV[Nk][d+4] | Qs[H][8][d] | pm[8][Nk] | ps[8][Nk]
__global__ void __launch_bounds__(TFT_THREADS) tft_fwd_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                              const float* __restrict__ V,
                                                              const float* __restrict__ mask, int H, int Nq, int Nk,
                                                              int d, float scale, float* __restrict__ out,
                                                              float* __restrict__ attn) {
  extern __shared__ __align__(16) float smem[];
  const int ld = d + 4;
  float* KV = smem;
  float* Qs = KV + (size_t)Nk * ld;
  float* pm = Qs + (size_t)H * TFT_ROWS * d;
  float* ps = pm + (size_t)TFT_ROWS * Nk;
  const int b = blockIdx.y, q0 = blockIdx.x * TFT_ROWS;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int i = q0 + w;
  const bool row_ok = i < Nq;
  const int d4 = d / 4;

  for (int idx = tid; idx < H * TFT_ROWS * d; idx += TFT_THREADS) {
    const int h = idx / (TFT_ROWS * d), r = (idx / d) % TFT_ROWS, c = idx % d;
    Qs[idx] = (q0 + r < Nq) ? Q[(((int64_t)b * H + h) * Nq + q0 + r) * d + c] : 0.f;
  }
  for (int idx = tid; idx < TFT_ROWS * Nk; idx += TFT_THREADS) pm[idx] = 0.f;

  for (int h = 0; h < H; ++h) {
    __syncthreads();  // previous head's readers of KV are done; Qs/pm initialised
    tile_to_smem_async(KV, K + ((int64_t)b * H + h) * Nk * d, Nk, d, tid);
    tile_wait();
    __syncthreads();
    const float* qrow = Qs + ((size_t)h * TFT_ROWS + w) * d;
    float mx = -INFINITY;
    for (int j = lane; j < Nk; j += 32) {
      const float* krow = KV + (size_t)j * ld;
      float acc = 0.f;
      for (int c = 0; c < d; c += 4) {
        const float4 kq = *reinterpret_cast<const float4*>(krow + c);
        const float4 qq = *reinterpret_cast<const float4*>(qrow + c);
        acc = fmaf(qq.x, kq.x, acc); acc = fmaf(qq.y, kq.y, acc);
        acc = fmaf(qq.z, kq.z, acc); acc = fmaf(qq.w, kq.w, acc);
      }
      acc *= scale;
      // mask_batch(..., search = 1, replace = -1e29), MultiHeadAttentionInterpLayer.cs:743
      if (mask != nullptr && row_ok && __ldg(mask + (int64_t)i * Nk + j) == 1.0f) acc = MCA_MASKED_LOGIT;
      ps[w * Nk + j] = acc;
      mx = fmaxf(mx, acc);
    }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int j = lane; j < Nk; j += 32) {
      const float e = expf(ps[w * Nk + j] - mx);
      ps[w * Nk + j] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int j = lane; j < Nk; j += 32) pm[w * Nk + j] += ps[w * Nk + j] * inv;  // running head sum (:255-260)
  }
  __syncthreads();
  tile_to_smem_async(KV, V + (int64_t)b * Nk * d, Nk, d, tid);
  const float inv_h = 1.f / (float)H;
  for (int j = lane; j < Nk; j += 32) pm[w * Nk + j] *= inv_h;  // one scale by 1/H (:263)
  tile_wait();
  __syncthreads();
  if (!row_ok) return;
  for (int j = lane; j < Nk; j += 32) attn[((int64_t)b * Nq + i) * Nk + j] = pm[w * Nk + j];
  for (int c = lane; c < d; c += 32) {
    float acc = 0.f;
    for (int j = 0; j < Nk; ++j) acc = fmaf(pm[w * Nk + j], KV[(size_t)j * ld + c], acc);
    out[((int64_t)b * Nq + i) * d + c] = acc;
  }
}

// Backward of the block above (MultiHeadAttentionInterpLayer<T>.backward,
// MultiHeadAttentionInterpLayer.cs:780-859: the two head-mean backward loops, matmul grads,
// softmax backward, scale, and the sum of the per-head V gradients into the shared V).
// One CTA per batch element walks the heads; K_h, V and the dK_h / dV accumulators live in shared
// memory (every thread owns fixed accumulator elements, so there are no atomics); eight query
// rows are processed per step, one per warp, with the probabilities recomputed.
// smem: Ks[Nk][d+4] | Vs[Nk][d+4] | dKs[Nk][d] | dVs[Nk][d] | ps[8][Nk] | dss[8][Nk] | qs[8][d] | gos[8][d]
__global__ void __launch_bounds__(TFT_THREADS) tft_bwd_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                              const float* __restrict__ V,
                                                              const float* __restrict__ mask,
                                                              const float* __restrict__ d_out,
                                                              const float* __restrict__ d_attn, int H, int Nq, int Nk,
                                                              int d, float scale, float* __restrict__ dQ,
                                                              float* __restrict__ dK, float* __restrict__ dV) {
  extern __shared__ __align__(16) float smem[];
  const int ld = d + 4;
  float* Ks = smem;
  float* Vs = Ks + (size_t)Nk * ld;
  float* dKs = Vs + (size_t)Nk * ld;
  float* dVs = dKs + (size_t)Nk * d;
  float* ps = dVs + (size_t)Nk * d;
  float* dss = ps + (size_t)TFT_ROWS * Nk;
  float* qs = dss + (size_t)TFT_ROWS * Nk;
  float* gos = qs + (size_t)TFT_ROWS * d;
  const int b = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int d4 = d / 4;
  const float inv_h = 1.f / (float)H;

  tile_to_smem_async(Vs, V + (int64_t)b * Nk * d, Nk, d, tid);
  for (int idx = tid; idx < Nk * d; idx += TFT_THREADS) dVs[idx] = 0.f;

  for (int h = 0; h < H; ++h) {
    __syncthreads();  // previous head's dKs written out, Ks readers done
    tile_to_smem_async(Ks, K + ((int64_t)b * H + h) * Nk * d, Nk, d, tid);
    for (int idx = tid; idx < Nk * d; idx += TFT_THREADS) dKs[idx] = 0.f;
    tile_wait();   // also covers the V tile requested before the loop
    for (int q0 = 0; q0 < Nq; q0 += TFT_ROWS) {
      __syncthreads();  // K tile loaded / previous step's accumulation done
      const int i = q0 + w;
      const bool row_ok = i < Nq;
      // this warp's query row and its output gradient (already divided by the number of heads)
      for (int c = lane; c < d; c += 32) {
        qs[w * d + c] = row_ok ? Q[(((int64_t)b * H + h) * Nq + i) * d + c] : 0.f;
        gos[w * d + c] = row_ok ? d_out[((int64_t)b * Nq + i) * d + c] * inv_h : 0.f;
      }
      __syncwarp();
      float mx = -INFINITY;
      for (int j = lane; j < Nk; j += 32) {
        const float* krow = Ks + (size_t)j * ld;
        const float* vrow = Vs + (size_t)j * ld;
        float acc = 0.f, dp = 0.f;
        for (int c = 0; c < d; c += 4) {
          const float4 kq = *reinterpret_cast<const float4*>(krow + c);
          const float4 vq = *reinterpret_cast<const float4*>(vrow + c);
          const float4 qq = *reinterpret_cast<const float4*>(qs + w * d + c);
          const float4 gq = *reinterpret_cast<const float4*>(gos + w * d + c);
          acc = fmaf(qq.x, kq.x, acc); acc = fmaf(qq.y, kq.y, acc); acc = fmaf(qq.z, kq.z, acc); acc = fmaf(qq.w, kq.w, acc);
          dp = fmaf(gq.x, vq.x, dp); dp = fmaf(gq.y, vq.y, dp); dp = fmaf(gq.z, vq.z, dp); dp = fmaf(gq.w, vq.w, dp);
        }
        acc *= scale;
        if (mask != nullptr && row_ok && __ldg(mask + (int64_t)i * Nk + j) == 1.0f) acc = MCA_MASKED_LOGIT;
        if (d_attn != nullptr && row_ok) dp += __ldg(d_attn + ((int64_t)b * Nq + i) * Nk + j) * inv_h;
        ps[w * Nk + j] = acc;
        dss[w * Nk + j] = dp;
        mx = fmaxf(mx, acc);
      }
      mx = warp_max(mx);
      float sum = 0.f;
      for (int j = lane; j < Nk; j += 32) {
        const float e = expf(ps[w * Nk + j] - mx);
        ps[w * Nk + j] = e;
        sum += e;
      }
      sum = warp_sum(sum);
      const float inv = row_ok ? 1.f / sum : 0.f;
      float dot = 0.f;
      for (int j = lane; j < Nk; j += 32) {
        const float pj = ps[w * Nk + j] * inv;
        ps[w * Nk + j] = pj;
        dot = fmaf(pj, dss[w * Nk + j], dot);
      }
      dot = warp_sum(dot);
      for (int j = lane; j < Nk; j += 32) dss[w * Nk + j] = ps[w * Nk + j] * (dss[w * Nk + j] - dot) * scale;
      __syncwarp();
      if (row_ok) {
        for (int c = lane; c < d; c += 32) {
          float acc = 0.f;
          for (int j = 0; j < Nk; ++j) acc = fmaf(dss[w * Nk + j], Ks[(size_t)j * ld + c], acc);
          dQ[(((int64_t)b * H + h) * Nq + i) * d + c] = acc;
        }
      }
      __syncthreads();
      // accumulate dK_h += dS^T Q_h and dV += P^T dO over the eight rows of this step
      for (int idx = tid; idx < Nk * d; idx += TFT_THREADS) {
        const int j = idx / d, c = idx % d;
        float ak = dKs[idx], av = dVs[idx];
#pragma unroll
        for (int r = 0; r < TFT_ROWS; ++r) {
          ak = fmaf(dss[r * Nk + j], qs[r * d + c], ak);
          av = fmaf(ps[r * Nk + j], gos[r * d + c], av);
        }
        dKs[idx] = ak;
        dVs[idx] = av;
      }
    }
    __syncthreads();
    float* dKg = dK + ((int64_t)b * H + h) * Nk * d;
    for (int idx = tid; idx < Nk * d; idx += TFT_THREADS) dKg[idx] = dKs[idx];
  }
  __syncthreads();
  float* dVg = dV + (int64_t)b * Nk * d;
  for (int idx = tid; idx < Nk * d; idx += TFT_THREADS) dVg[idx] = dVs[idx];
}

}  // namespace

int mca_tft_attention_backward_f32(const float* q, const float* k, const float* v, const float* mask,
                                   const float* d_out, const float* d_attn, int B, int H, int Nq, int Nk, int d,
                                   float* dq, float* dk, float* dv, void* stream) {
  if (!q || !k || !v || !d_out || !dq || !dk || !dv) return ERROR_PARAM_NULL;
  if (B <= 0 || H <= 0 || Nq <= 0 || Nk <= 0 || d <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (d % 4 != 0 || (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15))
    return ERROR_ATTN_UNSUPPORTED_SHAPE;
  const size_t smem = sizeof(float) * (2 * (size_t)Nk * (d + 4) + 2 * (size_t)Nk * d + 2 * (size_t)TFT_ROWS * Nk +
                                       2 * (size_t)TFT_ROWS * d);
  if (smem > 227 * 1024) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  MCA_CUDA_TRY(cudaFuncSetAttribute(tft_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  tft_bwd_kernel<<<B, TFT_THREADS, smem, (cudaStream_t)stream>>>(q, k, v, mask, d_out, d_attn, H, Nq, Nk, d,
                                                                  1.0f / sqrtf((float)d), dq, dk, dv);
  return mca_launch_status();
}

int mca_tft_attention_forward_f32(const float* q, const float* k, const float* v, const float* mask, int B, int H,
                                  int Nq, int Nk, int d, float* out, float* attn, void* stream) {
  if (!q || !k || !v || !out || !attn) return ERROR_PARAM_NULL;
  if (B <= 0 || H <= 0 || Nq <= 0 || Nk <= 0 || d <= 0 || B > 65535) return ERROR_PARAM_OUT_OF_RANGE;
  if (d % 4 != 0 || (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15))
    return ERROR_ATTN_UNSUPPORTED_SHAPE;
  const size_t smem = sizeof(float) * ((size_t)Nk * (d + 4) + (size_t)H * TFT_ROWS * d + 2 * (size_t)TFT_ROWS * Nk);
  if (smem > 227 * 1024) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  MCA_CUDA_TRY(cudaFuncSetAttribute(tft_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(mca_ceil_div(Nq, TFT_ROWS), B);
  tft_fwd_kernel<<<grid, TFT_THREADS, smem, (cudaStream_t)stream>>>(q, k, v, mask, H, Nq, Nk, d,
                                                                    1.0f / sqrtf((float)d), out, attn);
  return mca_launch_status();
}

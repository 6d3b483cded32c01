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
constexpr int TFT_TQ_ROWS = 24;   // query rows of a tile of the tiled kernels

// e^x for x <= 0 as one multiply and one ex2.approx (2 ulp): the softmax of the tiled kernels.  Arguments far below
// the fp32 range (a masked logit against a real maximum) give exactly 0.
__device__ __forceinline__ float tft_exp(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}

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


// ---------------------------------------------------------------------------------------------
// Forward, tiled form (the shapes the TFT network runs: d in {16, 32, 64}, Nk <= 192).
//
// One CTA = one batch item x 24 query rows, all heads.  The K tiles of the heads and then V (Nk x d each) stream through
// two shared-memory buffers filled by asynchronous copies, two tiles ahead of the arithmetic.  The scores of the 24 rows
// are computed in 6-row x 3-key register tiles (warps 0-3 take the rows six at a time over keys [0,96), warps 4-7 over
// [96,192)): per four values of the head dimension a warp issues 6 broadcast reads of Q and 3 conflict-free reads of K
// for 72 FMAs, which balances the shared-memory pipe against the FMA pipes (one row per warp, as the generic kernel
// below does it, is bound by shared memory four times over).  The softmax stays in that register layout: a row's two
// half-maxima and half-sums cross between the two warps that share it through 2 x 24 floats of shared memory, and the
// sum over the heads of the probabilities is 18 registers per thread.  Because V is shared by the heads the output is
// (mean_h P_h) V, one product at the end.  Two CTAs fit an SM.
// smem: Kt[2][Nk][d] (16-byte pieces swizzled by row) | Qs[2][24][d] | ex[2][2][24]
// ---------------------------------------------------------------------------------------------
constexpr int TQ = TFT_TQ_ROWS;    // query rows per CTA
constexpr int TQ_R = 6;            // rows of a register tile
constexpr int TQ_C = 3;            // keys per lane of a register tile (32 lanes: 96 keys per warp)
constexpr int TQ_KEYS = 2 * 32 * TQ_C;   // keys a CTA covers: 192

// (Nk, D) tile -> shared memory rows of exactly D floats; the 16-byte pieces of row j are stored at piece ^ (j & SW), so
// that lanes reading the same piece of consecutive rows hit different banks without padding the rows.
template <int D>
__device__ __forceinline__ void tile_rows_async_swz(float* dst, const float* __restrict__ src, int Nk, int tid) {
  constexpr int D4 = D / 4, SW = D4 >= 8 ? 7 : D4 - 1;
  for (int idx = tid; idx < Nk * D4; idx += TFT_THREADS) {
    const int j = idx / D4, c4 = idx - j * D4;
    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(dst + (size_t)j * D + ((c4 ^ (j & SW)) << 2));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(src + (size_t)idx * 4) : "memory");
  }
}

template <int D>
__device__ __forceinline__ void tile_to_smem_async_swz(float* dst, const float* __restrict__ src, int Nk, int tid) {
  tile_rows_async_swz<D>(dst, src, Nk, tid);
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// (24, D) block of consecutive rows -> shared memory, rows beyond `rows` zero-filled (copies with source size 0)
template <int D>
__device__ __forceinline__ void rows24_async(float* dst, const float* __restrict__ src, int rows, int tid) {
  for (int idx = tid; idx < TFT_TQ_ROWS * (D / 4); idx += TFT_THREADS) {
    const int r = idx / (D / 4);
    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(dst + idx * 4);
    const int nbytes = r < rows ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sa), "l"(src + (r < rows ? idx * 4 : 0)), "r"(nbytes) : "memory");
  }
}

__device__ __forceinline__ void cp_async_wait_all_but(int n) {
  if (n == 0) asm volatile("cp.async.wait_group 0;" ::: "memory");
  else asm volatile("cp.async.wait_group 1;" ::: "memory");
}

template <int D>
__global__ void __launch_bounds__(TFT_THREADS, 2) tft_fwd_tiled_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                                       const float* __restrict__ V,
                                                                       const float* __restrict__ mask, int H, int Nq, int Nk,
                                                                       float scale, float* __restrict__ out,
                                                                       float* __restrict__ attn) {
  extern __shared__ __align__(16) float smem[];
  constexpr int SW = D / 4 >= 8 ? 7 : D / 4 - 1;     // swizzle of the 16-byte pieces of a tile row
  const size_t tile = (size_t)Nk * D;
  float* Kt = smem;                                  // two tiles
  float* Qs = Kt + 2 * tile;                         // two (24, D) blocks
  float* ex = Qs + 2 * TQ * D;                       // [2 (max | sum)][2 key halves][24 rows]
  const int b = blockIdx.y, q0 = blockIdx.x * TQ;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int rows = min(TQ, Nq - q0);

  // tile t: K of head t (with that head's 24 query rows) or, for t == H, V; one commit group per call.  Query rows
  // beyond Nq are zero-filled (a copy with source size 0).
  auto load_tile = [&](int t) {
    if (t > H) return;
    if (t < H) {
      const float* src = Q + (((int64_t)b * H + t) * Nq + q0) * D;
      float* dst = Qs + (t & 1) * TQ * D;
      for (int idx = tid; idx < TQ * (D / 4); idx += TFT_THREADS) {
        const int r = idx / (D / 4);
        const uint32_t sa = (uint32_t)__cvta_generic_to_shared(dst + idx * 4);
        const int nbytes = r < rows ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sa), "l"(src + (r < rows ? idx * 4 : 0)), "r"(nbytes) : "memory");
      }
    }
    tile_to_smem_async_swz<D>(Kt + (t & 1) * tile, t < H ? K + ((int64_t)b * H + t) * Nk * D : V + (int64_t)b * Nk * D, Nk, tid);
  };
  load_tile(0);
  load_tile(1);

  const float inv_h = 1.f / (float)H;
  const int rg = w & 3;                 // this warp's six rows: rg*6 .. rg*6+5
  const int khalf = w >> 2;             // its half of the keys: khalf*96 + lane + 32c
  // The mask is the same for every head (and batch item): this thread's entries are kept as bits, bit r*3+c = row
  // rg*6+r, key khalf*96 + lane + 32c is masked (mask_batch(..., search = 1, replace = -1e29),
  // MultiHeadAttentionInterpLayer.cs:743).  Keys beyond Nk are marked in `dead` and never contribute.
  unsigned mbits = 0, dead = 0;
  {
    float mv[TQ_R][TQ_C];               // all eighteen loads first (clamped addresses), then the tests
#pragma unroll
    for (int r = 0; r < TQ_R; ++r)
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) {
        const int i = min(rg * TQ_R + r, rows - 1), j = min(khalf * (32 * TQ_C) + lane + 32 * c, Nk - 1);
        mv[r][c] = mask != nullptr ? __ldg(mask + (int64_t)(q0 + i) * Nk + j) : 0.f;
      }
#pragma unroll
    for (int r = 0; r < TQ_R; ++r)
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) {
        const int i = rg * TQ_R + r, j = khalf * (32 * TQ_C) + lane + 32 * c;
        if (j >= Nk) dead |= 1u << (r * TQ_C + c);
        else if (i < rows && mv[r][c] == 1.0f) mbits |= 1u << (r * TQ_C + c);
      }
  }
  float pmr[TQ_R][TQ_C];                // sum over the heads of this thread's probabilities
#pragma unroll
  for (int r = 0; r < TQ_R; ++r)
#pragma unroll
    for (int c = 0; c < TQ_C; ++c) pmr[r][c] = 0.f;

  for (int h = 0; h < H; ++h) {
    cp_async_wait_all_but(h + 1 <= H ? 1 : 0);   // tile h has landed (tile h+1 may still be in flight)
    __syncthreads();                    // K_h and Q_h visible to all; everyone is past the previous head
    const float* Kh = Kt + (h & 1) * tile;
    float acc[TQ_R][TQ_C];
#pragma unroll
    for (int r = 0; r < TQ_R; ++r)
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) acc[r][c] = 0.f;
    const float* krow[TQ_C];
    int ksw[TQ_C];
#pragma unroll
    for (int c = 0; c < TQ_C; ++c) {
      const int j = min(khalf * (32 * TQ_C) + lane + 32 * c, Nk - 1);
      krow[c] = Kh + (size_t)j * D;
      ksw[c] = j & SW;
    }
    const float* qrow = Qs + (h & 1) * TQ * D + rg * TQ_R * D;
#pragma unroll
    for (int i = 0; i < D / 4; ++i) {
      float4 kv[TQ_C], qv[TQ_R];
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) kv[c] = *reinterpret_cast<const float4*>(krow[c] + ((i ^ ksw[c]) << 2));
#pragma unroll
      for (int r = 0; r < TQ_R; ++r) qv[r] = *reinterpret_cast<const float4*>(qrow + r * D + 4 * i);
      // component-major order: eighteen independent FMAs stand between two that depend on each other
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) acc[r][c] = fmaf(qv[r].x, kv[c].x, acc[r][c]);
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) acc[r][c] = fmaf(qv[r].y, kv[c].y, acc[r][c]);
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) acc[r][c] = fmaf(qv[r].z, kv[c].z, acc[r][c]);
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) acc[r][c] = fmaf(qv[r].w, kv[c].w, acc[r][c]);
    }
    // scale, mask, and this warp's half of every row maximum
    float hm[TQ_R];
#pragma unroll
    for (int r = 0; r < TQ_R; ++r) {
      float m = -INFINITY;
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) {
        const unsigned bit = 1u << (r * TQ_C + c);
        acc[r][c] = (mbits & bit) ? MCA_MASKED_LOGIT : acc[r][c] * scale;
        if (!(dead & bit)) m = fmaxf(m, acc[r][c]);
      }
      hm[r] = warp_max(m);
    }
    if (lane < TQ_R) {
      float v = hm[0];
#pragma unroll
      for (int r = 1; r < TQ_R; ++r) v = lane == r ? hm[r] : v;
      ex[khalf * TQ + rg * TQ_R + lane] = v;
    }
    __syncthreads();                    // half-maxima exchanged; every reader of K_h is done
    load_tile(h + 2);                   // into the buffers K_h and Q_h occupied
    if (h + 2 > H) asm volatile("cp.async.commit_group;" ::: "memory");   // keep one group per iteration
    float hs[TQ_R];
#pragma unroll
    for (int r = 0; r < TQ_R; ++r) {
      const float m = fmaxf(ex[rg * TQ_R + r], ex[TQ + rg * TQ_R + r]);
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) {
        acc[r][c] = (dead & (1u << (r * TQ_C + c))) ? 0.f : tft_exp(acc[r][c] - m);
        sum += acc[r][c];
      }
      hs[r] = warp_sum(sum);
    }
    if (lane < TQ_R) {
      float v = hs[0];
#pragma unroll
      for (int r = 1; r < TQ_R; ++r) v = lane == r ? hs[r] : v;
      ex[2 * TQ + khalf * TQ + rg * TQ_R + lane] = v;
    }
    __syncthreads();                    // half-sums exchanged
#pragma unroll
    for (int r = 0; r < TQ_R; ++r) {
      const float inv = inv_h / (ex[2 * TQ + rg * TQ_R + r] + ex[3 * TQ + rg * TQ_R + r]);   // the 1/H of the head mean (:263) goes in here
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) pmr[r][c] = fmaf(acc[r][c], inv, pmr[r][c]);   // running head sum (:255-260)
    }
  }
  // mean probabilities: to global memory from the registers, and into the free K buffer for the product with V
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  float* pm = Kt + ((H + 1) & 1) * tile;                  // V is tile H, in buffer H & 1
#pragma unroll
  for (int r = 0; r < TQ_R; ++r)
#pragma unroll
    for (int c = 0; c < TQ_C; ++c) {
      const int i = rg * TQ_R + r, j = khalf * (32 * TQ_C) + lane + 32 * c;
      if (j < Nk) {
        pm[i * Nk + j] = pmr[r][c];
        if (i < rows) attn[((int64_t)b * Nq + q0 + i) * Nk + j] = pmr[r][c];
      }
    }
  __syncthreads();                      // V in place, pm complete
  const float* Vt = Kt + (H & 1) * tile;
  // out = pm V.  A thread owns four columns of six rows (rq, rq + 4, ...) over a slice of the keys: per key one
  // 16-byte read of V and six (broadcast) reads of pm feed 24 FMAs.  The slices' partial sums meet in shared memory
  // behind pm (the buffer holds Nk x D floats, pm takes 24 x Nk of them).
  constexpr int C4 = D / 4;                               // column groups
  constexpr int SLOTS = TFT_THREADS / (C4 * 4);           // key slices (4 at D = 64)
  const int c4 = tid % C4, rq = (tid / C4) & 3, ks = tid / (C4 * 4);
  const int per = (Nk + SLOTS - 1) / SLOTS;
  const int j0 = ks * per, j1 = min(Nk, j0 + per);
  float o[TQ / 4][4];
#pragma unroll
  for (int r = 0; r < TQ / 4; ++r) { o[r][0] = o[r][1] = o[r][2] = o[r][3] = 0.f; }
  for (int j = j0; j < j1; ++j) {
    const float4 vv = *reinterpret_cast<const float4*>(Vt + (size_t)j * D + ((c4 ^ (j & SW)) << 2));
#pragma unroll
    for (int r = 0; r < TQ / 4; ++r) {
      const float pj = pm[(rq + 4 * r) * Nk + j];
      o[r][0] = fmaf(pj, vv.x, o[r][0]); o[r][1] = fmaf(pj, vv.y, o[r][1]);
      o[r][2] = fmaf(pj, vv.z, o[r][2]); o[r][3] = fmaf(pj, vv.w, o[r][3]);
    }
  }
  float* part = pm + (size_t)TQ * Nk;                     // (SLOTS - 1) x 24 x D floats (the launcher checks the room)
  if (ks > 0) {
#pragma unroll
    for (int r = 0; r < TQ / 4; ++r)
      *reinterpret_cast<float4*>(part + (size_t)(ks - 1) * TQ * D + (rq + 4 * r) * D + c4 * 4) = make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
  }
  __syncthreads();
  if (ks == 0) {
#pragma unroll
    for (int r = 0; r < TQ / 4; ++r) {
      const int i = rq + 4 * r;
      float4 acc4 = make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
      for (int s2 = 0; s2 < SLOTS - 1; ++s2) {
        const float4 t = *reinterpret_cast<const float4*>(part + (size_t)s2 * TQ * D + i * D + c4 * 4);
        acc4.x += t.x; acc4.y += t.y; acc4.z += t.z; acc4.w += t.w;
      }
      if (i < rows) *reinterpret_cast<float4*>(out + ((int64_t)b * Nq + q0 + i) * D + c4 * 4) = acc4;
    }
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

// ---------------------------------------------------------------------------------------------
// Backward, tiled form (the shapes of the tiled forward: d in {16, 32, 64}, Nk <= 192).
//
// One CTA = one batch item; it walks the 24-row tiles of the queries and, inside a tile, the heads.  V stays in shared
// memory; K_h, the 24 rows of Q_h and of the output gradient are double-buffered (the next iteration's arrive while
// this one is worked on).  Per (tile, head):
//   A  S = Q K^T in the forward's 6 x 3 register tiles; for the tile's first head the same loop also forms
//      dP = dO V^T, which does not depend on the head and stays in registers for the others;
//   B  mask, softmax and its backward in that layout: the row maximum, then the row sum together with sum_j P dP,
//      cross the two warps that share a row through shared memory; dS = P (dP - sum) scale goes to shared memory and P
//      is added to the running sum over the heads (18 registers);
//   C  this tile's part of dK_h = dS^T Q_h: a thread owns 3 keys x d/4 columns in registers (the contraction runs over
//      the 24 rows); it is written for the first tile and added in global memory for the later ones -- one CTA, a
//      fixed order, no atomics;
//   D  dQ = dS K_h: a thread owns a few rows x 4 columns over a slice of the keys, four keys per step (one 16-byte read
//      of dS per row, four of K); the slices' partial sums meet in shared memory;
//   after the tile's last head, dV (+)= (sum_h P_h)^T dO / H, one product for all heads.
// The 1/H of the head mean is applied to dP once and to dV.
// smem: Vt[nk4][d] | Kt[2][nk4][d] (16-byte pieces swizzled by row; nk4 = Nk rounded up to 4, rows beyond Nk zero) |
//       Qs[2][24][d] | Gs[2][24][d] | Ps[24][192] | Ss[24][192] | ex[6][24]
// ---------------------------------------------------------------------------------------------
template <int D, bool WITH_DP>
__device__ __forceinline__ void tft_bwd_scores(const float* const (&krow)[TQ_C], const float* const (&vrow)[TQ_C],
                                               const int (&ksw)[TQ_C], const float* __restrict__ qrow,
                                               const float* __restrict__ grow, float (&s)[TQ_R][TQ_C],
                                               float (&dp)[TQ_R][TQ_C]) {
#pragma unroll 4
  for (int i = 0; i < D / 4; ++i) {
    float4 kv[TQ_C], qv[TQ_R];
#pragma unroll
    for (int c = 0; c < TQ_C; ++c) kv[c] = *reinterpret_cast<const float4*>(krow[c] + ((i ^ ksw[c]) << 2));
#pragma unroll
    for (int r = 0; r < TQ_R; ++r) qv[r] = *reinterpret_cast<const float4*>(qrow + r * D + 4 * i);
#pragma unroll
    for (int r = 0; r < TQ_R; ++r)
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) s[r][c] = fmaf(qv[r].x, kv[c].x, s[r][c]);
#pragma unroll
    for (int r = 0; r < TQ_R; ++r)
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) s[r][c] = fmaf(qv[r].y, kv[c].y, s[r][c]);
#pragma unroll
    for (int r = 0; r < TQ_R; ++r)
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) s[r][c] = fmaf(qv[r].z, kv[c].z, s[r][c]);
#pragma unroll
    for (int r = 0; r < TQ_R; ++r)
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) s[r][c] = fmaf(qv[r].w, kv[c].w, s[r][c]);
    if (WITH_DP) {
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) kv[c] = *reinterpret_cast<const float4*>(vrow[c] + ((i ^ ksw[c]) << 2));
#pragma unroll
      for (int r = 0; r < TQ_R; ++r) qv[r] = *reinterpret_cast<const float4*>(grow + r * D + 4 * i);
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) dp[r][c] = fmaf(qv[r].x, kv[c].x, dp[r][c]);
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) dp[r][c] = fmaf(qv[r].y, kv[c].y, dp[r][c]);
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) dp[r][c] = fmaf(qv[r].z, kv[c].z, dp[r][c]);
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) dp[r][c] = fmaf(qv[r].w, kv[c].w, dp[r][c]);
    }
  }
}

template <int D>
__global__ void __launch_bounds__(TFT_THREADS, 1) tft_bwd_tiled_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                                       const float* __restrict__ V,
                                                                       const float* __restrict__ mask,
                                                                       const float* __restrict__ d_out,
                                                                       const float* __restrict__ d_attn, int H, int Nq, int Nk,
                                                                       float scale, float* __restrict__ dQ,
                                                                       float* __restrict__ dK, float* __restrict__ dV) {
  extern __shared__ __align__(16) float smem[];
  constexpr int D4 = D / 4, SW = D4 >= 8 ? 7 : D4 - 1;
  constexpr int NV = D / 16;                          // 16-byte column pieces of a thread's dK / dV tile
  constexpr int RPT = D == 64 ? 6 : 3;                // phase D: rows per thread,
  constexpr int RQ = TQ / RPT;                        //   row classes (a thread's rows are rq, rq + RQ, ...)
  constexpr int SLOTS = TFT_THREADS / (D4 * RQ);      //   key slices
  static_assert((SLOTS - 1) * TQ * D <= TQ * TQ_KEYS, "the partial sums of dQ must fit the buffer of P");
  const int nk4 = (Nk + 3) & ~3;
  const size_t tile = (size_t)nk4 * D;
  float* Vt = smem;
  float* Kt = Vt + tile;                              // two tiles
  float* Qs = Kt + 2 * tile;                          // two (24, D) blocks
  float* Gs = Qs + 2 * TQ * D;                        // two (24, D) blocks of the output gradient
  float* Ps = Gs + 2 * TQ * D;                        // (24, 192) probabilities; later the partial sums of dQ
  float* Ss = Ps + TQ * TQ_KEYS;                      // (24, 192) dS
  float* ex = Ss + TQ * TQ_KEYS;                      // [max | sum | dot][2 key halves][24 rows]
  const int b = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int tiles = (Nq + TQ - 1) / TQ, iters = H * tiles;
  const float inv_h = 1.f / (float)H;

  // what iteration `it` = (row tile, head) reads; one commit group per call, empty beyond the last iteration
  auto load_iter = [&](int it) {
    if (it < iters) {
      const int t = it / H, h = it - t * H, q0 = t * TQ, rows = min(TQ, Nq - q0);
      rows24_async<D>(Qs + (it & 1) * TQ * D, Q + (((int64_t)b * H + h) * Nq + q0) * D, rows, tid);
      rows24_async<D>(Gs + (it & 1) * TQ * D, d_out + ((int64_t)b * Nq + q0) * D, rows, tid);
      tile_rows_async_swz<D>(Kt + (it & 1) * tile, K + ((int64_t)b * H + h) * Nk * D, Nk, tid);
      if (it == 0) tile_rows_async_swz<D>(Vt, V + (int64_t)b * Nk * D, Nk, tid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_iter(0);
  // phase D reads K four rows at a time: the rows between Nk and nk4 are never copied, they must be zero
  for (int idx = tid; idx < (nk4 - Nk) * D; idx += TFT_THREADS) {
    Kt[(size_t)Nk * D + idx] = 0.f;
    Kt[tile + (size_t)Nk * D + idx] = 0.f;
  }

  const int rg = w & 3, khalf = w >> 2;               // phases A, B: rows rg*6 .. +5, keys khalf*96 + lane + 32c
  const int kg = tid >> 2, cg = tid & 3;              // phase C: keys kg + 64c, 16-byte column pieces cg, cg + 4, ...
  const int c4 = tid % D4, rq = (tid / D4) % RQ, ks = tid / (D4 * RQ);   // phase D
  const int n4 = nk4 / 4, per4 = (n4 + SLOTS - 1) / SLOTS;
  const int jq0 = ks * per4, jq1 = min(n4, jq0 + per4);

  float dk[TQ_C][NV * 4];
#pragma unroll
  for (int c = 0; c < TQ_C; ++c)
#pragma unroll
    for (int x = 0; x < NV * 4; ++x) dk[c][x] = 0.f;
  float dp[TQ_R][TQ_C];
  float pm[TQ_R][TQ_C];                               // the sum over the heads of this thread's probabilities (one row tile)
  unsigned mbits = 0, dead = 0;

  for (int it = 0; it < iters; ++it) {
    const int t = it / H, h = it - t * H, q0 = t * TQ, rows = min(TQ, Nq - q0);
    const bool fresh = h == 0;                        // new rows: mask bits and dP have to be formed, the head sum starts
    load_iter(it + 1);                                // into the buffers iteration it - 1 read (it ended with a barrier)
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();                                  // this iteration's tiles visible; everyone is past the previous one
    const float* Kh = Kt + (it & 1) * tile;
    const float* Qh = Qs + (it & 1) * TQ * D;
    const float* Gh = Gs + (it & 1) * TQ * D;

    // ---- A: scores and dP
    float da[TQ_R][TQ_C];
    if (fresh) {
      float mv[TQ_R][TQ_C];
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) {
          const int i = min(rg * TQ_R + r, rows - 1), j = min(khalf * (32 * TQ_C) + lane + 32 * c, Nk - 1);
          mv[r][c] = mask != nullptr ? __ldg(mask + (int64_t)(q0 + i) * Nk + j) : 0.f;
          da[r][c] = d_attn != nullptr ? __ldg(d_attn + ((int64_t)b * Nq + q0 + i) * Nk + j) : 0.f;
        }
      mbits = dead = 0;
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) {
          const int i = rg * TQ_R + r, j = khalf * (32 * TQ_C) + lane + 32 * c;
          if (j >= Nk) dead |= 1u << (r * TQ_C + c);
          else if (i < rows && mv[r][c] == 1.0f) mbits |= 1u << (r * TQ_C + c);
          if (i >= rows || j >= Nk) da[r][c] = 0.f;
          dp[r][c] = 0.f;
          pm[r][c] = 0.f;
        }
    }
    float s[TQ_R][TQ_C];
#pragma unroll
    for (int r = 0; r < TQ_R; ++r)
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) s[r][c] = 0.f;
    {
      const float* krow[TQ_C];
      const float* vrow[TQ_C];
      int ksw[TQ_C];
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) {
        const int j = min(khalf * (32 * TQ_C) + lane + 32 * c, Nk - 1);
        krow[c] = Kh + (size_t)j * D;
        vrow[c] = Vt + (size_t)j * D;
        ksw[c] = j & SW;
      }
      if (fresh) {
        tft_bwd_scores<D, true>(krow, vrow, ksw, Qh + rg * TQ_R * D, Gh + rg * TQ_R * D, s, dp);
#pragma unroll
        for (int r = 0; r < TQ_R; ++r)
#pragma unroll
          for (int c = 0; c < TQ_C; ++c) dp[r][c] = (dp[r][c] + da[r][c]) * inv_h;   // both head-mean terms (:797-812)
      } else {
        tft_bwd_scores<D, false>(krow, vrow, ksw, Qh + rg * TQ_R * D, Gh + rg * TQ_R * D, s, dp);
      }
    }

    // ---- B: softmax and its backward
    float hm[TQ_R];
#pragma unroll
    for (int r = 0; r < TQ_R; ++r) {
      float m = -INFINITY;
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) {
        const unsigned bit = 1u << (r * TQ_C + c);
        s[r][c] = (mbits & bit) ? MCA_MASKED_LOGIT : s[r][c] * scale;
        if (!(dead & bit)) m = fmaxf(m, s[r][c]);
      }
      hm[r] = warp_max(m);
    }
    if (lane < TQ_R) {
      float v = hm[0];
#pragma unroll
      for (int r = 1; r < TQ_R; ++r) v = lane == r ? hm[r] : v;
      ex[khalf * TQ + rg * TQ_R + lane] = v;
    }
    __syncthreads();
    float hs[TQ_R], hd[TQ_R];
#pragma unroll
    for (int r = 0; r < TQ_R; ++r) {
      const float m = fmaxf(ex[rg * TQ_R + r], ex[TQ + rg * TQ_R + r]);
      float sum = 0.f, dot = 0.f;
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) {
        s[r][c] = (dead & (1u << (r * TQ_C + c))) ? 0.f : tft_exp(s[r][c] - m);
        sum += s[r][c];
        dot = fmaf(s[r][c], dp[r][c], dot);
      }
      hs[r] = warp_sum(sum);
      hd[r] = warp_sum(dot);
    }
    if (lane < TQ_R) {
      float v = hs[0], u = hd[0];
#pragma unroll
      for (int r = 1; r < TQ_R; ++r) {
        v = lane == r ? hs[r] : v;
        u = lane == r ? hd[r] : u;
      }
      ex[2 * TQ + khalf * TQ + rg * TQ_R + lane] = v;
      ex[4 * TQ + khalf * TQ + rg * TQ_R + lane] = u;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < TQ_R; ++r) {
      const int i = rg * TQ_R + r;
      const float inv = 1.f / (ex[2 * TQ + i] + ex[3 * TQ + i]);
      const float dot = (ex[4 * TQ + i] + ex[5 * TQ + i]) * inv;      // sum_j P dP of the row
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) {
        const int j = khalf * (32 * TQ_C) + lane + 32 * c;
        const float pj = s[r][c] * inv;
        pm[r][c] += pj;
        Ss[i * TQ_KEYS + j] = pj * (dp[r][c] - dot) * scale;          // softmax backward, then the 1/sqrt(d) (:822-831)
      }
    }
    __syncthreads();                                  // P and dS complete

    // ---- C: dK_h (this tile's part) = dS^T Q_h
#pragma unroll 2
    for (int r = 0; r < TQ; ++r) {
      float sv[TQ_C];
      float4 qv[NV];
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) sv[c] = Ss[r * TQ_KEYS + kg + 64 * c];
#pragma unroll
      for (int x = 0; x < NV; ++x)
        qv[x] = *reinterpret_cast<const float4*>(Qh + r * D + 4 * (cg + 4 * x));   // the four lanes of a key: distinct banks
#pragma unroll
      for (int c = 0; c < TQ_C; ++c)
#pragma unroll
        for (int x = 0; x < NV; ++x) {
          dk[c][4 * x + 0] = fmaf(sv[c], qv[x].x, dk[c][4 * x + 0]);
          dk[c][4 * x + 1] = fmaf(sv[c], qv[x].y, dk[c][4 * x + 1]);
          dk[c][4 * x + 2] = fmaf(sv[c], qv[x].z, dk[c][4 * x + 2]);
          dk[c][4 * x + 3] = fmaf(sv[c], qv[x].w, dk[c][4 * x + 3]);
        }
    }

    // ---- D: dQ = dS K_h over this thread's slice of the keys
    float o[RPT][4];
#pragma unroll
    for (int r = 0; r < RPT; ++r) o[r][0] = o[r][1] = o[r][2] = o[r][3] = 0.f;
    for (int jq = jq0; jq < jq1; ++jq) {
      const int j = 4 * jq;
      float4 kv[4], sv[RPT];
#pragma unroll
      for (int u = 0; u < 4; ++u) kv[u] = *reinterpret_cast<const float4*>(Kh + (size_t)(j + u) * D + ((c4 ^ ((j + u) & SW)) << 2));
#pragma unroll
      for (int r = 0; r < RPT; ++r) sv[r] = *reinterpret_cast<const float4*>(Ss + (rq + RQ * r) * TQ_KEYS + j);
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        o[r][0] = fmaf(sv[r].x, kv[0].x, o[r][0]); o[r][1] = fmaf(sv[r].x, kv[0].y, o[r][1]);
        o[r][2] = fmaf(sv[r].x, kv[0].z, o[r][2]); o[r][3] = fmaf(sv[r].x, kv[0].w, o[r][3]);
      }
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        o[r][0] = fmaf(sv[r].y, kv[1].x, o[r][0]); o[r][1] = fmaf(sv[r].y, kv[1].y, o[r][1]);
        o[r][2] = fmaf(sv[r].y, kv[1].z, o[r][2]); o[r][3] = fmaf(sv[r].y, kv[1].w, o[r][3]);
      }
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        o[r][0] = fmaf(sv[r].z, kv[2].x, o[r][0]); o[r][1] = fmaf(sv[r].z, kv[2].y, o[r][1]);
        o[r][2] = fmaf(sv[r].z, kv[2].z, o[r][2]); o[r][3] = fmaf(sv[r].z, kv[2].w, o[r][3]);
      }
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        o[r][0] = fmaf(sv[r].w, kv[3].x, o[r][0]); o[r][1] = fmaf(sv[r].w, kv[3].y, o[r][1]);
        o[r][2] = fmaf(sv[r].w, kv[3].z, o[r][2]); o[r][3] = fmaf(sv[r].w, kv[3].w, o[r][3]);
      }
    }
    __syncthreads();                                  // the buffer of the head sum now takes the partial sums of dQ
    if (ks > 0) {
#pragma unroll
      for (int r = 0; r < RPT; ++r)
        *reinterpret_cast<float4*>(Ps + (size_t)(ks - 1) * TQ * D + (rq + RQ * r) * D + c4 * 4) = make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
    }
    __syncthreads();
    if (ks == 0) {
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        const int i = rq + RQ * r;
        float4 a = make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
#pragma unroll
        for (int s2 = 0; s2 < SLOTS - 1; ++s2) {
          const float4 p4 = *reinterpret_cast<const float4*>(Ps + (size_t)s2 * TQ * D + i * D + c4 * 4);
          a.x += p4.x; a.y += p4.y; a.z += p4.z; a.w += p4.w;
        }
        if (i < rows) *reinterpret_cast<float4*>(dQ + (((int64_t)b * H + h) * Nq + q0 + i) * D + c4 * 4) = a;
      }
    }
    // this tile's part of dK_h leaves the registers: the first tile writes, later ones add (one CTA, fixed order)
#pragma unroll
    for (int c = 0; c < TQ_C; ++c) {
      const int j = kg + 64 * c;
#pragma unroll
      for (int x = 0; x < NV; ++x) {
        if (j < Nk) {
          float4* g = reinterpret_cast<float4*>(dK + (((int64_t)b * H + h) * Nk + j) * D + 4 * (cg + 4 * x));
          float4 acc4 = make_float4(dk[c][4 * x], dk[c][4 * x + 1], dk[c][4 * x + 2], dk[c][4 * x + 3]);
          if (t > 0) { const float4 old = *g; acc4.x += old.x; acc4.y += old.y; acc4.z += old.z; acc4.w += old.w; }
          *g = acc4;
        }
        dk[c][4 * x] = dk[c][4 * x + 1] = dk[c][4 * x + 2] = dk[c][4 * x + 3] = 0.f;
      }
    }
    if (h == H - 1) {
      // the tile's last head: V's gradient is (sum_h P_h)^T dO / H, one product for all heads (the rows of dO are
      // those of this iteration's buffer)
      __syncthreads();                                // the partial sums of dQ have been read
#pragma unroll
      for (int r = 0; r < TQ_R; ++r)
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) Ps[(rg * TQ_R + r) * TQ_KEYS + khalf * (32 * TQ_C) + lane + 32 * c] = pm[r][c];
      __syncthreads();
      float dv[TQ_C][NV * 4];
#pragma unroll
      for (int c = 0; c < TQ_C; ++c)
#pragma unroll
        for (int x = 0; x < NV * 4; ++x) dv[c][x] = 0.f;
#pragma unroll 2
      for (int r = 0; r < TQ; ++r) {
        float pv[TQ_C];
        float4 gv[NV];
#pragma unroll
        for (int c = 0; c < TQ_C; ++c) pv[c] = Ps[r * TQ_KEYS + kg + 64 * c];
#pragma unroll
        for (int x = 0; x < NV; ++x) gv[x] = *reinterpret_cast<const float4*>(Gh + r * D + 4 * (cg + 4 * x));
#pragma unroll
        for (int c = 0; c < TQ_C; ++c)
#pragma unroll
          for (int x = 0; x < NV; ++x) {
            dv[c][4 * x + 0] = fmaf(pv[c], gv[x].x, dv[c][4 * x + 0]);
            dv[c][4 * x + 1] = fmaf(pv[c], gv[x].y, dv[c][4 * x + 1]);
            dv[c][4 * x + 2] = fmaf(pv[c], gv[x].z, dv[c][4 * x + 2]);
            dv[c][4 * x + 3] = fmaf(pv[c], gv[x].w, dv[c][4 * x + 3]);
          }
      }
#pragma unroll
      for (int c = 0; c < TQ_C; ++c) {
        const int j = kg + 64 * c;
        if (j < Nk) {
#pragma unroll
          for (int x = 0; x < NV; ++x) {
            float4* g = reinterpret_cast<float4*>(dV + ((int64_t)b * Nk + j) * D + 4 * (cg + 4 * x));
            float4 acc4 = make_float4(dv[c][4 * x] * inv_h, dv[c][4 * x + 1] * inv_h, dv[c][4 * x + 2] * inv_h, dv[c][4 * x + 3] * inv_h);
            if (t > 0) { const float4 old = *g; acc4.x += old.x; acc4.y += old.y; acc4.z += old.z; acc4.w += old.w; }
            *g = acc4;
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

}  // namespace

int mca_tft_attention_backward_f32(const float* q, const float* k, const float* v, const float* mask,
                                   const float* d_out, const float* d_attn, int B, int H, int Nq, int Nk, int d,
                                   float* dq, float* dk, float* dv, void* stream) {
  if (!q || !k || !v || !d_out || !dq || !dk || !dv) return ERROR_PARAM_NULL;
  if (B <= 0 || H <= 0 || Nq <= 0 || Nk <= 0 || d <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (d % 4 != 0 || (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15))
    return ERROR_ATTN_UNSUPPORTED_SHAPE;
  // the tiled kernel where the shape fits it, else the generic one
  const auto aligned = [](const void* p_) { return (reinterpret_cast<uintptr_t>(p_) & 15) == 0; };
  if ((d == 16 || d == 32 || d == 64) && Nk <= TQ_KEYS && aligned(q) && aligned(d_out) && aligned(dq) && aligned(dk) && aligned(dv)) {
    const size_t nk4 = ((size_t)Nk + 3) & ~(size_t)3;
    const size_t smem_t = sizeof(float) * (3 * nk4 * d + 4 * (size_t)TQ * d + 2 * (size_t)TQ * TQ_KEYS + 6 * TQ);
    const float sc = 1.0f / sqrtf((float)d);
    cudaStream_t st = (cudaStream_t)stream;
#define MCA_TFT_BWD_TILED(D_)                                                                                                 \
    MCA_CUDA_TRY(cudaFuncSetAttribute(tft_bwd_tiled_kernel<D_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_t)); \
    tft_bwd_tiled_kernel<D_><<<B, TFT_THREADS, smem_t, st>>>(q, k, v, mask, d_out, d_attn, H, Nq, Nk, sc, dq, dk, dv);
    if (d == 64) { MCA_TFT_BWD_TILED(64) } else if (d == 32) { MCA_TFT_BWD_TILED(32) } else { MCA_TFT_BWD_TILED(16) }
#undef MCA_TFT_BWD_TILED
    return mca_launch_status();
  }
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
  // the tiled kernel where the shape fits it (two K buffers and two CTAs per SM), else the generic one
  const size_t smem_t = sizeof(float) * (2 * (size_t)Nk * d + 2 * (size_t)TQ * d + 4 * TQ);
  const int slices = TFT_THREADS / d;   // key slices of the final product: TFT_THREADS / ((d / 4) * 4)
  // a K buffer must also hold the mean probabilities (24 x Nk) and the partial outputs of the other slices
  const bool room = (size_t)TQ * Nk + (size_t)(slices - 1) * TQ * d <= (size_t)Nk * d;
  if ((d == 16 || d == 32 || d == 64) && Nk <= TQ_KEYS && smem_t <= 113 * 1024 && room && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    dim3 grid_t(mca_ceil_div(Nq, TQ), B);
    const float sc = 1.0f / sqrtf((float)d);
    cudaStream_t st = (cudaStream_t)stream;
#define MCA_TFT_TILED(D_)                                                                                                 \
    MCA_CUDA_TRY(cudaFuncSetAttribute(tft_fwd_tiled_kernel<D_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_t)); \
    tft_fwd_tiled_kernel<D_><<<grid_t, TFT_THREADS, smem_t, st>>>(q, k, v, mask, H, Nq, Nk, sc, out, attn);
    if (d == 64) { MCA_TFT_TILED(64) } else if (d == 32) { MCA_TFT_TILED(32) } else { MCA_TFT_TILED(16) }
#undef MCA_TFT_TILED
    return mca_launch_status();
  }
  const size_t smem = sizeof(float) * ((size_t)Nk * (d + 4) + (size_t)H * TFT_ROWS * d + 2 * (size_t)TFT_ROWS * Nk);
  if (smem > 227 * 1024) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  MCA_CUDA_TRY(cudaFuncSetAttribute(tft_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(mca_ceil_div(Nq, TFT_ROWS), B);
  tft_fwd_kernel<<<grid, TFT_THREADS, smem, (cudaStream_t)stream>>>(q, k, v, mask, H, Nq, Nk, d,
                                                                    1.0f / sqrtf((float)d), out, attn);
  return mca_launch_status();
}

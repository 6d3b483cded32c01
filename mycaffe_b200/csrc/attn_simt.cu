// Exact-fp32 scaled-dot-product attention on CUDA cores: forward, and a recompute-based
// backward.  This is the default fp32 path behind ATTN_FWD / ATTN_BWD: it reproduces the
// reference's arithmetic (attn.cu:518-661 of CudaDnnDLL) -- scale applied to the finished dot
// product, masked logits overwritten with the finite value -1e29, max-subtracted softmax --
// without ever materialising the (B,H,T,T) score tensors the reference allocates in
// attnHandle::Set (attn.cu:436-452).  It accepts every mask form of the reference and any head
// size up to 128.  The tensor-core kernels in attn_tc.cu cover the bf16 / tf32 variants.
//
// Tiling: one CTA owns 64 query rows of one (batch, head) and walks the keys 64 at a time.
// 256 threads form a 16x16 grid; thread (ty,tx) owns rows ty+16a and columns tx+16b of the
// 64x64 score tile, so a row's softmax statistics live in one half-warp (shuffle reductions).
// Shared tiles are row-major with a stride of DP+4 floats, which keeps every 128-bit shared
// load of the inner products conflict-free.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int BM = 64;        // query rows per CTA
constexpr int BN = 64;        // keys per step
constexpr int NT = 256;       // threads per CTA
constexpr int PLD = BN + 4;   // leading dimension of the 64x64 probability tile

template <int DP> struct Tile {
  static constexpr int LD = DP + 4;
  static constexpr int VEC = (DP >= 64) ? 4 : (DP / 16);
  static constexpr int NU = DP / 16 / VEC;
  static constexpr int CPT = DP / 16;  // output columns per thread
};

// Copy rows [row0, row0+64) of a (T,D) matrix with row stride ld into smem[64][DP+4], zero-filling
// rows >= T and columns >= D.
template <int DP>
__device__ __forceinline__ void load_tile(float* __restrict__ s, const float* __restrict__ g, int64_t ld, int row0,
                                          int T, int D, bool vec_ok, int tid) {
  constexpr int LD = Tile<DP>::LD;
  if (vec_ok) {
    constexpr int C4 = DP / 4;
    for (int idx = tid; idx < 64 * C4; idx += NT) {
      const int r = idx / C4, c4 = idx % C4;
      float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row0 + r < T && c4 * 4 < D) val = __ldg(reinterpret_cast<const float4*>(g + (int64_t)(row0 + r) * ld) + c4);
      *reinterpret_cast<float4*>(s + r * LD + c4 * 4) = val;
    }
  } else {
    for (int idx = tid; idx < 64 * DP; idx += NT) {
      const int r = idx / DP, c = idx % DP;
      float val = 0.f;
      if (row0 + r < T && c < D) val = __ldg(g + (int64_t)(row0 + r) * ld + c);
      s[r * LD + c] = val;
    }
  }
}

// s[a][b] = sum_d A[ty+16a][d] * B[tx+16b][d]
template <int DP>
__device__ __forceinline__ void tile_nt(const float* __restrict__ As, const float* __restrict__ Bs, float (&s)[4][4],
                                        int ty, int tx) {
  constexpr int LD = Tile<DP>::LD;
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) s[a][b] = 0.f;
#pragma unroll 4
  for (int d = 0; d < DP; d += 4) {
    float4 av[4], bv[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) av[a] = *reinterpret_cast<const float4*>(As + (ty + 16 * a) * LD + d);
#pragma unroll
    for (int b = 0; b < 4; ++b) bv[b] = *reinterpret_cast<const float4*>(Bs + (tx + 16 * b) * LD + d);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        s[a][b] = fmaf(av[a].x, bv[b].x, s[a][b]);
        s[a][b] = fmaf(av[a].y, bv[b].y, s[a][b]);
        s[a][b] = fmaf(av[a].z, bv[b].z, s[a][b]);
        s[a][b] = fmaf(av[a].w, bv[b].w, s[a][b]);
      }
  }
}

// Column owned by (tx, u, w): u*16*VEC + tx*VEC + w.
template <int DP> __device__ __forceinline__ int out_col(int tx, int c) {
  constexpr int VEC = Tile<DP>::VEC;
  return (c / VEC) * 16 * VEC + tx * VEC + (c % VEC);
}

// acc[a][c] += sum_j P[ty+16a][j] * V[j][col(c)]   (P: 64 x 64, ld PLD; V: 64 x DP, ld DP+4)
template <int DP>
__device__ __forceinline__ void tile_nn(const float* __restrict__ Ps, const float* __restrict__ Vs,
                                        float (&acc)[4][Tile<DP>::CPT], int ty, int tx) {
  constexpr int LD = Tile<DP>::LD, VEC = Tile<DP>::VEC, NU = Tile<DP>::NU;
#pragma unroll 2
  for (int j4 = 0; j4 < BN / 4; ++j4) {
    float4 p[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) p[a] = *reinterpret_cast<const float4*>(Ps + (ty + 16 * a) * PLD + j4 * 4);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* vrow = Vs + (j4 * 4 + w) * LD + tx * VEC;
      float vv[Tile<DP>::CPT];
#pragma unroll
      for (int u = 0; u < NU; ++u) {
        if constexpr (VEC == 4) {
          const float4 t = *reinterpret_cast<const float4*>(vrow + u * 64);
          vv[u * 4 + 0] = t.x; vv[u * 4 + 1] = t.y; vv[u * 4 + 2] = t.z; vv[u * 4 + 3] = t.w;
        } else if constexpr (VEC == 2) {
          const float2 t = *reinterpret_cast<const float2*>(vrow + u * 32);
          vv[u * 2 + 0] = t.x; vv[u * 2 + 1] = t.y;
        } else {
          vv[u] = vrow[u * 16];
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float pw = (w == 0) ? p[a].x : (w == 1) ? p[a].y : (w == 2) ? p[a].z : p[a].w;
#pragma unroll
        for (int c = 0; c < Tile<DP>::CPT; ++c) acc[a][c] = fmaf(pw, vv[c], acc[a][c]);
      }
    }
  }
}

__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Logit after scale and mask, the reference's order (attn.cu:567-583).  Keys beyond T do not
// exist: they get -inf so that they contribute exactly zero probability.
__device__ __forceinline__ float masked_logit(float dot, float scale, int i, int j, int b, int T, int mode,
                                              const float* __restrict__ mask) {
  if (j >= T) return -INFINITY;
  float s = dot * scale;
  if (mode == MCA_MASK_CAUSAL) { if (j > i) s = MCA_MASKED_LOGIT; }
  else if (mode == MCA_MASK_TT) { if (i < T && __ldg(mask + (int64_t)i * T + j) == 0.f) s = MCA_MASKED_LOGIT; }
  else if (mode == MCA_MASK_BATCH) { if (__ldg(mask + (int64_t)b * T + j) == 0.f) s = MCA_MASKED_LOGIT; }
  return s;
}

// A (T,T) mask that a preceding classification launch found to be exactly tril(ones) is
// treated as analytic causal (tiles above the diagonal are skipped).
__device__ __forceinline__ int effective_mode(int mode, const int* __restrict__ causal_flag) {
  if (mode == MCA_MASK_TT && causal_flag != nullptr && *causal_flag != 0) return MCA_MASK_CAUSAL;
  return mode;
}

template <int DP>
constexpr size_t fwd_smem_bytes() {
  // Q, K, V tiles; the probability tile aliases the K tile when it fits (DP >= 64).
  return sizeof(float) * (3 * 64 * (DP + 4) + ((DP >= 64) ? 0 : 64 * PLD));
}

template <int DP>
__global__ void __launch_bounds__(NT) sdpa_fwd_f32_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                         const float* __restrict__ V,
                                                         const float* __restrict__ mask, int mask_mode,
                                                         const int* __restrict__ causal_flag, int H, int T, int D,
                                                         float scale, float* __restrict__ Y,
                                                         float* __restrict__ row_max, float* __restrict__ row_sum,
                                                         float* __restrict__ y_copy, int vec_ok,
                                                         const McaStrides sin, const McaStrides sout) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = Tile<DP>::LD, CPT = Tile<DP>::CPT;
  float* Qs = smem;
  float* Ks = Qs + 64 * LD;
  float* Vs = Ks + 64 * LD;
  float* Ps = (DP >= 64) ? Ks : (Vs + 64 * LD);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y, b = bh / H;
  // Longest (most keys) causal tiles first.
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * BM;
  const int mode = effective_mode(mask_mode, causal_flag);
  const int64_t in_base = (int64_t)b * sin.b + (int64_t)(bh - b * H) * sin.h;
  const float* Qg = Q + in_base;
  const float* Kg = K + in_base;
  const float* Vg = V + in_base;

  load_tile<DP>(Qs, Qg, sin.t, q0, T, D, vec_ok, tid);

  float m[4], l[4], acc[4][CPT];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    m[a] = -INFINITY; l[a] = 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) acc[a][c] = 0.f;
  }
  const int kv_end = (mode == MCA_MASK_CAUSAL) ? min(T, q0 + BM) : T;
  for (int k0 = 0; k0 < kv_end; k0 += BN) {
    __syncthreads();  // previous step's readers of Ks/Vs/Ps are done (also orders the Q load)
    load_tile<DP>(Ks, Kg, sin.t, k0, T, D, vec_ok, tid);
    load_tile<DP>(Vs, Vg, sin.t, k0, T, D, vec_ok, tid);
    __syncthreads();
    float s[4][4];
    tile_nt<DP>(Qs, Ks, s, ty, tx);
    if (DP >= 64) __syncthreads();  // Ps aliases Ks
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = q0 + ty + 16 * a;
      float mx = -INFINITY;
#pragma unroll
      for (int bb = 0; bb < 4; ++bb) {
        s[a][bb] = masked_logit(s[a][bb], scale, i, k0 + tx + 16 * bb, b, T, mode, mask);
        mx = fmaxf(mx, s[a][bb]);
      }
      mx = half_warp_max(mx);
      const float m_new = fmaxf(m[a], mx);
      const float corr = __expf(m[a] - m_new);  // exp(-inf) = 0 on the first step
      float rs = 0.f;
#pragma unroll
      for (int bb = 0; bb < 4; ++bb) {
        const float p = expf(s[a][bb] - m_new);
        rs += p;
        Ps[(ty + 16 * a) * PLD + tx + 16 * bb] = p;
      }
      rs = half_warp_sum(rs);
      l[a] = l[a] * corr + rs;
      m[a] = m_new;
#pragma unroll
      for (int c = 0; c < CPT; ++c) acc[a][c] *= corr;
    }
    __syncthreads();
    tile_nn<DP>(Ps, Vs, acc, ty, tx);
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = q0 + ty + 16 * a;
    if (i >= T) continue;
    const float inv = 1.f / l[a];
    float* yo = Y + (int64_t)b * sout.b + (int64_t)(bh - b * H) * sout.h + (int64_t)i * sout.t;
    float* yc = y_copy ? y_copy + ((int64_t)bh * T + i) * D : nullptr;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int col = out_col<DP>(tx, c);
      if (col < D) {
        const float o = acc[a][c] * inv;
        yo[col] = o;
        if (yc) yc[col] = o;
      }
    }
    if (tx == 0 && row_max) { row_max[(int64_t)bh * T + i] = m[a]; row_sum[(int64_t)bh * T + i] = l[a]; }
  }
}

// delta[i] = sum_c dY[i][c] * Y[i][c]  (the rowsum(dP o P) term of the softmax backward).
__global__ void sdpa_bwd_delta_kernel(const float* __restrict__ dY, const float* __restrict__ Ysaved, int64_t rows,
                                      int H, int T, int D, const McaStrides sdy, float* __restrict__ delta) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t bh = row / T;
  const int64_t b = bh / H;
  const float* dyr = dY + b * sdy.b + (bh - b * H) * sdy.h + (row - bh * T) * sdy.t;   // Ysaved is the handle's own contiguous copy
  float acc = 0.f;
  for (int c = lane; c < D; c += 32) acc = fmaf(dyr[c], Ysaved[row * D + c], acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) delta[row] = acc;
}

template <int DP>
constexpr size_t bwd_smem_bytes() { return sizeof(float) * (4 * 64 * (DP + 4) + 2 * 64 * PLD); }

// dK, dV for one 64-key tile: walks the query tiles, recomputes P from the saved row
// statistics, and accumulates dV += P^T dY, dK += dS^T Q (attn.cu:380-397, 637-657).
template <int DP>
__global__ void __launch_bounds__(NT) sdpa_bwd_dkdv_f32_kernel(
    const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
    const float* __restrict__ dY, const float* __restrict__ mask, int mask_mode, const int* __restrict__ causal_flag,
    const float* __restrict__ row_max, const float* __restrict__ row_sum, const float* __restrict__ delta, int H,
    int T, int D, float scale, float* __restrict__ dK, float* __restrict__ dV, int vec_ok, const McaStrides sin,
    const McaStrides sout) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = Tile<DP>::LD, CPT = Tile<DP>::CPT;
  float* Ks = smem;
  float* Vs = Ks + 64 * LD;
  float* Qs = Vs + 64 * LD;
  float* dOs = Qs + 64 * LD;
  float* PsT = dOs + 64 * LD;    // [key][query]
  float* dSsT = PsT + 64 * PLD;  // [key][query]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y, b = bh / H;
  const int k0 = blockIdx.x * BN;
  const int mode = effective_mode(mask_mode, causal_flag);
  const int64_t base = (int64_t)b * sin.b + (int64_t)(bh - b * H) * sin.h;
  const int64_t base_dy = (int64_t)b * sout.b + (int64_t)(bh - b * H) * sout.h;
  load_tile<DP>(Ks, K + base, sin.t, k0, T, D, vec_ok, tid);
  load_tile<DP>(Vs, V + base, sin.t, k0, T, D, vec_ok, tid);
  float dk[4][CPT], dv[4][CPT];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int c = 0; c < CPT; ++c) { dk[a][c] = 0.f; dv[a][c] = 0.f; }
  const int q_begin = (mode == MCA_MASK_CAUSAL) ? k0 : 0;  // k0 is a multiple of 64
  for (int q0 = q_begin; q0 < T; q0 += BM) {
    __syncthreads();
    load_tile<DP>(Qs, Q + base, sin.t, q0, T, D, vec_ok, tid);
    load_tile<DP>(dOs, dY + base_dy, sout.t, q0, T, D, vec_ok, tid);
    __syncthreads();
    float s[4][4], dp[4][4];
    tile_nt<DP>(Qs, Ks, s, ty, tx);     // s[a][b]: query ty+16a, key tx+16b
    tile_nt<DP>(dOs, Vs, dp, ty, tx);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = q0 + ty + 16 * a;
      float mi = 0.f, li = 1.f, di = 0.f;
      if (i < T) { mi = row_max[(int64_t)bh * T + i]; li = row_sum[(int64_t)bh * T + i]; di = delta[(int64_t)bh * T + i]; }
      const float inv_l = 1.f / li;
#pragma unroll
      for (int bb = 0; bb < 4; ++bb) {
        const int j = k0 + tx + 16 * bb;
        const float sv = masked_logit(s[a][bb], scale, i, j, b, T, mode, mask);
        const float p = (i < T) ? expf(sv - mi) * inv_l : 0.f;
        const float ds = p * (dp[a][bb] - di) * scale;
        PsT[(tx + 16 * bb) * PLD + ty + 16 * a] = p;
        dSsT[(tx + 16 * bb) * PLD + ty + 16 * a] = ds;
      }
    }
    __syncthreads();
    tile_nn<DP>(PsT, dOs, dv, ty, tx);   // rows = keys ty+16a
    tile_nn<DP>(dSsT, Qs, dk, ty, tx);
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int j = k0 + ty + 16 * a;
    if (j >= T) continue;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int col = out_col<DP>(tx, c);
      if (col < D) { dK[base + (int64_t)j * sin.t + col] = dk[a][c]; dV[base + (int64_t)j * sin.t + col] = dv[a][c]; }
    }
  }
}

// dQ for one 64-query tile: dQ = dS K with dS recomputed per key tile.
template <int DP>
__global__ void __launch_bounds__(NT) sdpa_bwd_dq_f32_kernel(
    const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
    const float* __restrict__ dY, const float* __restrict__ mask, int mask_mode, const int* __restrict__ causal_flag,
    const float* __restrict__ row_max, const float* __restrict__ row_sum, const float* __restrict__ delta, int H,
    int T, int D, float scale, float* __restrict__ dQ, int vec_ok, const McaStrides sin, const McaStrides sout) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = Tile<DP>::LD, CPT = Tile<DP>::CPT;
  float* Qs = smem;
  float* dOs = Qs + 64 * LD;
  float* Ks = dOs + 64 * LD;
  float* Vs = Ks + 64 * LD;
  float* dSs = Vs + 64 * LD;  // [query][key]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y, b = bh / H;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * BM;
  const int mode = effective_mode(mask_mode, causal_flag);
  const int64_t base = (int64_t)b * sin.b + (int64_t)(bh - b * H) * sin.h;
  load_tile<DP>(Qs, Q + base, sin.t, q0, T, D, vec_ok, tid);
  load_tile<DP>(dOs, dY + (int64_t)b * sout.b + (int64_t)(bh - b * H) * sout.h, sout.t, q0, T, D, vec_ok, tid);
  float mi[4], inv_l[4], di[4], dq[4][CPT];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = q0 + ty + 16 * a;
    mi[a] = 0.f; inv_l[a] = 0.f; di[a] = 0.f;
    if (i < T) { mi[a] = row_max[(int64_t)bh * T + i]; inv_l[a] = 1.f / row_sum[(int64_t)bh * T + i]; di[a] = delta[(int64_t)bh * T + i]; }
#pragma unroll
    for (int c = 0; c < CPT; ++c) dq[a][c] = 0.f;
  }
  const int kv_end = (mode == MCA_MASK_CAUSAL) ? min(T, q0 + BM) : T;
  for (int k0 = 0; k0 < kv_end; k0 += BN) {
    __syncthreads();
    load_tile<DP>(Ks, K + base, sin.t, k0, T, D, vec_ok, tid);
    load_tile<DP>(Vs, V + base, sin.t, k0, T, D, vec_ok, tid);
    __syncthreads();
    float s[4][4], dp[4][4];
    tile_nt<DP>(Qs, Ks, s, ty, tx);
    tile_nt<DP>(dOs, Vs, dp, ty, tx);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = q0 + ty + 16 * a;
#pragma unroll
      for (int bb = 0; bb < 4; ++bb) {
        const int j = k0 + tx + 16 * bb;
        const float sv = masked_logit(s[a][bb], scale, i, j, b, T, mode, mask);
        const float p = (i < T) ? expf(sv - mi[a]) * inv_l[a] : 0.f;
        dSs[(ty + 16 * a) * PLD + tx + 16 * bb] = p * (dp[a][bb] - di[a]) * scale;
      }
    }
    __syncthreads();
    tile_nn<DP>(dSs, Ks, dq, ty, tx);
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = q0 + ty + 16 * a;
    if (i >= T) continue;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int col = out_col<DP>(tx, c);
      if (col < D) dQ[base + (int64_t)i * sin.t + col] = dq[a][c];
    }
  }
}

// Sets *flag to 1 iff mask (T,T) is exactly lower-triangular ones (fillMask,
// CausalSelfAttentionLayer.cs:276-291).  *flag must hold 1 on entry.
__global__ void classify_causal_kernel(const float* __restrict__ mask, int T, int* __restrict__ flag) {
  const int64_t n = (int64_t)T * T;
  bool ok = true;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx / T), j = (int)(idx % T);
    const float want = (j <= i) ? 1.f : 0.f;
    if (mask[idx] != want) ok = false;
  }
  if (!ok) *flag = 0;
}
__global__ void set_int_kernel(int* p, int v) { *p = v; }

// The same answer from one launch: a warp per row (16-byte loads when T allows), the blocks' mismatch counts and a
// ticket in two scratch words that are zero before and after; the last block to finish writes the flag.
__global__ void __launch_bounds__(256) classify_causal_rows_kernel(const float* __restrict__ mask, int T, int* __restrict__ flag,
                                                                   int* __restrict__ scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  bool bad = false;
  for (int i = blockIdx.x * 8 + warp; i < T; i += gridDim.x * 8) {
    const float* row = mask + (int64_t)i * T;
    if ((T & 3) == 0) {
      for (int j = lane * 4; j < T; j += 128) {
        const float4 m = *reinterpret_cast<const float4*>(row + j);
        bad |= m.x != (j <= i ? 1.f : 0.f) || m.y != (j + 1 <= i ? 1.f : 0.f) || m.z != (j + 2 <= i ? 1.f : 0.f) ||
               m.w != (j + 3 <= i ? 1.f : 0.f);
      }
    } else {
      for (int j = lane; j < T; j += 32) bad |= row[j] != (j <= i ? 1.f : 0.f);
    }
  }
  const int any_bad = __syncthreads_or(bad ? 1 : 0);
  if (threadIdx.x == 0) {
    if (any_bad) atomicAdd(scratch, 1);
    __threadfence();
    if (atomicAdd(scratch + 1, 1) == (int)gridDim.x - 1) {
      __threadfence();
      *flag = atomicExch(scratch, 0) == 0 ? 1 : 0;
      scratch[1] = 0;
    }
  }
}

int pick_dp(int D) { return D <= 16 ? 16 : D <= 32 ? 32 : D <= 64 ? 64 : D <= 128 ? 128 : 0; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename F> int set_smem(F kernel, size_t bytes) {
  if (bytes > 48 * 1024) MCA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return 0;
}

}  // namespace

int mca_classify_causal_mask_ws(const float* mask, int T, int* flag, int* scratch, void* stream) {
  if (!mask || !flag || !scratch) return ERROR_PARAM_NULL;
  if (T <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  const int blocks = std::min(1184, (T + 7) / 8);
  classify_causal_rows_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(mask, T, flag, scratch);
  return mca_launch_status();
}

int mca_classify_causal_mask(const float* mask, int T, int* flag, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  set_int_kernel<<<1, 1, 0, st>>>(flag, 1);
  const int64_t n = (int64_t)T * T;
  const int blocks = (int)((n + 1023) / 1024 > 1184 ? 1184 : (n + 1023) / 1024);
  classify_causal_kernel<<<blocks, 256, 0, st>>>(mask, T, flag);
  return mca_launch_status();
}

template <int DP>
static int launch_fwd(const float* q, const float* k, const float* v, const float* mask, int mode, const int* flag,
                      int B, int H, int T, int D, float* y, float* rmax, float* rsum, float* ycopy, int layout,
                      cudaStream_t st) {
  const size_t smem = fwd_smem_bytes<DP>();
  int e = set_smem(sdpa_fwd_f32_kernel<DP>, smem);
  if (e) return e;
  const McaStrides sin = mca_in_strides(layout, H, T, D), sout = mca_out_strides(layout, H, T, D);
  const int vec_ok = (D % 4 == 0) && aligned16(q) && aligned16(k) && aligned16(v);  // every stride is a multiple of D
  dim3 grid(mca_ceil_div(T, BM), B * H);
  sdpa_fwd_f32_kernel<DP><<<grid, NT, smem, st>>>(q, k, v, mask, mode, flag, H, T, D, 1.0f / sqrtf((float)D), y, rmax,
                                                  rsum, ycopy, vec_ok, sin, sout);
  return mca_launch_status();
}

int mca_sdpa_forward_f32(const float* q, const float* k, const float* v, const float* mask, int mask_mode,
                         const int* causal_flag, int B, int H, int T, int D, float* y, float* row_max,
                         float* row_sum, float* y_copy, void* stream) {
  return mca_sdpa_forward_f32_layout(q, k, v, mask, mask_mode, causal_flag, B, H, T, D, y, row_max, row_sum, y_copy,
                                     MCA_LAYOUT_BHTD, stream);
}

int mca_sdpa_forward_f32_layout(const float* q, const float* k, const float* v, const float* mask, int mask_mode,
                                const int* causal_flag, int B, int H, int T, int D, float* y, float* row_max,
                                float* row_sum, float* y_copy, int layout, void* stream) {
  if (!q || !k || !v || !y) return ERROR_PARAM_NULL;
  if (layout != MCA_LAYOUT_BHTD && layout != MCA_LAYOUT_PACKED) return ERROR_PARAM_OUT_OF_RANGE;
  if (B <= 0 || H <= 0 || T <= 0 || D <= 0 || (int64_t)B * H > 65535) return ERROR_PARAM_OUT_OF_RANGE;
  if ((mask_mode == MCA_MASK_TT || mask_mode == MCA_MASK_BATCH) && !mask) return ERROR_PARAM_NULL;
  if ((row_max == nullptr) != (row_sum == nullptr)) return ERROR_PARAM_NULL;
  cudaStream_t st = (cudaStream_t)stream;
  switch (pick_dp(D)) {
    case 16: return launch_fwd<16>(q, k, v, mask, mask_mode, causal_flag, B, H, T, D, y, row_max, row_sum, y_copy, layout, st);
    case 32: return launch_fwd<32>(q, k, v, mask, mask_mode, causal_flag, B, H, T, D, y, row_max, row_sum, y_copy, layout, st);
    case 64: return launch_fwd<64>(q, k, v, mask, mask_mode, causal_flag, B, H, T, D, y, row_max, row_sum, y_copy, layout, st);
    case 128: return launch_fwd<128>(q, k, v, mask, mask_mode, causal_flag, B, H, T, D, y, row_max, row_sum, y_copy, layout, st);
  }
  return ERROR_ATTN_UNSUPPORTED_SHAPE;
}

template <int DP>
static int launch_bwd(const float* q, const float* k, const float* v, const float* dy, const float* mask, int mode,
                      const int* flag, const float* rmax, const float* rsum, const float* delta, int B, int H, int T,
                      int D, float* dq, float* dk, float* dv, int layout, cudaStream_t st) {
  const McaStrides sin = mca_in_strides(layout, H, T, D), sout = mca_out_strides(layout, H, T, D);
  const size_t smem_a = bwd_smem_bytes<DP>();
  const size_t smem_b = sizeof(float) * (4 * 64 * (DP + 4) + 64 * PLD);
  int e = set_smem(sdpa_bwd_dkdv_f32_kernel<DP>, smem_a);
  if (e) return e;
  e = set_smem(sdpa_bwd_dq_f32_kernel<DP>, smem_b);
  if (e) return e;
  const int vec_ok = (D % 4 == 0) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(dy);
  const float scale = 1.0f / sqrtf((float)D);
  dim3 grid(mca_ceil_div(T, BM), B * H);
  sdpa_bwd_dkdv_f32_kernel<DP><<<grid, NT, smem_a, st>>>(q, k, v, dy, mask, mode, flag, rmax, rsum, delta, H, T, D,
                                                         scale, dk, dv, vec_ok, sin, sout);
  e = mca_launch_status();
  if (e) return e;
  sdpa_bwd_dq_f32_kernel<DP><<<grid, NT, smem_b, st>>>(q, k, v, dy, mask, mode, flag, rmax, rsum, delta, H, T, D, scale,
                                                       dq, vec_ok, sin, sout);
  return mca_launch_status();
}

int mca_sdpa_backward_f32(const float* q, const float* k, const float* v, const float* dy, const float* y_saved,
                          const float* mask, int mask_mode, const int* causal_flag, const float* row_max,
                          const float* row_sum, float* delta_scratch, int B, int H, int T, int D, float* dq,
                          float* dk, float* dv, void* stream) {
  return mca_sdpa_backward_f32_layout(q, k, v, dy, y_saved, mask, mask_mode, causal_flag, row_max, row_sum, delta_scratch,
                                      B, H, T, D, dq, dk, dv, MCA_LAYOUT_BHTD, stream);
}

int mca_sdpa_backward_f32_layout(const float* q, const float* k, const float* v, const float* dy, const float* y_saved,
                                 const float* mask, int mask_mode, const int* causal_flag, const float* row_max,
                                 const float* row_sum, float* delta_scratch, int B, int H, int T, int D, float* dq,
                                 float* dk, float* dv, int layout, void* stream) {
  if (layout != MCA_LAYOUT_BHTD && layout != MCA_LAYOUT_PACKED) return ERROR_PARAM_OUT_OF_RANGE;
  if (!q || !k || !v || !dy || !y_saved || !row_max || !row_sum || !delta_scratch || !dq || !dk || !dv)
    return ERROR_PARAM_NULL;
  if (B <= 0 || H <= 0 || T <= 0 || D <= 0 || (int64_t)B * H > 65535) return ERROR_PARAM_OUT_OF_RANGE;
  if ((mask_mode == MCA_MASK_TT || mask_mode == MCA_MASK_BATCH) && !mask) return ERROR_PARAM_NULL;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows = (int64_t)B * H * T;
  sdpa_bwd_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(dy, y_saved, rows, H, T, D,
                                                                    mca_out_strides(layout, H, T, D), delta_scratch);
  int e = mca_launch_status();
  if (e) return e;
  switch (pick_dp(D)) {
    case 16: return launch_bwd<16>(q, k, v, dy, mask, mask_mode, causal_flag, row_max, row_sum, delta_scratch, B, H, T, D, dq, dk, dv, layout, st);
    case 32: return launch_bwd<32>(q, k, v, dy, mask, mask_mode, causal_flag, row_max, row_sum, delta_scratch, B, H, T, D, dq, dk, dv, layout, st);
    case 64: return launch_bwd<64>(q, k, v, dy, mask, mask_mode, causal_flag, row_max, row_sum, delta_scratch, B, H, T, D, dq, dk, dv, layout, st);
    case 128: return launch_bwd<128>(q, k, v, dy, mask, mask_mode, causal_flag, row_max, row_sum, delta_scratch, B, H, T, D, dq, dk, dv, layout, st);
  }
  return ERROR_ATTN_UNSUPPORTED_SHAPE;
}

// Fused flash-style attention forward on the 5th-generation tensor cores (sm_100a):
// S = Q K^T by tcgen05.mma into TMEM, online softmax by two warpgroups that read S from TMEM
// and write the probabilities back to TMEM as the A operand of the second product, O += P V
// accumulated in TMEM; Q/K/V tiles arrive by TMA (cp.async.bulk.tensor, no multicast) into
// 128-byte-swizzled shared memory behind mbarrier pipelines.
//
// Same mathematics as the reference's attnHandle<T>::Forward (CudaDnnDLL/Cuda Files/
// attn.cu:518-602: scale, mask, max-subtracted softmax, times V) for a causal or absent mask.
// The reference materialises the (B,H,T,T) logits and probabilities in HBM and makes three
// passes over them; here they never leave the SM.
//
// One CTA owns two 128-row query tiles of one (batch, head) and walks the keys 128 at a time:
//   warps 0-15    softmax: all sixteen warps work on one query tile at a time, alternating between
//                 the two tiles.  Four threads share a row (warp w owns rows 32*(w%4).. and the
//                 32 key columns / quarter of the O columns number w/4), so a tile's softmax is
//                 short and four warps per scheduler keep the ex2 unit busy; the four threads
//                 exchange their maxima through shared memory once per tile.
//   warp 16       TMA producer (one lane)
//   warp 17       MMA issuer (one lane); owns the TMEM allocation
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P (bf16, packed two per
// column) overwrites the first columns of its S.  The MMA lane alternates between the two
// query tiles so one tile's softmax overlaps the other tile's products.  The running maximum
// used for the exponent is only raised when the true maximum has grown by more than 2^8, so
// the O accumulator in TMEM is rescaled rarely; the final division by the row sum makes the
// result exact regardless.
//
// Every wait on an mbarrier is bounded: after about a second without progress the waiting
// thread records where it gave up in a status word and the CTA drains and exits.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int NQT = 2;                 // query tiles per CTA
constexpr int WARP_TMA = NQT * 8;       // after the softmax warps (two warpgroups per query tile)
constexpr int WARP_MMA = NQT * 8 + 1;
constexpr int TC_THREADS = (NQT * 8 + 2) * 32;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

// ---------------------------------------------------------------------------------------------
// Shared-memory plan (all tiles 1024-byte aligned)
// ---------------------------------------------------------------------------------------------
template <int ROW_BYTES> struct Plan {                     // ROW_BYTES = head size x element size
  static constexpr int SUB = ROW_BYTES / 128;              // 128-byte sub-tiles per row
  static constexpr uint32_t SUB_BYTES = BLK * 128;         // one sub-tile: 128 rows x 128 bytes
  static constexpr uint32_t TILE_BYTES = SUB * SUB_BYTES;  // 128 rows of one tensor
  static constexpr int STAGES = 2;
  static constexpr uint32_t OFF_Q = 0;
  static constexpr uint32_t OFF_K = OFF_Q + NQT * TILE_BYTES;
  static constexpr uint32_t OFF_V = OFF_K + STAGES * TILE_BYTES;
  static constexpr uint32_t OFF_BAR = OFF_V + STAGES * TILE_BYTES;
  static constexpr uint32_t OFF_RED = OFF_BAR + 256;       // row-max / row-sum exchange: [2][4][128] floats
  static constexpr uint32_t BYTES = OFF_RED + 2 * 4 * 128 * 4 + 1024;  // + alignment slack
};

enum Bar : int {  // mbarrier indices
  BAR_Q_FULL = 0,    // [NQT]
  BAR_K_FULL = 2,    // [STAGES]
  BAR_K_EMPTY = 4,
  BAR_V_FULL = 6,
  BAR_V_EMPTY = 8,
  BAR_S_FULL = 10,   // [NQT]  S tile written by the MMA
  BAR_P_READY = 12,  // [NQT]  P written (and O rescaled) by the softmax warpgroup
  BAR_O_DONE = 14,   // [NQT]  P V product of the step finished
  BAR_DRAIN = 16,
  BAR_P_HALF = 17,   // [NQT]  first 64 key columns of P written
  BAR_RED = 19,      // all softmax threads have published their partial row maximum / sum
  BAR_COUNT = 20
};

// Optional timeline capture for tuning (compiled out unless MCA_TC_TRACE is defined): one CTA
// writes clock64 stamps of its softmax and MMA threads into a small global buffer.
#ifdef MCA_TC_TRACE
__device__ long long g_tc_trace[3 * 64 * 8];
__device__ long long g_tc_trace_w[16 * 64 * 4];  // per softmax warp, query tile 0: got S, local max done, exchange done, arrived
#define TC_TRACE_W(it, slot)                                                                              \
  do {                                                                                                   \
    if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && x == 0 && (it) < 64) g_tc_trace_w[(warp * 64 + (it)) * 4 + (slot)] = clock64(); \
  } while (0)
#define TC_TRACE(role, it, slot)                                                                         \
  do {                                                                                                   \
    if (trace_on && (it) < 64) g_tc_trace[((role) * 64 + (it)) * 8 + (slot)] = clock64();                \
  } while (0)
#else
#define TC_TRACE(role, it, slot) do { } while (0)
#define TC_TRACE_W(it, slot) do { } while (0)
#endif

struct TcParams {
  void* y;        // (B*H, T, HD) bf16
  float* lse;     // (B*H, T) or null: log2-domain log-sum-exp of the scaled logits
  int* status;
  int T, causal;
  float scale_log2;  // (1/sqrt(HD)) * log2(e)
};

// TF32 = false: bf16 tensors, kind::f16.  TF32 = true: fp32 tensors read as tf32 (kind::tf32),
// P handed to the second product as fp32 in place of S, fp32 output.
template <int HD, bool TF32>
__global__ void __launch_bounds__(TC_THREADS, 1)
sdpa_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const TcParams p) {
  constexpr int ELT = TF32 ? 4 : 2;            // bytes per element
  constexpr int BOX = 128 / ELT;               // elements per 128-byte sub-tile row
  using PL = Plan<HD * ELT>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar0 = smem_base + PL::OFF_BAR;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + PL::OFF_BAR + BAR_COUNT * 8);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y;
  const int T = p.T;
  // longest causal work first
  const int pair = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int q0 = pair * (NQT * BLK);
  int n_tiles[NQT];
#pragma unroll
  for (int x = 0; x < NQT; ++x) {
    const int qx = q0 + x * BLK;
    if (qx >= T) n_tiles[x] = 0;
    else n_tiles[x] = p.causal ? (min(qx + BLK, T) + BLK - 1) / BLK : (T + BLK - 1) / BLK;
  }
  const int n_max = max(n_tiles[0], n_tiles[1]);
#ifdef MCA_TC_TRACE
  const bool trace_on = (blockIdx.x == 0 && blockIdx.y == 0) && (lane == 0) && (warp == 0 || warp == WARP_MMA);
#endif

  // An earlier CTA already failed: leave before touching barriers or TMEM (uniform decision).
  __shared__ int s_abort;
  if (tid == 0) s_abort = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (s_abort != 0) return;

  if (tid == 0) {
    for (int i = 0; i < BAR_COUNT; ++i) {
      const bool softmax_bar = (i >= BAR_P_READY && i < BAR_P_READY + NQT) || (i >= BAR_P_HALF && i < BAR_P_HALF + NQT);
      mbar_init(bar(i), i == BAR_RED ? 16u : softmax_bar ? 8u : 1u);  // softmax warps arrive once per warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (warp == WARP_MMA) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == WARP_TMA) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
#pragma unroll
      for (int x = 0; x < NQT; ++x) {
        if (n_tiles[x] == 0) continue;
        mbar_expect_tx(bar(BAR_Q_FULL + x), PL::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < PL::SUB; ++s)
          tma_load_3d(smem_base + PL::OFF_Q + x * PL::TILE_BYTES + s * PL::SUB_BYTES, &map_q, bar(BAR_Q_FULL + x), s * BOX,
                      q0 + x * BLK, bh);
      }
      int issued_k = 0, issued_v = 0;
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        ok = mbar_wait(bar(BAR_K_EMPTY + st), ph ^ 1u, p.status, 10, j);
        if (!ok) break;
        mbar_expect_tx(bar(BAR_K_FULL + st), PL::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < PL::SUB; ++s)
          tma_load_3d(smem_base + PL::OFF_K + st * PL::TILE_BYTES + s * PL::SUB_BYTES, &map_k, bar(BAR_K_FULL + st), s * BOX,
                      j * BLK, bh);
        issued_k = j + 1;
        ok = mbar_wait(bar(BAR_V_EMPTY + st), ph ^ 1u, p.status, 11, j);
        if (!ok) break;
        mbar_expect_tx(bar(BAR_V_FULL + st), PL::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < PL::SUB; ++s)
          tma_load_3d(smem_base + PL::OFF_V + st * PL::TILE_BYTES + s * PL::SUB_BYTES, &map_v, bar(BAR_V_FULL + st), s * BOX,
                      j * BLK, bh);
        issued_v = j + 1;
      }
      if (!ok) {
        // give copies already in flight a bounded time to land before the CTA's memory is released
        for (int x = 0; x < NQT; ++x)
          if (n_tiles[x]) mbar_wait(bar(BAR_Q_FULL + x), 0, p.status, 12, x);
        for (int j = max(0, issued_k - 2); j < issued_k; ++j) mbar_wait(bar(BAR_K_FULL + (j & 1)), (uint32_t)((j >> 1) & 1), p.status, 13, j);
        for (int j = max(0, issued_v - 2); j < issued_v; ++j) mbar_wait(bar(BAR_V_FULL + (j & 1)), (uint32_t)((j >> 1) & 1), p.status, 14, j);
      }
    }
  } else if (warp == WARP_MMA) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = make_idesc_fmt(BLK, BLK, 0, 0, TF32 ? 2 : 1);
      constexpr uint32_t IDESC_PV = make_idesc_fmt(BLK, HD, 0, 1, TF32 ? 2 : 1);
      constexpr int KSTEPS_QK = HD * ELT / 32;   // 32 bytes of the head dimension per MMA
      constexpr int KSTEPS_PV = BLK * ELT / 32;  // 16 (bf16) or 8 (tf32) keys per MMA
      auto issue_qk = [&](int x, int st) {
        const uint32_t q_addr = smem_base + PL::OFF_Q + x * PL::TILE_BYTES;
        const uint32_t k_addr = smem_base + PL::OFF_K + st * PL::TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < KSTEPS_QK; ++kk) {
          const uint32_t off = (kk / 4) * PL::SUB_BYTES + (kk % 4) * 32;
          umma_ss_t<TF32>(tmem_base + x * BLK, make_desc(q_addr + off, 16, 1024), make_desc(k_addr + off, 16, 1024),
                          IDESC_QK, kk > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int x, int st, bool first, int half) {
        const uint32_t v_addr = smem_base + PL::OFF_V + st * PL::TILE_BYTES;
#pragma unroll
        for (int kk = half * (KSTEPS_PV / 2); kk < (half + 1) * (KSTEPS_PV / 2); ++kk) {
          // A: P rows in TMEM, 8 columns per step (16 bf16 or 8 tf32).  bf16 P of keys 32q..32q+31 sits in
          // the first 16 columns of quarter q of the S tile; tf32 P overwrites S column for column.
          // B: V, one step = 16 or 8 key rows of 128 bytes per sub-tile.
          const uint32_t a_col = TF32 ? (uint32_t)(kk * 8) : (uint32_t)((kk / 2) * 32 + (kk % 2) * 8);
          const uint64_t v_desc = TF32 ? make_desc_mn32(v_addr + kk * 1024, PL::SUB_BYTES, 512)
                                       : make_desc(v_addr + kk * 2048, PL::SUB_BYTES, 1024);
          umma_ts_t<TF32>(tmem_base + 2 * BLK + x * BLK, tmem_base + x * BLK + a_col, v_desc, IDESC_PV,
                          (first && kk == 0) ? 0u : 1u);
        }
      };
#pragma unroll
      for (int x = 0; x < NQT; ++x)
        if (n_tiles[x] && ok) ok = mbar_wait(bar(BAR_Q_FULL + x), 0, p.status, 20, x);
      if (ok && n_max > 0) {
        ok = mbar_wait(bar(BAR_K_FULL + 0), 0, p.status, 21, 0);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int x = 0; x < NQT; ++x) {
            if (n_tiles[x] > 0) { issue_qk(x, 0); umma_commit(bar(BAR_S_FULL + x)); }
          }
          umma_commit(bar(BAR_K_EMPTY + 0));
        }
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j & 1, st_n = (j + 1) & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1), ph_n = (uint32_t)(((j + 1) >> 1) & 1);
        ok = mbar_wait(bar(BAR_V_FULL + st), ph, p.status, 22, j);
        if (!ok) break;
        bool k_next_ready = false;
#pragma unroll
        for (int x = 0; x < NQT; ++x) {
          if (j < n_tiles[x]) {
            TC_TRACE(2, j, x * 4 + 0);
            ok = mbar_wait(bar(BAR_P_HALF + x), (uint32_t)(j & 1), p.status, 28 + x, j);
            if (!ok) break;
            TC_TRACE(2, j, x * 4 + 1);
            tc_fence_after();
            issue_pv(x, st, j == 0, 0);
            ok = mbar_wait(bar(BAR_P_READY + x), (uint32_t)(j & 1), p.status, 23 + x, j);
            if (!ok) break;
            TC_TRACE(2, j, x * 4 + 3);
            tc_fence_after();
            issue_pv(x, st, j == 0, 1);
            umma_commit(bar(BAR_O_DONE + x));
          }
          if (x == NQT - 1) umma_commit(bar(BAR_V_EMPTY + st));
          if (j + 1 < n_tiles[x]) {
            if (!k_next_ready) {
              ok = mbar_wait(bar(BAR_K_FULL + st_n), ph_n, p.status, 25, j);
              if (!ok) break;
              tc_fence_after();
              k_next_ready = true;
            }
            issue_qk(x, st_n);
            umma_commit(bar(BAR_S_FULL + x));
            TC_TRACE(2, j, x * 4 + 2);
          }
          if (x == NQT - 1 && j + 1 < n_max) {
            if (!k_next_ready) {  // no query tile needs this K tile any more (cannot happen for n_max), keep the ring moving
              ok = mbar_wait(bar(BAR_K_FULL + st_n), ph_n, p.status, 26, j);
              if (!ok) break;
            }
            umma_commit(bar(BAR_K_EMPTY + st_n));
          }
        }
      }
      // all products issued: wait (bounded) until the tensor pipe is idle before TMEM is freed
      umma_commit(bar(BAR_DRAIN));
      mbar_wait(bar(BAR_DRAIN), 0, p.status, 27, 0);
    }
  } else if (warp < WARP_TMA) {
    // ------------------------------------------------------------------ softmax warps
    const int qtr = warp >> 2;                     // which 32 keys of each tile / which quarter of the O columns
    const int lane_base = (warp & 3) * 32;         // TMEM lanes this warp may touch
    const int row = lane_base + lane;              // row within the tile
    constexpr int OC = HD / 4;                     // O columns per thread
    const uint32_t t_row = tmem_base + ((uint32_t)lane_base << 16);
    float* red = reinterpret_cast<float*>(smem_gen + PL::OFF_RED);
    auto red_at = [&](int parity, int q) { return red + (parity * 4 + q) * 128 + row; };
    uint32_t red_cnt = 0;                          // exchanges done so far (parity of the BAR_RED phase)
    float m_used[NQT], l[NQT];
#pragma unroll
    for (int x = 0; x < NQT; ++x) { m_used[x] = -INFINITY; l[x] = 0.f; }
    for (int j = 0; j < n_max && ok; ++j) {
#pragma unroll
      for (int x = 0; x < NQT; ++x) {
        if (j >= n_tiles[x] || !ok) continue;
        const int qi = q0 + x * BLK + row;
        const uint32_t t_s = t_row + (uint32_t)(x * BLK + qtr * 32);
        const uint32_t t_o = t_row + (uint32_t)(2 * BLK + x * BLK + qtr * OC);
        TC_TRACE(x, j, 0);
        ok = __all_sync(0xffffffffu, mbar_wait_hot(bar(BAR_S_FULL + x), (uint32_t)(j & 1), p.status, 30 + x, j));
        if (!ok) break;
        TC_TRACE(x, j, 1);
        TC_TRACE_W(j, 0);
        tc_fence_after();
        uint32_t s[32];
        tmem_ld32(t_s, s);
        tmem_wait_ld();
        TC_TRACE(x, j, 2);
        const int k0 = j * BLK + qtr * 32;
        // Only the diagonal tile (causal) and the last tile (keys beyond T) need masking.
        if ((p.causal && j * BLK + BLK - 1 > q0 + x * BLK) || (j * BLK + BLK > T)) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kj = k0 + i;
            if (kj >= T || (p.causal && kj > qi)) s[i] = 0xff800000u;  // -inf
          }
        }
        // maximum of this thread's 32 raw logits, then of the four threads of the row
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          mx4[0] = max3(mx4[0], __uint_as_float(s[i + 0]), __uint_as_float(s[i + 1]));
          mx4[1] = max3(mx4[1], __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
          mx4[2] = max3(mx4[2], __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
          mx4[3] = max3(mx4[3], __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
        }
        const int par = (int)(red_cnt & 1u);
        *red_at(par, qtr) = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        __syncwarp();
        TC_TRACE_W(j, 1);
        if (lane == 0) mbar_arrive(bar(BAR_RED));
        // p = 2^(s * scale_log2 - m): one FFMA and one exponential per element, packed to bf16;
        // the row sum is taken in fp32.
        uint32_t pk[16];
        float rs;
        auto exp_tile = [&](float neg_m) {
          float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float p0 = exp2_sel(fmaf(__uint_as_float(s[i + 0]), p.scale_log2, neg_m), i + 0);
            const float p1 = exp2_sel(fmaf(__uint_as_float(s[i + 1]), p.scale_log2, neg_m), i + 1);
            const float p2 = exp2_sel(fmaf(__uint_as_float(s[i + 2]), p.scale_log2, neg_m), i + 2);
            const float p3 = exp2_sel(fmaf(__uint_as_float(s[i + 3]), p.scale_log2, neg_m), i + 3);
            if constexpr (TF32) {
              s[i + 0] = __float_as_uint(p0); s[i + 1] = __float_as_uint(p1);
              s[i + 2] = __float_as_uint(p2); s[i + 3] = __float_as_uint(p3);
            } else {
              pk[i / 2] = pack_bf16(p0, p1);
              pk[i / 2 + 1] = pack_bf16(p2, p3);
            }
            rs4[0] += p0; rs4[1] += p1; rs4[2] += p2; rs4[3] += p3;
          }
          rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
        };
        ok = __all_sync(0xffffffffu, mbar_wait_hot(bar(BAR_RED), red_cnt & 1u, p.status, 36, j));
        if (!ok) break;
        TC_TRACE_W(j, 2);
        ++red_cnt;
        const float mx = fmaxf(fmaxf(*red_at(par, 0), *red_at(par, 1)), fmaxf(*red_at(par, 2), *red_at(par, 3))) * p.scale_log2;
        float m_new = m_used[x];
        bool raise = false;
        if (mx > m_used[x] + RESCALE_THRESHOLD || j == 0) { m_new = fmaxf(mx, m_used[x]); raise = (j > 0); }
        if (m_new == -INFINITY) m_new = 0.f;  // a row with no visible key yet (rows beyond T)
        if (__any_sync(0xffffffffu, raise)) {
          // rescale this thread's quarter of O in TMEM: the previous P V product must have finished
          ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_O_DONE + x), (uint32_t)((j - 1) & 1), p.status, 32 + x, j));
          if (!ok) break;
          tc_fence_after();
          const float f = raise ? fast_exp2(m_used[x] - m_new) : 1.0f;
#pragma unroll
          for (int c = 0; c < OC / 16; ++c) {
            uint32_t o[16];
            tmem_ld16(t_o + c * 16, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tmem_st16(t_o + c * 16, o);
          }
          l[x] *= f;
        }
        exp_tile(-m_new);
        m_used[x] = m_new;
        TC_TRACE(x, j, 3);
        if constexpr (TF32) tmem_st32(t_s, s);
        else tmem_st16(t_s, pk);
        l[x] += rs;
        TC_TRACE(x, j, 4);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar((qtr < 2 ? BAR_P_HALF : BAR_P_READY) + x));
        TC_TRACE(x, j, 5);
        TC_TRACE_W(j, 3);
      }
    }
    // epilogue: row sums of the four threads, then O / l -> bf16 -> global
#pragma unroll
    for (int x = 0; x < NQT; ++x) {
      const int n = n_tiles[x];
      if (!ok || n == 0) continue;
      const int qi = q0 + x * BLK + row;
      const uint32_t t_o = t_row + (uint32_t)(2 * BLK + x * BLK + qtr * OC);
      const int par = (int)(red_cnt & 1u);
      *red_at(par, qtr) = l[x];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_RED));
      ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_RED), red_cnt & 1u, p.status, 37, x));
      if (!ok) break;
      ++red_cnt;
      const float lsum = (*red_at(par, 0) + *red_at(par, 1)) + (*red_at(par, 2) + *red_at(par, 3));
      ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_O_DONE + x), (uint32_t)((n - 1) & 1), p.status, 34 + x, n));
      if (!ok) break;
      tc_fence_after();
      const float inv = 1.0f / lsum;
      __nv_bfloat16* yrow = reinterpret_cast<__nv_bfloat16*>(p.y) + ((int64_t)bh * T + qi) * HD + qtr * OC;
      float* yrow_f = reinterpret_cast<float*>(p.y) + ((int64_t)bh * T + qi) * HD + qtr * OC;
#pragma unroll
      for (int c = 0; c < OC / 16; ++c) {
        uint32_t o[16];
        tmem_ld16(t_o + c * 16, o);
        tmem_wait_ld();
        if constexpr (TF32) {
          if (qi < T) {
#pragma unroll
            for (int i = 0; i < 16; i += 4)
              *reinterpret_cast<float4*>(yrow_f + c * 16 + i) =
                  make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv, __uint_as_float(o[i + 2]) * inv,
                              __uint_as_float(o[i + 3]) * inv);
          }
        } else if (qi < T) {
#pragma unroll
          for (int i = 0; i < 16; i += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(o[i + 0]) * inv, __uint_as_float(o[i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(yrow + c * 16 + i) = w;
          }
        }
      }
      if (qtr == 0 && p.lse != nullptr && qi < T) p.lse[(int64_t)bh * T + qi] = m_used[x] + log2f(lsum);
    }
  }
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


template <int HD, bool TF32>
int launch_tc(const void* q, const void* k, const void* v, int causal, int B, int H, int T, void* y, float* lse,
              int* status, cudaStream_t st) {
  CUtensorMap mq, mk, mv;
  int e;
  if constexpr (TF32) {
    if ((e = make_map_f32(&mq, q, B * H, T, HD)) || (e = make_map_f32(&mk, k, B * H, T, HD)) ||
        (e = make_map_f32(&mv, v, B * H, T, HD, true)))
      return e;
  } else {
    if ((e = make_map_bf16(&mq, q, B * H, T, HD)) || (e = make_map_bf16(&mk, k, B * H, T, HD)) ||
        (e = make_map_bf16(&mv, v, B * H, T, HD)))
      return e;
  }
  TcParams p;
  p.y = y; p.lse = lse; p.status = status; p.T = T; p.causal = causal;
  p.scale_log2 = (1.0f / sqrtf((float)HD)) * 1.4426950408889634f;
  const size_t smem = Plan<HD * (TF32 ? 4 : 2)>::BYTES;
  MCA_CUDA_TRY(cudaFuncSetAttribute(sdpa_fwd_tc_kernel<HD, TF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(mca_ceil_div(T, NQT * BLK), B * H);
  sdpa_fwd_tc_kernel<HD, TF32><<<grid, TC_THREADS, smem, st>>>(mq, mk, mv, p);
  return mca_launch_status();
}

}  // namespace

#ifdef MCA_TC_TRACE
extern "C" __attribute__((visibility("default"))) int mca_tc_trace_fetch(long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, g_tc_trace, sizeof(long long) * count);
}
extern "C" __attribute__((visibility("default"))) int mca_tc_trace_fetch_w(long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, g_tc_trace_w, sizeof(long long) * count);
}
#endif

int mca_sdpa_forward_tc(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H, int T, int D,
                        void* y, float* lse, int* status, void* stream) {
  if (!q || !k || !v || !y || !status) return ERROR_PARAM_NULL;
  if (B <= 0 || H <= 0 || T <= 0 || (int64_t)B * H > 65535) return ERROR_PARAM_OUT_OF_RANGE;
  if (dtype != MCA_DTYPE_BF16 && dtype != MCA_DTYPE_TF32) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(y)) & 15)
    return ERROR_PARAM_OUT_OF_RANGE;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == MCA_DTYPE_TF32) {
    // fp32 rows are twice as wide: only the 64-wide head fits the shared-memory plan (two query tiles,
    // two K/V stages); wider heads use the exact fp32 kernel
    if (D == 64) return launch_tc<64, true>(q, k, v, causal, B, H, T, y, lse, status, st);
    return ERROR_ATTN_UNSUPPORTED_SHAPE;
  }
  if (D == 128) return launch_tc<128, false>(q, k, v, causal, B, H, T, y, lse, status, st);
  if (D == 64) return launch_tc<64, false>(q, k, v, causal, B, H, T, y, lse, status, st);
  return ERROR_ATTN_UNSUPPORTED_SHAPE;
}

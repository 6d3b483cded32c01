// Fused flash-style attention forward on the 5th-generation tensor cores (sm_100a):
// S = Q K^T by tcgen05.mma into TMEM, online softmax by two groups of eight warps that read S from TMEM
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
//   warps 0-7     softmax of query tile 0, warps 8-15 of query tile 1.  A warp reads 16 rows x
//                 128 keys of S in the 16-lane quad layout (four threads per row), so the row
//                 maximum and sum are two shuffles, no shared memory and no barrier; the two
//                 groups run independently, one tile's exponentials over the other's loads.
//   warp 16       TMA producer (one lane)
//   warp 17       MMA issuer: the warp runs in lock step and one elected lane issues, so that
//                 descriptors are warp-uniform values (the issuing thread's instruction count per
//                 tcgen05.mma bounds the tensor rate when it shares a scheduler with four busy
//                 softmax warps); owns the TMEM allocation
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P (bf16, packed two per
// column) overwrites the first columns of its S.  The MMA lane alternates between the two
// query tiles so one tile's softmax overlaps the other tile's products.  The running maximum
// used for the exponent is only raised when the true maximum has grown by more than 2^8, so
// the O accumulator in TMEM is rescaled rarely; the final division by the row sum makes the
// result exact regardless.
//
// Every wait on an mbarrier is bounded: after about a second without progress the waiting
// thread records where it gave up in a status word and the CTA drains and exits.
//
// Three operand modes share the kernel:
//   MODE_BF16   bf16 tensors, one kind::f16 product per contraction.
//   MODE_TF32   fp32 tensors read as tf32 (kind::tf32), 64-wide heads.
//   MODE_SPLIT  fp32 callers at fp32 accuracy: every operand x is carried as two fp16 values hi = fp16(x),
//               lo = fp16(x - hi) (22 mantissa bits together; a pre-pass writes rows [hi | lo] after scaling each
//               tensor by a power of two so that neither half leaves the fp16 range), and every contraction is three
//               kind::f16 products hi.hi + hi.lo + lo.hi accumulated in the same fp32 TMEM tile.  P is split the
//               same way by the softmax warps.  Measured against the fp64 oracle this is within 1e-5 of the output
//               scale (what limits it is the fp32 accumulation inside the tensor core, not the operands), at a third of
//               the bf16 tensor rate.
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

#include "tc_common.cuh"
#include "split_prepass.cuh"

namespace {

using namespace tc;

constexpr int NQT = 2;                 // query tiles per CTA, at most
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units
constexpr int MODE_BF16 = 0, MODE_TF32 = 1, MODE_SPLIT = 2;

// ---------------------------------------------------------------------------------------------
// Shared-memory plan (all tiles 1024-byte aligned)
// ---------------------------------------------------------------------------------------------
// QT query tiles of a CTA are in use (the second group of softmax warps idles when QT is 1) and K and V each have STG
// stages.  Rows of 512 bytes (128-wide heads with split operands) leave room for one query tile and one stage: K(j+1)
// then arrives while P V(j) runs and V(j+1) while S(j+1) does, which is the order the products need them in anyway.
template <int ROW_BYTES, int QT = 2, int STG = 2> struct Plan {   // ROW_BYTES = head size x element size
  static constexpr int SUB = ROW_BYTES / 128;              // 128-byte sub-tiles per row
  static constexpr uint32_t SUB_BYTES = BLK * 128;         // one sub-tile: 128 rows x 128 bytes
  static constexpr uint32_t TILE_BYTES = SUB * SUB_BYTES;  // 128 rows of one tensor
  static constexpr int STAGES = STG;
  static constexpr uint32_t OFF_Q = 0;
  static constexpr uint32_t OFF_K = OFF_Q + QT * TILE_BYTES;
  static constexpr uint32_t OFF_V = OFF_K + STAGES * TILE_BYTES;
  static constexpr uint32_t OFF_BAR = OFF_V + STAGES * TILE_BYTES;
  static constexpr uint32_t OFF_RED = OFF_BAR + 256;       // row sums and maxima for the epilogue: [NQT][2][128] floats
  static constexpr uint32_t BYTES = OFF_RED + 2 * 4 * 128 * 4 + 1024;  // + alignment slack
};

// What a CTA of the kernel looks like for a head size, an operand mode and the NARROW choice of the launcher.
//   two query tiles (the default): 16 softmax warps + TMA + MMA warps, one CTA per SM, all 512 TMEM columns;
//   WIDE (512-byte split rows): one query tile, single-stage K and V, one CTA per SM;
//   NARROW: one query tile and a shared-memory plan of under 110 KB, so that two CTAs share an SM: each one's set-up,
//           first loads and epilogue overlap the other's key loop.  For short sequences, where a CTA walks only a few
//           key tiles and that fixed part is a third of its life; K and V are then read from L2 once per query tile
//           instead of once per pair, which long sequences would pay for.
template <int HD, int MODE, bool NARROW> struct Shape {
  static constexpr int ROW_BYTES = MODE == MODE_SPLIT ? 2 * split::row_halves(HD) : HD * (MODE == MODE_TF32 ? 4 : 2);
  static constexpr bool WIDE = ROW_BYTES > 256;
  static_assert(!(WIDE && NARROW), "a wide CTA is already a single query tile");
  static constexpr int QT = (WIDE || NARROW) ? 1 : 2;
  static constexpr int STG = WIDE ? 1 : (NARROW ? (ROW_BYTES <= 128 ? 2 : 1) : 2);
  using PL = Plan<ROW_BYTES, QT, STG>;
  static constexpr int WARP_TMA = QT * 8;          // after the softmax warps (eight per query tile)
  static constexpr int WARP_MMA = QT * 8 + 1;
  static constexpr int THREADS = (QT * 8 + 2) * 32;
  static constexpr int CTAS_PER_SM = NARROW ? 2 : 1;
  static constexpr uint32_t TMEM_COLS = QT == 1 ? 256 : 512;   // S tiles in [0, QT x 128), O tiles behind them
  static_assert(CTAS_PER_SM * (PL::BYTES + 1024) <= 227 * 1024, "shared memory of the CTAs of one SM");
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
  BAR_RED = 19,      // [NQT]  the group's row sums are in shared memory (epilogue)
  BAR_COUNT = 21
};

// Optional timeline capture for tuning (compiled out unless MCA_TC_TRACE is defined): one CTA
// writes clock64 stamps of its softmax and MMA threads into a small global buffer.
#ifdef MCA_TC_TRACE
__device__ long long g_tc_trace[4 * 64 * 8];
__device__ long long g_tc_trace_w[16 * 64 * 4];  // per softmax warp, query tile 0: got S, local max done, exchange done, arrived
__device__ long long g_tc_phase[16];   // whole-CTA phases of block (0,0): entry, set-up, first loads, loop, epilogue, exit
#define TC_PHASE(i, who)                                                                                 \
  do {                                                                                                   \
    if (blockIdx.x == 0 && blockIdx.y == 0 && (who)) g_tc_phase[i] = clock64();                          \
  } while (0)
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
#define TC_PHASE(i, who) do { } while (0)
#endif

struct TcParams {
  void* y;        // (B*H, T, HD) bf16
  float* lse;     // (B*H, T) or null: log2-domain log-sum-exp of the scaled logits
  int* status;
  int T, causal, H;
  int group;         // (batch, head) pairs whose CTAs are interleaved longest-first (their K, V fit in L2 together)
  float scale_log2;  // (1/sqrt(HD)) * log2(e)
  McaStrides ys;     // element strides of the output view
  void* y_more[7];   // further destinations of the same bf16 output tile (peer GPUs' buffers), same strides
  int n_more;
  // MODE_SPLIT: the pre-pass's scale factors (split::SplitFac, device memory); exact softmax statistics for
  // the fp32 backward: row_max in natural-log units of the scaled logits and the matching row sum, (B*H, T) each
  const float* split_fac;
  float* row_max;
  float* row_sum;
  float* y_copy;      // second copy of the fp32 output, (B*H, T, HD) contiguous, or null
  // MASKED: keep-bits of the caller's mask, one bit per (row, key), rows padded to whole 128-key tiles; the words of
  // query row r, batch item b and key tile j start at mask_bits + b * mask_batch_stride + r * mask_row_stride + 4 j
  // (a (B,T) key mask has row stride 0, a (T,T) mask batch stride 0)
  const uint32_t* mask_bits;
  int64_t mask_batch_stride, mask_row_stride;
};

// The logit a masked entry is given, in the log2 domain of the softmax.  The reference writes -1e29 over the scaled
// logit (attn.cu:302-311, math.cu mask kernels): any finite value far below every real logit gives the same result --
// probability exactly 0 next to an unmasked key, a uniform row when every key is masked.  2^17 keeps the product
// masked_logit x scale exact to 2^-7, so that the exponent of a fully masked row is 0 +- 0.01.
constexpr float MASKED_LOG2 = -131072.0f;

// MODE_TF32: P is handed to the second product as fp32 in place of S; MODE_TF32 and MODE_SPLIT write fp32 output.
template <int HD, int MODE, bool MASKED, bool NARROW>
__global__ void __launch_bounds__((Shape<HD, MODE, NARROW>::THREADS), (Shape<HD, MODE, NARROW>::CTAS_PER_SM))
sdpa_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const TcParams p) {
  constexpr bool TF32 = MODE == MODE_TF32;
  constexpr bool SPLIT = MODE == MODE_SPLIT;
  constexpr bool F32_OUT = TF32 || SPLIT;
  constexpr int ELT = TF32 ? 4 : 2;            // bytes per element
  constexpr int BOX = 128 / ELT;               // elements per 128-byte sub-tile row
  // split rows are [hi (64 fp16, HD used) | lo (64 fp16, HD used)]: two 128-byte sub-tiles for head sizes up to 64;
  // 128-wide heads have [hi (128) | lo (128)], four sub-tiles, one query tile per CTA and single-stage K and V
  using SH = Shape<HD, MODE, NARROW>;
  using PL = typename SH::PL;
  constexpr int QT = SH::QT, STG = SH::STG;
  constexpr int WARP_TMA = SH::WARP_TMA, WARP_MMA = SH::WARP_MMA;
  constexpr uint32_t TMEM_COLS = SH::TMEM_COLS;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar0 = smem_base + PL::OFF_BAR;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + PL::OFF_BAR + BAR_COUNT * 8);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Launch order -> work item.  Causal work per CTA grows with the query position, so CTAs are handed out
  // longest first; to keep that order across heads without losing the L2 reuse of K and V, the heads are taken in
  // groups of p.group whose K and V fit in L2 together, and inside a group the order is (work rank, head).
  const int lin = (int)(blockIdx.y * gridDim.x + blockIdx.x);
  const int grp = lin / (p.group * (int)gridDim.x);
  const int in_grp = lin - grp * p.group * (int)gridDim.x;
  const int grp_heads = min(p.group, (int)gridDim.y - grp * p.group);
  const int rank = in_grp / grp_heads;
  const int bh = grp * p.group + (in_grp - rank * grp_heads);
  const int bi = bh / p.H, hi = bh - bi * p.H;   // batch item and head
  const int T = p.T;
  const int pair = (int)gridDim.x - 1 - rank;
  const int q0 = pair * (QT * BLK);
  int n_tiles[NQT];
#pragma unroll
  for (int x = 0; x < NQT; ++x) {
    const int qx = q0 + x * BLK;
    if (qx >= T || x >= QT) n_tiles[x] = 0;
    else n_tiles[x] = p.causal ? (min(qx + BLK, T) + BLK - 1) / BLK : (T + BLK - 1) / BLK;
  }
  const int n_max = max(n_tiles[0], n_tiles[1]);
#ifdef MCA_TC_TRACE
  const bool trace_on = (blockIdx.x == 0 && blockIdx.y == 0) && (lane == 0) && (warp == 0 || warp == 8 || warp == WARP_MMA);
#endif

  // Set-up, each part by another warp so that their latencies overlap: the status word of the launch (has an
  // earlier CTA failed?), the barriers, the tensor maps' descriptors, the TMEM allocation.
  __shared__ int s_abort;
  TC_PHASE(0, tid == 0);
  mca_pdl_launch_dependents();   // a kernel launched behind this one may set itself up as this one's CTAs leave
  if (tid == 32) s_abort = *reinterpret_cast<volatile int*>(p.status);
  if (warp == WARP_TMA && lane == 0) {
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (tid == 0) {
    for (int i = 0; i < BAR_COUNT; ++i) {
      const bool softmax_bar = (i >= BAR_P_READY && i < BAR_P_READY + NQT) || (i >= BAR_P_HALF && i < BAR_P_HALF + NQT);
      mbar_init(bar(i), (softmax_bar || i >= BAR_RED) ? 8u : 1u);  // the eight warps of a group arrive once per warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == WARP_MMA) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  mca_pdl_wait();   // launched ahead of the kernels before it: from here on their results are complete and visible
  if (s_abort != 0) {   // an earlier CTA already failed: leave (uniform decision) before any copy or product is issued
    if (warp == WARP_MMA) tmem_dealloc(tmem_base, TMEM_COLS);
    return;
  }
  bool ok = true;
  TC_PHASE(2, tid == 0);

  if (warp == WARP_TMA) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
#pragma unroll
      for (int x = 0; x < NQT; ++x) {
        if (n_tiles[x] == 0) continue;
        mbar_expect_tx(bar(BAR_Q_FULL + x), PL::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < PL::SUB; ++s)
          tma_load_4d(smem_base + PL::OFF_Q + x * PL::TILE_BYTES + s * PL::SUB_BYTES, &map_q, bar(BAR_Q_FULL + x), s * BOX,
                      q0 + x * BLK, hi, bi);
      }
      int issued_k = 0, issued_v = 0;
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j % STG;
        const uint32_t ph = (uint32_t)((j / STG) & 1);
        ok = mbar_wait(bar(BAR_K_EMPTY + st), ph ^ 1u, p.status, 10, j);
        if (!ok) break;
        mbar_expect_tx(bar(BAR_K_FULL + st), PL::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < PL::SUB; ++s)
          tma_load_4d(smem_base + PL::OFF_K + st * PL::TILE_BYTES + s * PL::SUB_BYTES, &map_k, bar(BAR_K_FULL + st), s * BOX,
                      j * BLK, hi, bi);
        issued_k = j + 1;
        if (j == 0) TC_PHASE(3, true);
        ok = mbar_wait(bar(BAR_V_EMPTY + st), ph ^ 1u, p.status, 11, j);
        if (!ok) break;
        mbar_expect_tx(bar(BAR_V_FULL + st), PL::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < PL::SUB; ++s)
          tma_load_4d(smem_base + PL::OFF_V + st * PL::TILE_BYTES + s * PL::SUB_BYTES, &map_v, bar(BAR_V_FULL + st), s * BOX,
                      j * BLK, hi, bi);
        issued_v = j + 1;
      }
      if (!ok) {
        // give copies already in flight a bounded time to land before the CTA's memory is released
        for (int x = 0; x < NQT; ++x)
          if (n_tiles[x]) mbar_wait(bar(BAR_Q_FULL + x), 0, p.status, 12, x);
        for (int j = max(0, issued_k - STG); j < issued_k; ++j) mbar_wait(bar(BAR_K_FULL + (j % STG)), (uint32_t)((j / STG) & 1), p.status, 13, j);
        for (int j = max(0, issued_v - STG); j < issued_v; ++j) mbar_wait(bar(BAR_V_FULL + (j % STG)), (uint32_t)((j / STG) & 1), p.status, 14, j);
      }
    }
  } else if (warp == WARP_MMA) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs this role in lock step and one elected lane issues the tcgen05
    // instructions: addresses and descriptors are then warp-uniform values, which keeps the
    // per-instruction overhead of the issuing thread small.
    {
      const uint32_t leader = elect_one() ? 1u : 0u;
      const uint32_t tmem_base_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr int FMT = TF32 ? 2 : (SPLIT ? 0 : 1);      // operand format of the instruction descriptor: tf32, fp16, bf16
      constexpr uint32_t IDESC_QK = make_idesc_fmt(BLK, BLK, 0, 0, FMT);
      constexpr uint32_t IDESC_PV = make_idesc_fmt(BLK, HD, 0, 1, FMT);
      constexpr int KSTEPS_QK = HD * ELT / 32;   // 32 bytes of the head dimension per MMA (per half in split mode)
      constexpr int KSTEPS_PV = BLK * ELT / 32;  // 16 (bf16, fp16) or 8 (tf32) keys per MMA
      // A descriptor's start-address field (bits 0-13, in 16-byte units) never carries for offsets
      // inside the CTA's shared memory, so stepping a tile is an add on the low word.
      const uint64_t desc_q0 = make_desc(smem_base + PL::OFF_Q, 16, 1024);
      const uint64_t desc_k0 = make_desc(smem_base + PL::OFF_K, 16, 1024);
      const uint64_t desc_v0 = TF32 ? make_desc_mn32(smem_base + PL::OFF_V, PL::SUB_BYTES, 512)
                                    : make_desc(smem_base + PL::OFF_V, PL::SUB_BYTES, 1024);
      constexpr uint32_t V_STEP = (TF32 ? 1024u : 2048u) >> 4;  // one MMA's key rows of V
      auto commit_by_leader = [&](uint32_t b) { umma_commit_if(leader, b); };
      auto issue_qk = [&](int x, int st) {
        const uint64_t dq = desc_q0 + (uint64_t)((x * PL::TILE_BYTES) >> 4);
        const uint64_t dk = desc_k0 + (uint64_t)((st * PL::TILE_BYTES) >> 4);
        const uint32_t d_tmem = tmem_base_u + x * BLK;
        if constexpr (SPLIT) {
          // S = Qhi Khi^T + Qhi Klo^T + Qlo Khi^T: the halves are the sub-tiles [0, SUB/2) and [SUB/2, SUB) of a row
          constexpr uint32_t LO = ((PL::SUB / 2) * PL::SUB_BYTES) >> 4;
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            const uint32_t oq = term == 2 ? LO : 0u, ok_ = term == 1 ? LO : 0u;
#pragma unroll
            for (int kk = 0; kk < KSTEPS_QK; ++kk) {
              const uint32_t off = ((uint32_t)(kk >> 2) * PL::SUB_BYTES + (uint32_t)(kk & 3) * 32u) >> 4;
              umma_ss_if<false>(leader, d_tmem, dq + oq + off, dk + ok_ + off, IDESC_QK, (term > 0 || kk > 0) ? 1u : 0u);
            }
          }
        } else {
#pragma unroll
          for (int kk = 0; kk < KSTEPS_QK; ++kk) {
            const uint32_t off = ((uint32_t)(kk >> 2) * PL::SUB_BYTES + (uint32_t)(kk & 3) * 32u) >> 4;
            umma_ss_if<TF32>(leader, d_tmem, dq + off, dk + off, IDESC_QK, kk > 0 ? 1u : 0u);
          }
        }
      };
      auto issue_pv = [&](int x, int st, bool first, int half) {
        // A: P rows in TMEM, 8 columns per step (16 bf16 or 8 tf32).  bf16 P is packed two keys per column
        // into the first 64 columns of the S tile; tf32 P overwrites S column for column.
        // B: V, one step = 16 or 8 key rows of 128 bytes per sub-tile.
        const uint64_t dv = desc_v0 + (uint64_t)((st * PL::TILE_BYTES) >> 4);
        const uint32_t d_tmem = tmem_base_u + QT * BLK + x * BLK;
        const uint32_t a_tmem = tmem_base_u + x * BLK;
#pragma unroll
        for (int kk = half * (KSTEPS_PV / 2); kk < (half + 1) * (KSTEPS_PV / 2); ++kk) {
          if constexpr (SPLIT) {
            // O += Phi Vhi + Phi Vlo + Plo Vhi: Phi in columns [0,64) of the S region, Plo in [64,128)
            const uint64_t dvk = dv + (uint64_t)((uint32_t)kk * V_STEP);
            const uint32_t a_hi = a_tmem + (uint32_t)(kk * 8);
            umma_ts_if<false>(leader, d_tmem, a_hi, dvk, IDESC_PV, (first && kk == 0) ? 0u : 1u);
            umma_ts_if<false>(leader, d_tmem, a_hi, dvk + (uint64_t)(((PL::SUB / 2) * PL::SUB_BYTES) >> 4), IDESC_PV, 1u);
            umma_ts_if<false>(leader, d_tmem, a_hi + 64u, dvk, IDESC_PV, 1u);
          } else {
            umma_ts_if<TF32>(leader, d_tmem, a_tmem + (uint32_t)(kk * 8), dv + (uint64_t)((uint32_t)kk * V_STEP), IDESC_PV,
                             (first && kk == 0) ? 0u : 1u);
          }
        }
      };
#pragma unroll
      for (int x = 0; x < NQT; ++x)
        if (n_tiles[x] && ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_Q_FULL + x), 0, p.status, 20, x));
      TC_PHASE(4, lane == 0);
      if (ok && n_max > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_K_FULL + 0), 0, p.status, 21, 0));
        TC_PHASE(5, lane == 0);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int x = 0; x < NQT; ++x) {
            if (n_tiles[x] > 0) { issue_qk(x, 0); commit_by_leader(bar(BAR_S_FULL + x)); }
          }
          commit_by_leader(bar(BAR_K_EMPTY + 0));
        }
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j % STG, st_n = (j + 1) % STG;
        const uint32_t ph = (uint32_t)((j / STG) & 1), ph_n = (uint32_t)(((j + 1) / STG) & 1);
        TC_TRACE(3, j, 0);
        ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_V_FULL + st), ph, p.status, 22, j));
        if (!ok) break;
        TC_TRACE(3, j, 1);
        bool k_next_ready = false;
#pragma unroll
        for (int x = 0; x < NQT; ++x) {
          if (j < n_tiles[x]) {
            TC_TRACE(2, j, x * 4 + 0);
            ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_P_HALF + x), (uint32_t)(j & 1), p.status, 28 + x, j));
            if (!ok) break;
            TC_TRACE(2, j, x * 4 + 1);
            tc_fence_after();
            issue_pv(x, st, j == 0, 0);
            ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_P_READY + x), (uint32_t)(j & 1), p.status, 23 + x, j));
            if (!ok) break;
            TC_TRACE(2, j, x * 4 + 3);
            tc_fence_after();
            issue_pv(x, st, j == 0, 1);
            TC_TRACE(3, j, 4 + x);
            commit_by_leader(bar(BAR_O_DONE + x));
          }
          if (x == NQT - 1) commit_by_leader(bar(BAR_V_EMPTY + st));
          if (j + 1 < n_tiles[x]) {
            if (!k_next_ready) {
              TC_TRACE(3, j, 2);
              ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_K_FULL + st_n), ph_n, p.status, 25, j));
              if (!ok) break;
              TC_TRACE(3, j, 3);
              tc_fence_after();
              k_next_ready = true;
            }
            issue_qk(x, st_n);
            commit_by_leader(bar(BAR_S_FULL + x));
            TC_TRACE(2, j, x * 4 + 2);
          }
          if (x == NQT - 1 && j + 1 < n_max) {
            if (!k_next_ready) {  // no query tile needs this K tile any more (cannot happen for n_max), keep the ring moving
              ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_K_FULL + st_n), ph_n, p.status, 26, j));
              if (!ok) break;
            }
            commit_by_leader(bar(BAR_K_EMPTY + st_n));
          }
        }
      }
      // all products issued: wait (bounded) until the tensor pipe is idle before TMEM is freed
      commit_by_leader(bar(BAR_DRAIN));
      mbar_wait(bar(BAR_DRAIN), 0, p.status, 27, 0);
      __syncwarp();
    }
  } else if (warp < WARP_TMA) {
    // ------------------------------------------------------------------ softmax warps
    // Group x = warp / 8 owns query tile x.  A warp covers 16 rows x all 128 keys in the quad
    // layout (four threads per row, rows r0 and r0 + 8 per thread), so row maxima and sums are
    // two shuffles and the two groups run independently of each other.
    const int x = warp >> 3;
    const int half = (warp >> 2) & 1;
    const int lane_base = (warp & 3) * 32 + half * 16;  // first of this warp's 16 TMEM lanes
    const int quad = lane & 3;
    const int r0 = lane_base + (lane >> 2);             // tile rows r0 and r0 + 8
    const uint32_t t_row = tmem_base + ((uint32_t)lane_base << 16);
    const uint32_t t_s = t_row + (uint32_t)(x * BLK);
    const uint32_t t_o = t_row + (uint32_t)(QT * BLK + x * BLK);
    const int n = n_tiles[x];
    const int qrow0 = q0 + x * BLK;
    float m_used[2] = {-INFINITY, -INFINITY};
    float l[2] = {0.f, 0.f};                            // this thread's part of the row sums
    // split mode: the pre-pass scaled q and k by powers of two; dividing them out of the logit scale is exact
    const float scale_log2 = SPLIT ? p.scale_log2 * __ldg(p.split_fac + split::FAC_INV_QK) : p.scale_log2;
    for (int j = 0; j < n && ok; ++j) {
      TC_TRACE(x, j, 0);
      ok = __all_sync(0xffffffffu, mbar_wait_hot(bar(BAR_S_FULL + x), (uint32_t)(j & 1), p.status, 30 + x, j));
      if (!ok) break;
      if (j == 0) TC_PHASE(6, warp == 0 && lane == 0);
      TC_TRACE(x, j, 1);
      TC_TRACE_W(j, 0);
      tc_fence_after();
      // s[4g + 2h + e] = logit of row r0 + 8h, key 8g + 2*quad + e
      uint32_t s[64];
      tmem_ldq256_x8(t_s, s);
      tmem_ldq256_x8(t_s + 64, s + 32);
      tmem_wait_ld();
      TC_TRACE(x, j, 2);
      // Only the diagonal tile (causal) and the last tile (keys beyond T) need masking.
      if ((p.causal && j * BLK + BLK - 1 > qrow0) || (j * BLK + BLK > T)) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int kj = j * BLK + 8 * (i >> 2) + 2 * quad + (i & 1);
          const int qi = qrow0 + r0 + 8 * ((i >> 1) & 1);
          if (kj >= T || (p.causal && kj > qi)) s[i] = 0xff800000u;  // -inf
        }
      }
      if constexpr (MASKED) {
        // the caller's mask: this thread's two rows x 128 keys of keep-bits (key 8g + 2 quad + e is bit
        // 8 (g & 3) + 2 quad + e of word g >> 2); a masked logit becomes the same finite value everywhere
        const uint32_t masked_s = __float_as_uint(MASKED_LOG2 / scale_log2);
        const uint32_t* mrow = p.mask_bits + (int64_t)bi * p.mask_batch_stride + 4 * j;
        const uint4 mb0 = __ldg(reinterpret_cast<const uint4*>(mrow + (int64_t)min(qrow0 + r0, T - 1) * p.mask_row_stride));
        const uint4 mb1 = __ldg(reinterpret_cast<const uint4*>(mrow + (int64_t)min(qrow0 + r0 + 8, T - 1) * p.mask_row_stride));
        const uint32_t w0[4] = {mb0.x >> (2 * quad), mb0.y >> (2 * quad), mb0.z >> (2 * quad), mb0.w >> (2 * quad)};
        const uint32_t w1[4] = {mb1.x >> (2 * quad), mb1.y >> (2 * quad), mb1.z >> (2 * quad), mb1.w >> (2 * quad)};
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int g = i >> 2, e = i & 1;
          const uint32_t w = ((i >> 1) & 1) ? w1[g >> 2] : w0[g >> 2];
          if (((w >> (8 * (g & 3) + e)) & 1u) == 0u && s[i] != 0xff800000u) s[i] = masked_s;
        }
      }
      float mx[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float ma = -INFINITY, mb = -INFINITY;
#pragma unroll
        for (int g = 0; g < 16; g += 2) {
          ma = max3(ma, __uint_as_float(s[4 * g + 2 * h]), __uint_as_float(s[4 * g + 2 * h + 1]));
          mb = max3(mb, __uint_as_float(s[4 * g + 4 + 2 * h]), __uint_as_float(s[4 * g + 4 + 2 * h + 1]));
        }
        float m = fmaxf(ma, mb);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        mx[h] = m * scale_log2;
      }
      TC_TRACE_W(j, 1);
      float m_new[2];
      bool raise = false;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        m_new[h] = m_used[h];
        if (mx[h] > m_used[h] + RESCALE_THRESHOLD || j == 0) { m_new[h] = fmaxf(mx[h], m_used[h]); raise = raise || (j > 0); }
        if (m_new[h] == -INFINITY) m_new[h] = 0.f;  // a row with no visible key yet (rows beyond T)
      }
      if (__any_sync(0xffffffffu, raise)) {
        // rescale this warp's 16 rows of O in TMEM: the previous P V product must have finished
        ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_O_DONE + x), (uint32_t)((j - 1) & 1), p.status, 32 + x, j));
        if (!ok) break;
        tc_fence_after();
        float f[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          f[h] = (m_new[h] != m_used[h]) ? fast_exp2(m_used[h] - m_new[h]) : 1.0f;
          l[h] *= f[h];
        }
        if constexpr (HD >= 32) {
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[16];
            tmem_ldq256_x4(t_o + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f[(i >> 1) & 1]);
            tmem_stq256_x4(t_o + c * 32, o);
          }
        } else {   // 16 columns
          uint32_t o[8];
          tmem_ldq256_x2(t_o, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f[(i >> 1) & 1]);
          tmem_stq256_x2(t_o, o);
        }
      }
      TC_TRACE_W(j, 2);
      // p = 2^(s * scale_log2 - m): one FFMA and one exponential per element, packed to bf16;
      // the row sum is taken in fp32.  The first 64 keys are handed to the MMA warp before the rest.
      // split mode: the probabilities are kept 2^6 larger (they stay below 2^14), so that their fp16 halves leave the
      // normal range only below 2^-20 of the row's largest; the row sum carries the same factor and it cancels
      constexpr float P_BIAS = SPLIT ? 6.0f : 0.0f;
      const float2 nm2[2] = {make_float2(P_BIAS - m_new[0], P_BIAS - m_new[0]), make_float2(P_BIAS - m_new[1], P_BIAS - m_new[1])};
      const float2 scale2 = make_float2(scale_log2, scale_log2);
      float2 rs2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      uint32_t pk[16];
      uint32_t pk_lo[SPLIT ? 16 : 1];
      // exponentials of key groups [g_lo, g_hi) (8 keys each); bf16 results packed into pk[0..], tf32 in place;
      // split mode: hi = p with the mantissa cut to fp16 width (so the conversion is exact), lo = p - hi.
      // A thread's two adjacent keys of a row go through the scale-and-subtract and the row sum as one fp32 pair.
      auto exp_groups = [&](const int g_lo, const int g_hi) {
#pragma unroll
        for (int g = g_lo; g < g_hi; ++g) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float2 xx = ffma2(make_float2(__uint_as_float(s[4 * g + 2 * h]), __uint_as_float(s[4 * g + 2 * h + 1])), scale2, nm2[h]);
            const float p0 = exp2_sel(xx.x, 2 * g);
            const float p1 = exp2_sel(xx.y, 2 * g + 1);
            if constexpr (TF32) {
              s[4 * g + 2 * h] = __float_as_uint(p0);
              s[4 * g + 2 * h + 1] = __float_as_uint(p1);
            } else if constexpr (SPLIT) {
              const float h0 = __uint_as_float(__float_as_uint(p0) & 0xffffe000u), h1 = __uint_as_float(__float_as_uint(p1) & 0xffffe000u);
              pk[2 * (g - g_lo) + h] = pack_f16(h0, h1);
              pk_lo[2 * (g - g_lo) + h] = pack_f16(p0 - h0, p1 - h1);
            } else {
              pk[2 * (g - g_lo) + h] = pack_bf16(p0, p1);
            }
            rs2[h] = fadd2(rs2[h], make_float2(p0, p1));
          }
        }
      };
      // bf16 P: keys 2c, 2c+1 in column c of the S region (64 columns); tf32 P: in place of S.
      // The store of the first 64 keys completes behind the next exponentials, so its wait is short;
      // only the last quarter's store latency is exposed before the second product can finish.
      exp_groups(0, 8);
      if constexpr (TF32) tmem_stq256_x8(t_s, s);
      else tmem_stq128_x8(t_s, pk);
      if constexpr (SPLIT) tmem_stq128_x8(t_s + 64, pk_lo);
      TC_TRACE(x, j, 3);
      exp_groups(8, 12);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_P_HALF + x));
      if constexpr (TF32) tmem_stq256_x4(t_s + 64, s + 32);
      else tmem_stq128_x4(t_s + 32, pk);
      if constexpr (SPLIT) tmem_stq128_x4(t_s + 96, pk_lo);
      exp_groups(12, 16);
      if constexpr (TF32) tmem_stq256_x4(t_s + 96, s + 48);
      else tmem_stq128_x4(t_s + 48, pk);
      if constexpr (SPLIT) tmem_stq128_x4(t_s + 112, pk_lo);
      TC_TRACE(x, j, 4);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_P_READY + x));
      l[0] += rs2[0].x + rs2[0].y;
      l[1] += rs2[1].x + rs2[1].y;
      m_used[0] = m_new[0];
      m_used[1] = m_new[1];
      TC_TRACE(x, j, 5);
      TC_TRACE_W(j, 3);
    }
    // epilogue: finish the row sums, hand them to the thread that owns the row in the one-lane-per-
    // thread layout, then O / l -> global
    TC_PHASE(7, warp == 0 && lane == 0);
    if (ok && n > 0) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
      }
      float* red_l = reinterpret_cast<float*>(smem_gen + PL::OFF_RED) + x * 256;
      float* red_m = red_l + 128;
      if (quad == 0) {
        red_l[r0] = l[0]; red_l[r0 + 8] = l[1];
        red_m[r0] = m_used[0]; red_m[r0 + 8] = m_used[1];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_RED + x));
      ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_RED + x), 0, p.status, 36 + x, n));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_O_DONE + x), (uint32_t)((n - 1) & 1), p.status, 34 + x, n));
      TC_PHASE(8, warp == 0 && lane == 0);
      if (ok) {
        tc_fence_after();
        constexpr int OC = HD / 2;                       // O columns per thread: row = lane, half of the head
        const int row = (warp & 3) * 32 + lane;
        const int qi = qrow0 + row;
        const float lsum = red_l[row];
        // split mode: the pre-pass scaled v by a power of two; dividing it out here is exact
        const float inv = SPLIT ? __ldg(p.split_fac + split::FAC_INV_V) / lsum : 1.0f / lsum;
        const uint32_t t_o32 = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(QT * BLK + x * BLK + half * OC);
        if constexpr (F32_OUT && QT == 2) {
          // fp32 output of the two-tile shape: each thread stores its own row's pieces.  (Staged like the other
          // shapes, this instantiation's key loop spilled twice as much and ran 17 % slower at T = 8192.)
          float* yrow_f = reinterpret_cast<float*>(p.y) + (int64_t)bi * p.ys.b + (int64_t)hi * p.ys.h + (int64_t)qi * p.ys.t + half * OC;
          constexpr int CHD = OC < 16 ? OC : 16;
#pragma unroll
          for (int c = 0; c < OC / CHD; ++c) {
            uint32_t o[CHD];
            if constexpr (CHD == 16) tmem_ld16(t_o32 + c * 16, o);
            else tmem_ld8(t_o32, o);
            tmem_wait_ld();
            if (qi < T) {
#pragma unroll
              for (int i = 0; i < CHD; i += 4) {
                const float4 w = make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv,
                                             __uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                *reinterpret_cast<float4*>(yrow_f + c * CHD + i) = w;
                if constexpr (SPLIT) {
                  if (p.y_copy) *reinterpret_cast<float4*>(p.y_copy + ((int64_t)bh * T + qi) * HD + half * OC + c * CHD + i) = w;
                }
              }
            }
          }
        } else {
        // Stage this warp's 32 rows x OC columns in the shared memory of its query tile (every product that read it
        // has completed), then store whole 16-byte pieces so that one store instruction covers full contiguous row
        // segments (128 bytes at head size 128 in bf16) instead of 32 pieces from 32 different rows: a fraction of
        // the memory transactions for the local copy, and NVLink carries the copies for the peers as full packets.
        constexpr int ESZ = F32_OUT ? 4 : 2;               // bytes per output element
        constexpr int EPP = 16 / ESZ;                      // elements per 16-byte piece
        constexpr int PIECES = OC / EPP;                   // pieces of a row-half
        constexpr int RPI = 32 / PIECES;                   // rows one store instruction covers
        constexpr int CH = OC < 16 ? OC : 16;              // columns per TMEM load
        static_assert(8 * 32 * PIECES * 16 <= (int)PL::TILE_BYTES, "the output tile is staged in its query tile");
        uint4* stage = reinterpret_cast<uint4*>(smem_gen + PL::OFF_Q + x * PL::TILE_BYTES) +
                       (size_t)((warp & 3) * 2 + half) * 32 * PIECES;   // private to this warp
#pragma unroll
        for (int c = 0; c < OC / CH; ++c) {
          uint32_t o[CH];
          if constexpr (CH == 16) tmem_ld16(t_o32 + c * 16, o);
          else tmem_ld8(t_o32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < CH; i += EPP) {
            uint4 w;
            if constexpr (F32_OUT) {
              w.x = __float_as_uint(__uint_as_float(o[i + 0]) * inv);
              w.y = __float_as_uint(__uint_as_float(o[i + 1]) * inv);
              w.z = __float_as_uint(__uint_as_float(o[i + 2]) * inv);
              w.w = __float_as_uint(__uint_as_float(o[i + 3]) * inv);
            } else {
              w.x = pack_bf16(__uint_as_float(o[i + 0]) * inv, __uint_as_float(o[i + 1]) * inv);
              w.y = pack_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
              w.z = pack_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
              w.w = pack_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            }
            const int piece = (c * CH + i) / EPP;
            stage[lane * PIECES + (piece ^ (lane & (PIECES - 1)))] = w;   // swizzled against bank conflicts
          }
        }
        __syncwarp();
#pragma unroll
        for (int kk = 0; kk < PIECES; ++kk) {
          const int r = kk * RPI + lane / PIECES, pc = lane % PIECES;
          const uint4 w = stage[r * PIECES + (pc ^ (r & (PIECES - 1)))];
          const int qr = qrow0 + (warp & 3) * 32 + r;
          if (qr < T) {
            const int64_t off = (int64_t)bi * p.ys.b + (int64_t)hi * p.ys.h + (int64_t)qr * p.ys.t + half * OC + pc * EPP;
            *reinterpret_cast<uint4*>(static_cast<char*>(p.y) + off * ESZ) = w;
            if constexpr (!F32_OUT) {
#pragma unroll
              for (int d = 0; d < 7; ++d)   // constant indices: the parameter block is not copied to local memory
                if (d < p.n_more) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.y_more[d]) + off) = w;
            }
            if constexpr (SPLIT) {
              if (p.y_copy) *reinterpret_cast<uint4*>(p.y_copy + ((int64_t)bh * T + qr) * HD + half * OC + pc * EPP) = w;
            }
          }
        }
        }
        if (half == 0 && p.lse != nullptr && qi < T) {
          float lse_row = red_m[row] + log2f(lsum) - (SPLIT ? 6.0f : 0.0f);
          // a row whose every key is masked has uniform probabilities 1 / T; its log-sum-exp cannot carry that next
          // to the masked logit's magnitude, so the backward is told by +inf instead
          if (MASKED && red_m[row] < 0.5f * MASKED_LOG2) lse_row = INFINITY;
          p.lse[(int64_t)bh * T + qi] = lse_row;
        }
        if constexpr (SPLIT) {
          // what the exact fp32 backward needs to recompute P = exp(s - row_max) / row_sum: the exponent's reference
          // point in natural-log units (it need not be the true maximum) and the sum taken against it
          if (half == 0 && p.row_max != nullptr && qi < T) {
            p.row_max[(int64_t)bh * T + qi] = (red_m[row] - 6.0f) * 0.6931471805599453f;   // the 2^6 kept in the probabilities
            p.row_sum[(int64_t)bh * T + qi] = lsum;
          }
        }
      }
    }
  }
  // ------------------------------------------------------------------ teardown
  TC_PHASE(9, warp == 0 && lane == 0);
  tc_fence_before();
  __syncthreads();
  TC_PHASE(10, tid == 0);
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


struct SplitExtras {
  const float* fac = nullptr;   // split::SplitFac
  float *row_max = nullptr, *row_sum = nullptr, *y_copy = nullptr;
};

// Which sequences run as NARROW CTAs (one query tile each, two CTAs per SM).  Rows of 128 bytes (64-wide bf16 heads):
// all of them -- a key tile costs the softmax as much as at 128 and the tensor pipe half, and two independent CTAs per
// SM keep both busier than one CTA's two tiles in anti-phase (T = 8192: 585 -> 711 TFLOP/s, T = 32768: 653 -> 780).
// Rows of 256 bytes: sequences up to a threshold, 8192 keys for 128-wide bf16 heads (+ 5 % at T = 8192, B = 1) and
// half of it for split fp32 operands (single-stage K and V; alike beyond), unless MCA_TC_NARROW_LEN in the environment
// or mca_tc_narrow_len() says otherwise (0: never, for either row size); beyond it the two shapes run alike (the
// headline shape within 1 %, the one-tile shape at lower clocks under the power cap) and the two-tile one reads K and V
// from L2 once per pair of tiles.
int& narrow_limit() {
  static int limit = [] {
    const char* e = getenv("MCA_TC_NARROW_LEN");
    return e != nullptr ? atoi(e) : 8192;
  }();
  return limit;
}
inline bool narrow_ctas(int T, int row_bytes, bool split_operands) {
  const int limit = narrow_limit();
  return limit > 0 && (row_bytes <= 128 || T <= (split_operands ? limit / 2 : limit));
}

template <int HD, int MODE, bool NARROW>
int launch_shape(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const TcParams& p, int B, int H, int T,
                 bool masked, cudaStream_t st) {
  using SH = Shape<HD, MODE, NARROW>;
  const size_t smem = SH::PL::BYTES;
  dim3 grid(mca_ceil_div(T, SH::QT * BLK), B * H);
  if constexpr (MODE != MODE_TF32) {
    if (masked) {
      MCA_CUDA_TRY(cudaFuncSetAttribute(sdpa_fwd_tc_kernel<HD, MODE, true, NARROW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      return mca_launch_pdl(sdpa_fwd_tc_kernel<HD, MODE, true, NARROW>, grid, dim3(SH::THREADS), smem, st, mq, mk, mv, p);
    }
  }
  MCA_CUDA_TRY(cudaFuncSetAttribute(sdpa_fwd_tc_kernel<HD, MODE, false, NARROW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  return mca_launch_pdl(sdpa_fwd_tc_kernel<HD, MODE, false, NARROW>, grid, dim3(SH::THREADS), smem, st, mq, mk, mv, p);
}

template <int HD, int MODE>
int launch_tc(const void* q, const void* k, const void* v, int causal, int B, int H, int T, void* y, float* lse,
              int* status, int layout, cudaStream_t st, void* const* y_more = nullptr, int n_more = 0,
              const McaStrides* y_strides = nullptr, const SplitExtras* split = nullptr, const McaMaskBits* mask = nullptr) {
  if (mask != nullptr && (MODE == MODE_TF32 || causal)) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  CUtensorMap mq, mk, mv;
  int e;
  const McaStrides sin = mca_in_strides(layout, H, T, HD);
  if constexpr (MODE == MODE_TF32) {
    if ((e = make_map_f32(&mq, q, B, H, T, HD, sin)) || (e = make_map_f32(&mk, k, B, H, T, HD, sin)) ||
        (e = make_map_f32(&mv, v, B, H, T, HD, sin, true)))
      return e;
  } else if constexpr (MODE == MODE_SPLIT) {
    // the pre-pass wrote contiguous (B, H, T, RH) fp16 rows [hi | lo], whatever layout the fp32 tensors have
    constexpr int RH = split::row_halves(HD);
    const McaStrides sp{(int64_t)H * T * RH, (int64_t)T * RH, RH};
    if ((e = make_map_4d(&mq, q, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, B, H, T, RH, sp, CU_TENSOR_MAP_SWIZZLE_128B)) ||
        (e = make_map_4d(&mk, k, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, B, H, T, RH, sp, CU_TENSOR_MAP_SWIZZLE_128B)) ||
        (e = make_map_4d(&mv, v, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, B, H, T, RH, sp, CU_TENSOR_MAP_SWIZZLE_128B)))
      return e;
  } else {
    if ((e = make_map_bf16(&mq, q, B, H, T, HD, sin)) || (e = make_map_bf16(&mk, k, B, H, T, HD, sin)) ||
        (e = make_map_bf16(&mv, v, B, H, T, HD, sin)))
      return e;
  }
  TcParams p;
  p.y = y; p.lse = lse; p.status = status; p.T = T; p.causal = causal; p.H = H;
  // K and V of one (batch, head) are 2 * T * HD elements; keep a group's set under about 64 MB of the 126 MB L2
  {
    const int64_t row_bytes = MODE == MODE_SPLIT ? 2 * split::row_halves(HD) : HD * (MODE == MODE_TF32 ? 4 : 2);
    const int64_t kv_bytes = (int64_t)2 * T * row_bytes;
    int64_t g = (64ll << 20) / kv_bytes;
    p.group = (int)std::max<int64_t>(1, std::min<int64_t>(g, (int64_t)B * H));
    if (!causal) p.group = 1;   // equal work per CTA: nothing to balance
  }
  p.ys = y_strides ? *y_strides : mca_out_strides(layout, H, T, HD);
  p.n_more = n_more;
  for (int i = 0; i < 7; ++i) p.y_more[i] = i < n_more ? y_more[i] : nullptr;
  p.scale_log2 = (1.0f / sqrtf((float)HD)) * 1.4426950408889634f;
  p.split_fac = split ? split->fac : nullptr;
  p.row_max = split ? split->row_max : nullptr;
  p.row_sum = split ? split->row_sum : nullptr;
  p.y_copy = split ? split->y_copy : nullptr;
  p.mask_bits = mask ? mask->bits : nullptr;
  p.mask_batch_stride = mask ? mask->batch_stride : 0;
  p.mask_row_stride = mask ? mask->row_stride : 0;
  if constexpr (!Shape<HD, MODE, false>::WIDE && MODE != MODE_TF32) {
    if (narrow_ctas(T, Shape<HD, MODE, false>::ROW_BYTES, MODE == MODE_SPLIT)) return launch_shape<HD, MODE, true>(mq, mk, mv, p, B, H, T, mask != nullptr, st);
  }
  return launch_shape<HD, MODE, false>(mq, mk, mv, p, B, H, T, mask != nullptr, st);
}

template <int HD>
int launch_split(const float* q, const float* k, const float* v, int causal, int B, int H, int T, float* y, float* row_max,
                 float* row_sum, float* y_copy, float* lse, void* workspace, int* status, int layout, cudaStream_t st,
                 const McaMaskBits* mask = nullptr) {
  const int64_t rows = (int64_t)B * H * T;
  const split::Workspace w = split::carve(workspace, rows, HD);
  split::Job job;
  job.src[0] = q; job.src[1] = k; job.src[2] = v;
  for (int i = 0; i < 3; ++i) { job.dst[i] = w.tensor[i]; job.slot[i] = i; }
  int e = split::run<HD>(job, 3, mca_in_strides(layout, H, T, HD), H, T, rows, w, false, st);
  if (e) return e;
  SplitExtras ex;
  ex.fac = w.fac; ex.row_max = row_max; ex.row_sum = row_sum; ex.y_copy = y_copy;
  return launch_tc<HD, MODE_SPLIT>(w.tensor[0], w.tensor[1], w.tensor[2], causal, B, H, T, y, lse, status, layout, st, nullptr, 0,
                                   nullptr, &ex, mask);
}

}  // namespace

#ifdef MCA_TC_TRACE
extern "C" __attribute__((visibility("default"))) int mca_tc_trace_fetch(long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, g_tc_trace, sizeof(long long) * count);
}
extern "C" __attribute__((visibility("default"))) int mca_tc_trace_fetch_phase(long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, g_tc_phase, sizeof(long long) * count);
}
extern "C" __attribute__((visibility("default"))) int mca_tc_trace_fetch_w(long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, g_tc_trace_w, sizeof(long long) * count);
}
#endif

int mca_sdpa_forward_tc(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H, int T, int D,
                        void* y, float* lse, int* status, void* stream) {
  return mca_sdpa_forward_tc_layout(q, k, v, dtype, causal, B, H, T, D, y, lse, status, MCA_LAYOUT_BHTD, stream);
}

int mca_sdpa_forward_tc_scatter(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H, int T,
                                int D, void* const* y_dst, int n_dst, int64_t y_stride_b, int64_t y_stride_h,
                                int64_t y_stride_t, float* lse, int* status, void* stream) {
  if (!q || !k || !v || !y_dst || !status) return ERROR_PARAM_NULL;
  if (n_dst < 1 || n_dst > 8) return ERROR_PARAM_OUT_OF_RANGE;
  if (B <= 0 || H <= 0 || T <= 0 || (int64_t)B * H > 65535) return ERROR_PARAM_OUT_OF_RANGE;
  if (dtype != MCA_DTYPE_BF16) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  if (y_stride_t < D || y_stride_h <= 0 || y_stride_b <= 0 || (y_stride_t | y_stride_h | y_stride_b) % 8) return ERROR_PARAM_OUT_OF_RANGE;
  uintptr_t bits = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v);
  for (int i = 0; i < n_dst; ++i) {
    if (!y_dst[i]) return ERROR_PARAM_NULL;
    bits |= reinterpret_cast<uintptr_t>(y_dst[i]);
  }
  if (bits & 15) return ERROR_PARAM_OUT_OF_RANGE;
  const McaStrides ys{y_stride_b, y_stride_h, y_stride_t};
  cudaStream_t st = (cudaStream_t)stream;
  if (D == 128) return launch_tc<128, MODE_BF16>(q, k, v, causal, B, H, T, y_dst[0], lse, status, MCA_LAYOUT_BHTD, st, y_dst + 1, n_dst - 1, &ys);
  if (D == 64) return launch_tc<64, MODE_BF16>(q, k, v, causal, B, H, T, y_dst[0], lse, status, MCA_LAYOUT_BHTD, st, y_dst + 1, n_dst - 1, &ys);
  return ERROR_ATTN_UNSUPPORTED_SHAPE;
}

int mca_sdpa_forward_tc_layout(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H, int T,
                               int D, void* y, float* lse, int* status, int layout, void* stream) {
  return mca_sdpa_forward_tc_masked(q, k, v, dtype, causal, B, H, T, D, y, lse, status, layout, nullptr, MCA_MASK_NONE, stream);
}

int mca_sdpa_forward_tc_masked(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H, int T, int D,
                               void* y, float* lse, int* status, int layout, const uint32_t* mask_bits, int mask_mode,
                               void* stream) {
  return mca_sdpa_forward_tc_keep(q, k, v, dtype, causal, B, H, T, D, y, nullptr, lse, status, layout, mask_bits, mask_mode, stream);
}

int mca_sdpa_forward_tc_keep(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H, int T, int D,
                             void* y, void* y_keep, float* lse, int* status, int layout, const uint32_t* mask_bits,
                             int mask_mode, void* stream) {
  McaMaskBits mb;
  const McaMaskBits* mask = nullptr;
  int me = mca_mask_bits_view(mask_bits, nullptr, mask_mode, T, false, &mb, &mask);
  if (me) return me;
  if (mask != nullptr && dtype != MCA_DTYPE_BF16) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  if (layout != MCA_LAYOUT_BHTD && layout != MCA_LAYOUT_PACKED) return ERROR_PARAM_OUT_OF_RANGE;
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
    if (y_keep != nullptr) return ERROR_ATTN_UNSUPPORTED_SHAPE;
    if (D == 64) return launch_tc<64, MODE_TF32>(q, k, v, causal, B, H, T, y, lse, status, layout, st);
    return ERROR_ATTN_UNSUPPORTED_SHAPE;
  }
  // a second copy of the output in the same layout (what a training handle keeps for its backward) is one more
  // destination of the epilogue's stores
  if (y_keep != nullptr && (reinterpret_cast<uintptr_t>(y_keep) & 15)) return ERROR_PARAM_OUT_OF_RANGE;
  void* const more[1] = {y_keep};
  const int n_more = y_keep != nullptr ? 1 : 0;
  if (D == 128) return launch_tc<128, MODE_BF16>(q, k, v, causal, B, H, T, y, lse, status, layout, st, more, n_more, nullptr, nullptr, mask);
  if (D == 64) return launch_tc<64, MODE_BF16>(q, k, v, causal, B, H, T, y, lse, status, layout, st, more, n_more, nullptr, nullptr, mask);
  return ERROR_ATTN_UNSUPPORTED_SHAPE;
}

int mca_tc_narrow_len(int len) {
  const int before = narrow_limit();
  if (len >= 0) narrow_limit() = len;
  return before;
}

int64_t mca_sdpa_forward_f32_tc_workspace_bytes(int B, int H, int T) {
  if (B <= 0 || H <= 0 || T <= 0) return -1;
  return split::workspace_bytes((int64_t)B * H * T);
}

int64_t mca_sdpa_forward_f32_tc_workspace_bytes_d(int B, int H, int T, int D) {
  if (B <= 0 || H <= 0 || T <= 0 || !mca_sdpa_forward_f32_tc_supported(D)) return -1;
  return split::workspace_bytes((int64_t)B * H * T, D);
}

int mca_sdpa_forward_f32_tc_supported(int D) { return D == 16 || D == 32 || D == 64 || D == 128; }

int mca_sdpa_backward_f32_tc_supported(int D) { return D == 16 || D == 32 || D == 64; }

int mca_sdpa_forward_f32_tc(const float* q, const float* k, const float* v, int causal, int B, int H, int T, int D, float* y,
                            float* row_max, float* row_sum, float* y_copy, float* lse, void* workspace,
                            int64_t workspace_bytes, int* status, int layout, void* stream) {
  return mca_sdpa_forward_f32_tc_masked(q, k, v, causal, B, H, T, D, y, row_max, row_sum, y_copy, lse, workspace, workspace_bytes,
                                        status, layout, nullptr, MCA_MASK_NONE, stream);
}

int mca_sdpa_forward_f32_tc_masked(const float* q, const float* k, const float* v, int causal, int B, int H, int T, int D,
                                   float* y, float* row_max, float* row_sum, float* y_copy, float* lse, void* workspace,
                                   int64_t workspace_bytes, int* status, int layout, const uint32_t* mask_bits, int mask_mode,
                                   void* stream) {
  McaMaskBits mb;
  const McaMaskBits* mask = nullptr;
  int me = mca_mask_bits_view(mask_bits, nullptr, mask_mode, T, false, &mb, &mask);
  if (me) return me;
  if (layout != MCA_LAYOUT_BHTD && layout != MCA_LAYOUT_PACKED) return ERROR_PARAM_OUT_OF_RANGE;
  if (!q || !k || !v || !y || !status || !workspace) return ERROR_PARAM_NULL;
  if ((row_max == nullptr) != (row_sum == nullptr)) return ERROR_PARAM_NULL;
  if (B <= 0 || H <= 0 || T <= 0 || (int64_t)B * H > 65535) return ERROR_PARAM_OUT_OF_RANGE;
  if (!mca_sdpa_forward_f32_tc_supported(D)) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  if (workspace_bytes < mca_sdpa_forward_f32_tc_workspace_bytes_d(B, H, T, D)) return ERROR_ATTN_SCRATCH_TOO_SMALL;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(y_copy)) & 15)
    return ERROR_PARAM_OUT_OF_RANGE;
  if (reinterpret_cast<uintptr_t>(workspace) & 15) return ERROR_PARAM_OUT_OF_RANGE;
  cudaStream_t st = (cudaStream_t)stream;
  switch (D) {
    case 16: return launch_split<16>(q, k, v, causal, B, H, T, y, row_max, row_sum, y_copy, lse, workspace, status, layout, st, mask);
    case 32: return launch_split<32>(q, k, v, causal, B, H, T, y, row_max, row_sum, y_copy, lse, workspace, status, layout, st, mask);
    case 64: return launch_split<64>(q, k, v, causal, B, H, T, y, row_max, row_sum, y_copy, lse, workspace, status, layout, st, mask);
    case 128: return launch_split<128>(q, k, v, causal, B, H, T, y, row_max, row_sum, y_copy, lse, workspace, status, layout, st, mask);
  }
  return ERROR_ATTN_UNSUPPORTED_SHAPE;
}


// ---------------------------------------------------------------------------------------------
// Keep-bits of a float mask for the tensor-core kernels.  One warp per output word: bit i of word w of row r is
// mask[r][32 w + i] != 0 (keys beyond T: 0); the transposed form has bit i of word w of key k = mask[32 w + i][k] != 0.
// Rows are padded to whole 128-key tiles (mca_mask_bits_row_words(T) words).
// ---------------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(256) mask_pack_kernel(const float* __restrict__ mask, int rows, int T, int wpr,
                                                        uint32_t* __restrict__ bits, uint32_t* __restrict__ bits_t) {
  const int64_t word = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (word >= (int64_t)rows * wpr) return;
  const int r = (int)(word / wpr), w = (int)(word - (int64_t)r * wpr);
  const int c = 32 * w + lane;
  const uint32_t keep = __ballot_sync(0xffffffffu, c < T && mask[(int64_t)r * T + c] != 0.f);
  if (lane == 0) bits[word] = keep;
  if (bits_t != nullptr) {   // square mask: the same word position of the transpose
    const uint32_t keep_t = __ballot_sync(0xffffffffu, c < T && mask[(int64_t)c * T + r] != 0.f);
    if (lane == 0) bits_t[word] = keep_t;
  }
}
}  // namespace

int mca_mask_bits_row_words(int T) { return T > 0 ? mca_ceil_div(T, 128) * 4 : 0; }

int mca_mask_bits_view(const uint32_t* bits, const uint32_t* bits_t, int mask_mode, int T, int need_transpose, McaMaskBits* out,
                       const McaMaskBits** view) {
  *view = nullptr;
  if (mask_mode == MCA_MASK_NONE || mask_mode == MCA_MASK_CAUSAL) return bits == nullptr ? 0 : ERROR_PARAM_OUT_OF_RANGE;
  if (mask_mode != MCA_MASK_TT && mask_mode != MCA_MASK_BATCH) return ERROR_PARAM_OUT_OF_RANGE;
  if (bits == nullptr || (mask_mode == MCA_MASK_TT && need_transpose && bits_t == nullptr)) return ERROR_PARAM_NULL;
  if ((reinterpret_cast<uintptr_t>(bits) | reinterpret_cast<uintptr_t>(bits_t)) & 15) return ERROR_PARAM_OUT_OF_RANGE;
  const int wpr = mca_mask_bits_row_words(T);
  out->bits = bits;
  out->bits_t = mask_mode == MCA_MASK_TT ? bits_t : nullptr;
  out->row_stride = mask_mode == MCA_MASK_TT ? wpr : 0;
  out->batch_stride = mask_mode == MCA_MASK_BATCH ? wpr : 0;
  *view = out;
  return 0;
}

int mca_mask_pack(const float* mask, int mask_mode, int B, int T, uint32_t* bits, uint32_t* bits_t, void* stream) {
  if (!mask || !bits) return ERROR_PARAM_NULL;
  if (T <= 0 || B <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (mask_mode != MCA_MASK_TT && mask_mode != MCA_MASK_BATCH) return ERROR_PARAM_OUT_OF_RANGE;
  const int rows = mask_mode == MCA_MASK_TT ? T : B, wpr = mca_mask_bits_row_words(T);
  const int64_t words = (int64_t)rows * wpr;
  mask_pack_kernel<<<(unsigned)((words + 7) / 8), 256, 0, (cudaStream_t)stream>>>(mask, rows, T, wpr, bits,
                                                                               mask_mode == MCA_MASK_TT ? bits_t : nullptr);
  return mca_launch_status();
}

// Fused attention backward on the tensor cores (sm_100a, bf16): the counterpart of the forward
// kernel in attn_tc.cu for training.
//
// Same mathematics as the reference's attnHandle<T>::Backward (CudaDnnDLL/Cuda Files/
// attn.cu:608-661 with blob<T>::matmulgrad attn.cu:380-397):
//   dP = dY V^T,  dV = P^T dY,  dS = P o (dP - rowsum(dP o P)),  dS *= 1/sqrt(D),
//   dQ = dS K,    dK = dS^T Q
// The reference reads the (B,H,T,T) probabilities its Forward saved; here P is recomputed tile
// by tile from the log-sum-exp kept by the forward kernel, and rowsum(dP o P) is taken as
// delta = rowsum(dY o Y), so no T x T tensor exists.
//
// Two kernels (no atomics, deterministic):
//   * dq kernel: one CTA per 128-row query tile walks the key tiles:  S = Q K^T and dP = dY V^T
//     (tcgen05.mma, both operands in shared memory), dS computed by sixteen warps straight from
//     TMEM and written back as a bf16 A operand, dQ += dS K accumulated in TMEM.
//   * dkdv kernel: one CTA per 128-row key tile walks the query tiles with the transposed
//     products S^T = K Q^T and dP^T = V dY^T, so that P^T and dS^T come out in the layout the
//     A operand of dV += P^T dY and dK += dS^T Q needs.
// Q/K/V/dY tiles arrive by TMA (no multicast) through two-stage rings; every mbarrier wait is
// bounded as in the forward kernel.
//
// SPLIT = true is the variant for fp32 callers: every operand is carried as two fp16 halves (rows [hi | lo] written by
// the pre-pass in split_prepass.cuh, each tensor scaled by a power of two), every product is the three kind::f16
// products hi.hi + hi.lo + lo.hi into one fp32 TMEM tile, P^T / dS / dS^T are split the same way by the element-wise
// warps, and the gradients are written in fp32.  Head sizes up to 64: a split tile is as large as a 128-wide bf16 one.
#include "kernels.h"
#include "tc_common.cuh"
#include "split_prepass.cuh"

namespace {

using namespace tc;

constexpr int EW_WARPS = 16;                 // element-wise warps: four threads per row, 32 columns each
constexpr int WARP_TMA = EW_WARPS;
constexpr int WARP_MMA = EW_WARPS + 1;
constexpr int BW_THREADS = (EW_WARPS + 2) * 32;

template <int HD> struct BwdPlan {
  static constexpr int SUB = HD / 64;
  static constexpr uint32_t SUB_BYTES = BLK * 128;
  static constexpr uint32_t TILE_BYTES = SUB * SUB_BYTES;  // 128 x HD bf16
  // [0] and [1]: the two resident tiles (Q,dY or K,V); then two ring stages of two tiles each
  static constexpr uint32_t OFF_RES0 = 0;
  static constexpr uint32_t OFF_RES1 = TILE_BYTES;
  static constexpr uint32_t OFF_RING = 2 * TILE_BYTES;     // stage s: tile a at +s*2*TILE, tile b at +TILE after it
  static constexpr uint32_t OFF_BAR = 6 * TILE_BYTES;
  static constexpr uint32_t BYTES = OFF_BAR + 256 + 1024;
  // dQ kernel: K lives until the step's dQ product, so its ring is one stage deeper than V's (K(j+2) could
  // otherwise only be requested when dQ(j) has finished, one step before it is needed, and every step
  // would wait out the load latency): K stages at OFF_RING + {0,1,2} tiles, V stages behind them.
  static constexpr int K_STAGES = 3, V_STAGES = 2;
  static constexpr uint32_t OFF_KRING = OFF_RING;
  static constexpr uint32_t OFF_VRING = OFF_RING + K_STAGES * TILE_BYTES;
  static constexpr uint32_t OFF_BAR_DQ = OFF_VRING + V_STAGES * TILE_BYTES;
  static constexpr uint32_t BYTES_DQ = OFF_BAR_DQ + 256 + 1024;
  // dK/dV kernel: the same seven tiles, then barriers, the staged per-query terms ([2][128] floats twice) and the
  // abort flag, all in dynamic shared memory (no static allocation, so the dynamic base keeps its alignment).
  // At HD = 128 this leaves 752 bytes for aligning the base to 1024; the kernel checks that it fits.
  static constexpr uint32_t OFF_STAGE_KV = OFF_BAR_DQ + 256;
  static constexpr uint32_t OFF_FLAG_KV = OFF_STAGE_KV + 2 * 2 * BLK * 4;
  static constexpr uint32_t NEED_KV = OFF_FLAG_KV + 16;
  static constexpr uint32_t BYTES_KV = (NEED_KV + 1024 <= 227u * 1024u) ? NEED_KV + 1024 : 227u * 1024u;
};

// fp16 halves of a value the tensor core must see at fp32 accuracy: hi = v with the mantissa cut to fp16 width (the
// conversion is then exact for normal numbers), lo = v - hi.
__device__ __forceinline__ void split_pack(float v0, float v1, uint32_t& hi, uint32_t& lo) {
  const float h0 = __uint_as_float(__float_as_uint(v0) & 0xffffe000u), h1 = __uint_as_float(__float_as_uint(v1) & 0xffffe000u);
  hi = pack_f16(h0, h1);
  lo = pack_f16(v0 - h0, v1 - h1);
}
// Split mode keeps dS 2^-19 smaller than dP' = dY' V'^T (both operands scaled to below 2^13, so |dP'| < 2^32 at 64-wide
// heads) and P^T 2^10 larger than P <= 1: both then sit in the middle of the fp16 range.
constexpr float DS_SHIFT = 1.0f / 524288.0f, DS_UNSHIFT = 524288.0f, PT_SHIFT = 1024.0f, PT_UNSHIFT = 1.0f / 1024.0f;

struct BwdParams {
  const float* fac;    // split mode: the pre-pass's scale factors (split::SplitFac), device memory
  const float* lse;    // (BH, T) log2-domain log-sum-exp of the scaled logits, from the forward kernel
  const float* delta;  // (BH, T) rowsum(dY o Y)
  void* out0;          // dq kernel: dQ;  dkdv kernel: dK
  void* out1;          // dkdv kernel: dV
  int* status;
  int T, causal, H;
  int group;           // (batch, head) pairs whose CTAs are interleaved longest-first (their tensors fit in L2 together)
  float scale_log2;    // (1/sqrt(HD)) * log2(e)
  float scale;         // 1/sqrt(HD)
  McaStrides os;       // element strides of the gradient views dQ, dK, dV
  // MASKED: keep-bits of the caller's mask as the forward kernel reads them (word of query row r, key tile j, quarter
  // c: mask_bits[b * batch_stride + r * row_stride + 4 j + c]) and, for a (T,T) mask, their transpose (word of key k,
  // query tile i, quarter c: mask_bits_t[k * row_stride + 4 i + c]); a (B,T) key mask has row stride 0 and no transpose.
  // A masked entry has probability 0, or 1 / T in a row whose every key is masked (the forward marks those rows
  // with lse = +inf).
  const uint32_t* mask_bits;
  const uint32_t* mask_bits_t;
  int64_t mask_batch_stride, mask_row_stride;
  float inv_T;
};


// The gradient tiles leave through shared memory.  In the TMEM layout a thread owns a quarter of one row, so direct
// stores are 32 sixteen-byte pieces from 32 rows per instruction (9-12 % of the backward at T = 1024 was these
// stores).  Instead the sixteen element-wise warps write their pieces into a resident operand tile that every product
// has finished with (Q or K for the first result, dY or V for the second), meet at a named barrier, and each warp
// stores eight whole rows.  Every element-wise warp reaches the barrier, also after a failed wait.
__device__ __forceinline__ void ew_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(EW_WARPS * 32) : "memory"); }
// 16-byte piece `piece` of row `row` of a staged 128-row tile with PR pieces per row (XOR-swizzled by row)
template <int PR> __device__ __forceinline__ uint4* staged_piece(uint8_t* tile, int row, int piece) {
  return reinterpret_cast<uint4*>(tile) + row * PR + (piece ^ (row & (PR - 1)));
}
// this thread's OC columns of its row, scaled, as 16-byte pieces of bf16 or fp32
template <int PR, int OC, bool F32>
__device__ __forceinline__ void stage_columns(uint8_t* tile, int row, int qtr, uint32_t t_addr, float mul) {
  constexpr int CH = OC < 16 ? OC : 16;
#pragma unroll
  for (int c = 0; c < OC / CH; ++c) {
    uint32_t o[CH];
    if constexpr (CH == 16) tmem_ld16(t_addr + c * 16, o);
    else if constexpr (CH == 8) tmem_ld8(t_addr, o);
    else tmem_ld4(t_addr, o);
    tmem_wait_ld();
    if constexpr (F32) {
#pragma unroll
      for (int i = 0; i < CH; i += 4)
        *staged_piece<PR>(tile, row, (qtr * OC + c * CH + i) / 4) =
            make_uint4(__float_as_uint(__uint_as_float(o[i]) * mul), __float_as_uint(__uint_as_float(o[i + 1]) * mul),
                       __float_as_uint(__uint_as_float(o[i + 2]) * mul), __float_as_uint(__uint_as_float(o[i + 3]) * mul));
    } else {
#pragma unroll
      for (int i = 0; i < CH; i += 8)
        *staged_piece<PR>(tile, row, (qtr * OC + c * CH + i) / 8) =
            make_uint4(pack_bf16(__uint_as_float(o[i + 0]) * mul, __uint_as_float(o[i + 1]) * mul),
                       pack_bf16(__uint_as_float(o[i + 2]) * mul, __uint_as_float(o[i + 3]) * mul),
                       pack_bf16(__uint_as_float(o[i + 4]) * mul, __uint_as_float(o[i + 5]) * mul),
                       pack_bf16(__uint_as_float(o[i + 6]) * mul, __uint_as_float(o[i + 7]) * mul));
    }
  }
}
// warp w of the sixteen stores rows 8 w .. 8 w + 7 of a staged tile; off0: element offset of the tile's row 0
template <int PR, int ESZ>
__device__ __forceinline__ void store_staged_rows(uint8_t* tile, int w, int lane, void* out, int64_t off0, int64_t row_stride,
                                                  int rows_valid) {
  constexpr int RPI = 32 / PR;   // rows per store instruction
#pragma unroll
  for (int kk = 0; kk < 8 / RPI; ++kk) {
    const int row = 8 * w + kk * RPI + lane / PR, piece = lane % PR;
    if (row < rows_valid)
      *reinterpret_cast<uint4*>(static_cast<char*>(out) + (off0 + (int64_t)row * row_stride) * ESZ + piece * 16) =
          *staged_piece<PR>(tile, row, piece);
  }
}

// ---------------------------------------------------------------------------------------------
// dQ kernel.  TMEM columns: S [0,128)  dP [128,256)  dS (bf16, packed) [256,320)  dQ [320,320+HD);
// split mode: dS hi [256,320), dS lo [320,384), dQ [384,384+HD)
// ---------------------------------------------------------------------------------------------
enum DqBar : int {
  DQ_QDO_FULL = 0,
  DQ_K_FULL = 1,    // [3]
  DQ_K_EMPTY = 4,   // [3]
  DQ_V_FULL = 7,    // [2]
  DQ_V_EMPTY = 9,   // [2]
  DQ_SDP_FULL = 11, // S and dP of the step written by the MMA
  DQ_SDP_FREE = 12, // element-wise warps have S and dP in registers
  DQ_DS_READY = 13, // dS written to TMEM
  DQ_DQ_DONE = 14,  // dQ += dS K of the step finished (dS may be overwritten)
  DQ_DRAIN = 15,
  DQ_BAR_COUNT = 16
};

template <int HD, bool SPLIT, bool MASKED>
__global__ void __launch_bounds__(BW_THREADS, 1)
sdpa_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                      const BwdParams p) {
  using PL = BwdPlan<SPLIT ? 128 : HD>;   // a split row is two 128-byte sub-tiles [hi | lo]
  constexpr int FMT = SPLIT ? 0 : 1;       // operand format of the instruction descriptor: fp16 or bf16
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar0 = smem_base + PL::OFF_BAR_DQ;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + PL::OFF_BAR_DQ + DQ_BAR_COUNT * 8);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // launch order -> work item: longest causal work first inside groups of p.group heads (see the forward kernel)
  const int lin = (int)(blockIdx.y * gridDim.x + blockIdx.x);
  const int grp = lin / (p.group * (int)gridDim.x);
  const int in_grp = lin - grp * p.group * (int)gridDim.x;
  const int grp_heads = min(p.group, (int)gridDim.y - grp * p.group);
  const int rank = in_grp / grp_heads;
  const int bh = grp * p.group + (in_grp - rank * grp_heads), T = p.T;
  const int bi = bh / p.H, hi = bh - bi * p.H;   // batch item and head
  const int qt = (int)gridDim.x - 1 - rank;
  const int q0 = qt * BLK;
  const int n = p.causal ? (min(q0 + BLK, T) + BLK - 1) / BLK : (T + BLK - 1) / BLK;

  // set-up, each part by another warp so that their latencies overlap (status word, barriers, descriptors, TMEM)
  __shared__ int s_abort;
  mca_pdl_launch_dependents();
  if (tid == 32) s_abort = *reinterpret_cast<volatile int*>(p.status);
  if (warp == WARP_TMA && lane == 0) {
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v); prefetch_tensormap(&map_do);
  }
  if (tid == 0) {
    for (int i = 0; i < DQ_BAR_COUNT; ++i)
      mbar_init(bar(i), (i == DQ_SDP_FREE || i == DQ_DS_READY) ? (uint32_t)EW_WARPS : 1u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == WARP_MMA) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // No wait here.  The kernel before this one in a backward is the dK/dV kernel, which lets its dependents go only
  // after its own wait: when a CTA of this kernel runs, everything before that kernel (delta, the forward, the operand
  // split) is complete and visible, and that is all this kernel reads.  It writes dQ only, which the dK/dV kernel does
  // not touch, so its CTAs work in the SMs that kernel's last wave leaves free.  The wait at the end keeps the order
  // for what follows: this kernel is not complete before the dK/dV kernel is.
  if (s_abort != 0) {   // an earlier CTA already failed: leave (uniform decision) before any copy or product is issued
    if (warp == WARP_MMA) tmem_dealloc(tmem_base, TMEM_COLS);
    mca_pdl_wait();
    return;
  }
  constexpr uint32_t C_S = 0, C_DP = 128, C_DS = 256, C_DQ = SPLIT ? 384 : 320;
  bool ok = true;

  if (warp == WARP_TMA) {
    if (lane == 0) {
      mbar_expect_tx(bar(DQ_QDO_FULL), 2 * PL::TILE_BYTES);
#pragma unroll
      for (int s = 0; s < PL::SUB; ++s) {
        tma_load_4d(smem_base + PL::OFF_RES0 + s * PL::SUB_BYTES, &map_q, bar(DQ_QDO_FULL), s * 64, q0, hi, bi);
        tma_load_4d(smem_base + PL::OFF_RES1 + s * PL::SUB_BYTES, &map_do, bar(DQ_QDO_FULL), s * 64, q0, hi, bi);
      }
      int issued_k = 0, issued_v = 0;
      for (int j = 0; j < n && ok; ++j) {
        const int ks = j % PL::K_STAGES, vs = j % PL::V_STAGES;
        const uint32_t kph = (uint32_t)((j / PL::K_STAGES) & 1), vph = (uint32_t)((j / PL::V_STAGES) & 1);
        const uint32_t k_dst = smem_base + PL::OFF_KRING + ks * PL::TILE_BYTES, v_dst = smem_base + PL::OFF_VRING + vs * PL::TILE_BYTES;
        ok = mbar_wait(bar(DQ_K_EMPTY + ks), kph ^ 1u, p.status, 110, j);
        if (!ok) break;
        mbar_expect_tx(bar(DQ_K_FULL + ks), PL::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < PL::SUB; ++s) tma_load_4d(k_dst + s * PL::SUB_BYTES, &map_k, bar(DQ_K_FULL + ks), s * 64, j * BLK, hi, bi);
        issued_k = j + 1;
        ok = mbar_wait(bar(DQ_V_EMPTY + vs), vph ^ 1u, p.status, 111, j);
        if (!ok) break;
        mbar_expect_tx(bar(DQ_V_FULL + vs), PL::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < PL::SUB; ++s) tma_load_4d(v_dst + s * PL::SUB_BYTES, &map_v, bar(DQ_V_FULL + vs), s * 64, j * BLK, hi, bi);
        issued_v = j + 1;
      }
      if (!ok) {  // let copies in flight land (bounded) before the CTA's memory is released
        mbar_wait(bar(DQ_QDO_FULL), 0, p.status, 112, 0);
        for (int j = max(0, issued_k - PL::K_STAGES); j < issued_k; ++j)
          mbar_wait(bar(DQ_K_FULL + j % PL::K_STAGES), (uint32_t)((j / PL::K_STAGES) & 1), p.status, 113, j);
        for (int j = max(0, issued_v - PL::V_STAGES); j < issued_v; ++j)
          mbar_wait(bar(DQ_V_FULL + j % PL::V_STAGES), (uint32_t)((j / PL::V_STAGES) & 1), p.status, 114, j);
      }
    }
  } else if (warp == WARP_MMA) {
    // The warp runs this role in lock step and one elected lane issues, so that addresses and
    // descriptors are warp-uniform values (fewer instructions per tcgen05.mma for the issuing thread).
    {
      const uint32_t leader = elect_one() ? 1u : 0u;
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr uint32_t IDESC_NT = make_idesc_fmt(BLK, BLK, 0, 0, FMT);  // both operands K-major
      constexpr uint32_t IDESC_DQ = make_idesc_fmt(BLK, HD, 0, 1, FMT);   // A from TMEM, B = K tile MN-major
      const uint32_t q_addr = smem_base + PL::OFF_RES0, do_addr = smem_base + PL::OFF_RES1;
      // D = A B^T over the head dimension, both operands K-major in shared memory; split mode: hi.hi + hi.lo + lo.hi
      auto issue_nt = [&](uint32_t d_col, uint32_t a_addr, uint32_t b_addr) {
        if constexpr (SPLIT) {
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            const uint32_t oa = term == 2 ? PL::SUB_BYTES : 0u, ob = term == 1 ? PL::SUB_BYTES : 0u;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk)
              umma_ss_if<false>(leader, tmem_u + d_col, make_desc(a_addr + oa + kk * 32, 16, 1024), make_desc(b_addr + ob + kk * 32, 16, 1024),
                                IDESC_NT, (term > 0 || kk > 0) ? 1u : 0u);
          }
        } else {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = (kk / 4) * PL::SUB_BYTES + (kk % 4) * 32;
            umma_ss_if<false>(leader, tmem_u + d_col, make_desc(a_addr + off, 16, 1024), make_desc(b_addr + off, 16, 1024), IDESC_NT, kk > 0);
          }
        }
      };
      auto issue_sdp = [&](int j) {
        const uint32_t k_addr = smem_base + PL::OFF_KRING + (j % PL::K_STAGES) * PL::TILE_BYTES;
        const uint32_t v_addr = smem_base + PL::OFF_VRING + (j % PL::V_STAGES) * PL::TILE_BYTES;
        issue_nt(C_S, q_addr, k_addr);
        issue_nt(C_DP, do_addr, v_addr);
      };
      ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_QDO_FULL), 0, p.status, 120, 0));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_K_FULL + 0), 0, p.status, 121, 0));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_V_FULL + 0), 0, p.status, 122, 0));
      if (ok) {
        tc_fence_after();
        issue_sdp(0);
        umma_commit_if(leader, bar(DQ_SDP_FULL));
        umma_commit_if(leader, bar(DQ_V_EMPTY + 0));
      }
      for (int j = 0; j < n && ok; ++j) {
        const int jn = j + 1;
        if (j + 1 < n) {
          // next S / dP as soon as the element-wise warps hold the current ones in registers
          ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_SDP_FREE), (uint32_t)(j & 1), p.status, 123, j));
          if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_K_FULL + jn % PL::K_STAGES), (uint32_t)((jn / PL::K_STAGES) & 1), p.status, 124, j));
          if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_V_FULL + jn % PL::V_STAGES), (uint32_t)((jn / PL::V_STAGES) & 1), p.status, 125, j));
          if (!ok) break;
          tc_fence_after();
          issue_sdp(jn);
          umma_commit_if(leader, bar(DQ_SDP_FULL));
          umma_commit_if(leader, bar(DQ_V_EMPTY + jn % PL::V_STAGES));
        }
        ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_DS_READY), (uint32_t)(j & 1), p.status, 126, j));
        if (!ok) break;
        tc_fence_after();
        const uint32_t k_addr = smem_base + PL::OFF_KRING + (j % PL::K_STAGES) * PL::TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk) {
          umma_ts_if<false>(leader, tmem_u + C_DQ, tmem_u + C_DS + kk * 8, make_desc(k_addr + kk * 2048, PL::SUB_BYTES, 1024), IDESC_DQ,
                  (j > 0 || kk > 0) ? 1u : 0u);
          if constexpr (SPLIT) {   // + dS_hi K_lo + dS_lo K_hi
            umma_ts_if<false>(leader, tmem_u + C_DQ, tmem_u + C_DS + kk * 8, make_desc(k_addr + PL::SUB_BYTES + kk * 2048, PL::SUB_BYTES, 1024),
                              IDESC_DQ, 1u);
            umma_ts_if<false>(leader, tmem_u + C_DQ, tmem_u + C_DS + 64 + kk * 8, make_desc(k_addr + kk * 2048, PL::SUB_BYTES, 1024), IDESC_DQ, 1u);
          }
        }
        umma_commit_if(leader, bar(DQ_DQ_DONE));
        umma_commit_if(leader, bar(DQ_K_EMPTY + j % PL::K_STAGES));
      }
      umma_commit_if(leader, bar(DQ_DRAIN));
      mbar_wait(bar(DQ_DRAIN), 0, p.status, 127, 0);
    }
  } else {
    // ------------------------------------------------------------------ element-wise warps
    const int qtr = warp >> 2, lane_base = (warp & 3) * 32, row = lane_base + lane;
    const int qi = q0 + row;
    constexpr int OC = HD / 4;
    const uint32_t t_row = tmem_base + ((uint32_t)lane_base << 16);
    const bool row_ok = qi < T;
    const float lse = row_ok ? p.lse[(int64_t)bh * T + qi] : 0.f;
    const float delta = row_ok ? p.delta[(int64_t)bh * T + qi] : 0.f;
    for (int j = 0; j < n && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_SDP_FULL), (uint32_t)(j & 1), p.status, 130, j));
      if (!ok) break;
      tc_fence_after();
      uint32_t s[32], dp[32];
      tmem_ld32(t_row + C_S + qtr * 32, s);
      tmem_ld32(t_row + C_DP + qtr * 32, dp);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DQ_SDP_FREE));
      const int k0 = j * BLK + qtr * 32;
      const bool edge = (p.causal && j * BLK + BLK - 1 > q0) || (j * BLK + BLK > T);
      uint32_t mw = 0xffffffffu;          // keep-bits of this thread's 32 keys
      float p_masked = 0.f;
      if constexpr (MASKED) {
        mw = __ldg(p.mask_bits + (int64_t)bi * p.mask_batch_stride + (int64_t)min(qi, T - 1) * p.mask_row_stride + 4 * j + qtr);
        p_masked = (row_ok && lse == INFINITY) ? p.inv_T : 0.f;
      }
      // dS = P o (dP - delta) scale with P = 2^(S scale_log2 - lse); adjacent keys go through as fp32 pairs.
      // Split mode: S and dP carry the pre-pass's scales; dS is kept in the units of dP' x 2^-19 and the factor
      // scale x 2^19 / (s_dy s_v s_k) is applied once to dQ.
      const float sl2 = SPLIT ? p.scale_log2 * __ldg(p.fac + split::FAC_INV_QK) : p.scale_log2;
      const float dmul = SPLIT ? DS_SHIFT : p.scale;
      const float dsub = SPLIT ? delta * __ldg(p.fac + split::FAC_DYV) * DS_SHIFT : delta * p.scale;
      const float2 sc2 = make_float2(sl2, sl2), nl2 = make_float2(-lse, -lse);
      const float2 ps2 = make_float2(dmul, dmul), nd2 = make_float2(-dsub, -dsub);
      const float2 zero2 = make_float2(0.f, 0.f);
      uint32_t pk[16];
      uint32_t pk_lo[SPLIT ? 16 : 1];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float2 x = ffma2(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), sc2, nl2);
        const float2 g = ffma2(make_float2(__uint_as_float(dp[i]), __uint_as_float(dp[i + 1])), ps2, nd2);
        float e0 = fast_exp2(x.x), e1 = fast_exp2(x.y);
        if constexpr (MASKED) {
          if (((mw >> i) & 1u) == 0u) e0 = p_masked;
          if (((mw >> (i + 1)) & 1u) == 0u) e1 = p_masked;
        }
        const float2 d = ffma2(make_float2(e0, e1), g, zero2);
        float d0 = d.x, d1 = d.y;
        if (edge) {
          const int kj = k0 + i;
          if (!row_ok || kj >= T || (p.causal && kj > qi)) d0 = 0.f;
          if (!row_ok || kj + 1 >= T || (p.causal && kj + 1 > qi)) d1 = 0.f;
        } else if (!row_ok) { d0 = 0.f; d1 = 0.f; }
        if constexpr (SPLIT) split_pack(d0, d1, pk[i / 2], pk_lo[i / 2]);
        else pk[i / 2] = pack_bf16(d0, d1);
      }
      if (j > 0) {  // the previous dQ product must have consumed the previous dS
        ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_DQ_DONE), (uint32_t)((j - 1) & 1), p.status, 131, j));
        if (!ok) break;
        tc_fence_after();
      }
      tmem_st16(t_row + C_DS + qtr * 16, pk);
      if constexpr (SPLIT) tmem_st16(t_row + C_DS + 64 + qtr * 16, pk_lo);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DQ_DS_READY));
    }
    if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_DQ_DONE), (uint32_t)((n - 1) & 1), p.status, 132, n));
    constexpr int ESZ = SPLIT ? 4 : 2, PR = HD * ESZ / 16;
    uint8_t* tile = smem_gen + PL::OFF_RES0;           // the Q tile: every product has finished with it
    const bool fin = ok && n > 0;
    if (fin) {
      tc_fence_after();
      const float mul = SPLIT ? p.scale * DS_UNSHIFT * __ldg(p.fac + split::FAC_INV_DYVK) : 1.0f;
      stage_columns<PR, OC, SPLIT>(tile, row, qtr, t_row + C_DQ + qtr * OC, mul);
    }
    ew_bar_sync();
    if (fin)
      store_staged_rows<PR, ESZ>(tile, warp, lane, p.out0, (int64_t)bi * p.os.b + (int64_t)hi * p.os.h + (int64_t)q0 * p.os.t, p.os.t,
                                 min(BLK, T - q0));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
  mca_pdl_wait();   // see the set-up: complete only after the kernels before it
}

// ---------------------------------------------------------------------------------------------
// dK/dV kernel.  TMEM columns: S^T [0,128)  dP^T [128,256)  dV [256,256+HD)  dK [384,384+HD);
// P^T and dS^T (bf16, packed) overwrite the first 16 columns of each 32-column quarter of S^T / dP^T; in split
// mode their fp16 hi halves do, and the lo halves take the other 16 columns of the quarter.
// ---------------------------------------------------------------------------------------------
enum KvBar : int {
  KV_KV_FULL = 0,
  KV_Q_FULL = 1,     // [3]  Q of a step (lives until the step's dK product: one stage deeper than dY)
  KV_Q_EMPTY = 4,    // [3]
  KV_DO_FULL = 7,    // [2]  dY of a step (last used by the step's dV product)
  KV_DO_EMPTY = 9,   // [2]
  KV_ST_FULL = 11,   // S^T written by the MMA
  KV_PT_READY = 12,  // P^T written to TMEM (over S^T)
  KV_ACC_DONE = 13,  // dV / dK products of the step finished
  KV_DRAIN = 14,
  KV_LD_READY = 15,  // the step's per-query log-sum-exp and delta are staged in shared memory
  KV_DPT_FULL = 16,  // dP^T written by the MMA
  KV_DST_READY = 17, // dS^T written to TMEM (over dP^T)
  KV_BAR_COUNT = 18
};

template <int HD, bool SPLIT, bool MASKED>
__global__ void __launch_bounds__(BW_THREADS, 1)
sdpa_bwd_dkdv_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                        const BwdParams p) {
  using PL = BwdPlan<SPLIT ? 128 : HD>;
  constexpr int FMT = SPLIT ? 0 : 1;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar0 = smem_base + PL::OFF_BAR_DQ;   // same seven-tile plan as the dQ kernel: Q ring where it has K, dY ring where it has V
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + PL::OFF_BAR_DQ + KV_BAR_COUNT * 8);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // launch order -> work item: longest causal work first inside groups of p.group heads (see the forward kernel)
  const int lin = (int)(blockIdx.y * gridDim.x + blockIdx.x);
  const int grp = lin / (p.group * (int)gridDim.x);
  const int in_grp = lin - grp * p.group * (int)gridDim.x;
  const int grp_heads = min(p.group, (int)gridDim.y - grp * p.group);
  const int rank = in_grp / grp_heads;
  const int bh = grp * p.group + (in_grp - rank * grp_heads), T = p.T;
  const int bi = bh / p.H, hi = bh - bi * p.H;   // batch item and head
  const int kt = rank;                  // key tile; tile 0 has the most causal work and comes first
  const int k0 = kt * BLK;
  const int n_q_tiles = (T + BLK - 1) / BLK;
  const int i_begin = p.causal ? kt : 0;
  const int n = n_q_tiles - i_begin;    // query tiles to walk

  // the aligned plan must fit in what was requested (it does unless the dynamic base is unusually placed)
  uint32_t dyn_bytes;
  asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
  if (smem_base + PL::NEED_KV > smem_u32(smem_raw) + dyn_bytes) {
    if (tid == 0 && atomicCAS(p.status, 0, 2) == 0) { p.status[1] = 299; p.status[2] = (int)(smem_base - smem_u32(smem_raw)); }
    return;
  }
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem_gen + PL::OFF_FLAG_KV);
  if (tid == 32) *s_abort = *reinterpret_cast<volatile int*>(p.status);
  if (warp == WARP_TMA && lane == 0) {
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v); prefetch_tensormap(&map_do);
  }
  if (tid == 0) {
    for (int i = 0; i < KV_BAR_COUNT; ++i) mbar_init(bar(i), (i == KV_PT_READY || i == KV_LD_READY || i == KV_DST_READY) ? (uint32_t)EW_WARPS : 1u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == WARP_MMA) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  mca_pdl_wait();   // launched ahead of the kernels before it: from here on their results are complete and visible
  mca_pdl_launch_dependents();   // only now: the dQ kernel behind this one starts without a wait of its own
  if (*s_abort != 0) {   // an earlier CTA already failed: leave (uniform decision) before any copy or product is issued
    if (warp == WARP_MMA) tmem_dealloc(tmem_base, TMEM_COLS);
    return;
  }
  constexpr uint32_t C_ST = 0, C_DPT = 128, C_DV = 256, C_DK = 384;
  bool ok = true;

  if (warp == WARP_TMA) {
    if (lane == 0) {
      mbar_expect_tx(bar(KV_KV_FULL), 2 * PL::TILE_BYTES);
#pragma unroll
      for (int s = 0; s < PL::SUB; ++s) {
        tma_load_4d(smem_base + PL::OFF_RES0 + s * PL::SUB_BYTES, &map_k, bar(KV_KV_FULL), s * 64, k0, hi, bi);
        tma_load_4d(smem_base + PL::OFF_RES1 + s * PL::SUB_BYTES, &map_v, bar(KV_KV_FULL), s * 64, k0, hi, bi);
      }
      int issued = 0, issued_do = 0;
      for (int it = 0; it < n && ok; ++it) {
        const int qs = it % PL::K_STAGES, ds = it % PL::V_STAGES;
        const uint32_t qph = (uint32_t)((it / PL::K_STAGES) & 1), dph = (uint32_t)((it / PL::V_STAGES) & 1);
        const uint32_t q_dst = smem_base + PL::OFF_KRING + qs * PL::TILE_BYTES, do_dst = smem_base + PL::OFF_VRING + ds * PL::TILE_BYTES;
        ok = mbar_wait(bar(KV_Q_EMPTY + qs), qph ^ 1u, p.status, 210, it);
        if (!ok) break;
        mbar_expect_tx(bar(KV_Q_FULL + qs), PL::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < PL::SUB; ++s)
          tma_load_4d(q_dst + s * PL::SUB_BYTES, &map_q, bar(KV_Q_FULL + qs), s * 64, (i_begin + it) * BLK, hi, bi);
        issued = it + 1;
        ok = mbar_wait(bar(KV_DO_EMPTY + ds), dph ^ 1u, p.status, 211, it);
        if (!ok) break;
        mbar_expect_tx(bar(KV_DO_FULL + ds), PL::TILE_BYTES);
#pragma unroll
        for (int s = 0; s < PL::SUB; ++s)
          tma_load_4d(do_dst + s * PL::SUB_BYTES, &map_do, bar(KV_DO_FULL + ds), s * 64, (i_begin + it) * BLK, hi, bi);
        issued_do = it + 1;
      }
      if (!ok) {
        mbar_wait(bar(KV_KV_FULL), 0, p.status, 212, 0);
        for (int it = max(0, issued - PL::K_STAGES); it < issued; ++it)
          mbar_wait(bar(KV_Q_FULL + it % PL::K_STAGES), (uint32_t)((it / PL::K_STAGES) & 1), p.status, 213, it);
        for (int it = max(0, issued_do - PL::V_STAGES); it < issued_do; ++it)
          mbar_wait(bar(KV_DO_FULL + it % PL::V_STAGES), (uint32_t)((it / PL::V_STAGES) & 1), p.status, 214, it);
      }
    }
  } else if (warp == WARP_MMA) {
    // The warp runs this role in lock step and one elected lane issues, so that addresses and
    // descriptors are warp-uniform values (fewer instructions per tcgen05.mma for the issuing thread).
    {
      const uint32_t leader = elect_one() ? 1u : 0u;
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr uint32_t IDESC_NT = make_idesc_fmt(BLK, BLK, 0, 0, FMT);
      constexpr uint32_t IDESC_ACC = make_idesc_fmt(BLK, HD, 0, 1, FMT);
      const uint32_t k_addr = smem_base + PL::OFF_RES0, v_addr = smem_base + PL::OFF_RES1;
      auto issue_nt = [&](uint32_t d_col, uint32_t a_addr, uint32_t b_addr) {
        if constexpr (SPLIT) {
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            const uint32_t oa = term == 2 ? PL::SUB_BYTES : 0u, ob = term == 1 ? PL::SUB_BYTES : 0u;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk)
              umma_ss_if<false>(leader, tmem_u + d_col, make_desc(a_addr + oa + kk * 32, 16, 1024), make_desc(b_addr + ob + kk * 32, 16, 1024),
                                IDESC_NT, (term > 0 || kk > 0) ? 1u : 0u);
          }
        } else {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = (kk / 4) * PL::SUB_BYTES + (kk % 4) * 32;
            umma_ss_if<false>(leader, tmem_u + d_col, make_desc(a_addr + off, 16, 1024), make_desc(b_addr + off, 16, 1024), IDESC_NT, kk > 0);
          }
        }
      };
      // acc += A^T-from-TMEM x B with B a 128 x HD tile read MN-major; split mode: hi.hi + hi.lo + lo.hi
      auto issue_acc = [&](uint32_t d_col, uint32_t a_col, uint32_t b_addr, bool first_step) {
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk) {
          const uint32_t a_hi = tmem_u + a_col + (kk / 2) * 32 + (kk % 2) * 8;
          umma_ts_if<false>(leader, tmem_u + d_col, a_hi, make_desc(b_addr + kk * 2048, PL::SUB_BYTES, 1024), IDESC_ACC,
                            (!first_step || kk > 0) ? 1u : 0u);
          if constexpr (SPLIT) {
            umma_ts_if<false>(leader, tmem_u + d_col, a_hi, make_desc(b_addr + PL::SUB_BYTES + kk * 2048, PL::SUB_BYTES, 1024), IDESC_ACC, 1u);
            umma_ts_if<false>(leader, tmem_u + d_col, a_hi + 16, make_desc(b_addr + kk * 2048, PL::SUB_BYTES, 1024), IDESC_ACC, 1u);
          }
        }
      };
      // S^T = K Q^T and dP^T = V dY^T (rows = keys, columns = queries); P^T overwrites S^T and dS^T overwrites
      // dP^T.  The two halves of a step are interleaved with the next step's first products,
      //   dV(it), S^T(it+1), dK(it), dP^T(it+1),
      // (the in-order pipe keeps every product behind the one that still reads the columns it overwrites),
      // so the element-wise warps work on P^T(it+1) while dK(it) and dP^T(it+1) run.
      auto q_stage = [&](int it) { return smem_base + PL::OFF_KRING + (it % PL::K_STAGES) * PL::TILE_BYTES; };
      auto do_stage = [&](int it) { return smem_base + PL::OFF_VRING + (it % PL::V_STAGES) * PL::TILE_BYTES; };
      auto wait_q = [&](int it) {
        return __all_sync(0xffffffffu, mbar_wait(bar(KV_Q_FULL + it % PL::K_STAGES), (uint32_t)((it / PL::K_STAGES) & 1), p.status, 221, it));
      };
      auto wait_do = [&](int it) {
        return __all_sync(0xffffffffu, mbar_wait(bar(KV_DO_FULL + it % PL::V_STAGES), (uint32_t)((it / PL::V_STAGES) & 1), p.status, 224, it));
      };
      auto issue_st = [&](int it) {
        issue_nt(C_ST, k_addr, q_stage(it));
        umma_commit_if(leader, bar(KV_ST_FULL));
      };
      auto issue_dpt = [&](int it) {
        issue_nt(C_DPT, v_addr, do_stage(it));
        umma_commit_if(leader, bar(KV_DPT_FULL));
      };
      ok = __all_sync(0xffffffffu, mbar_wait(bar(KV_KV_FULL), 0, p.status, 220, 0));
      if (ok && n > 0) {
        ok = wait_q(0);
        if (ok) ok = wait_do(0);
        if (ok) {
          tc_fence_after();
          issue_st(0);
          issue_dpt(0);
        }
      }
      for (int it = 0; it < n && ok; ++it) {
        const uint32_t q_addr = q_stage(it), do_addr = do_stage(it);
        // dV += P^T dY: A from TMEM (16 queries = 8 packed columns per step), B MN-major
        ok = __all_sync(0xffffffffu, mbar_wait(bar(KV_PT_READY), (uint32_t)(it & 1), p.status, 222, it));
        if (!ok) break;
        tc_fence_after();
        issue_acc(C_DV, C_ST, do_addr, it == 0);
        umma_commit_if(leader, bar(KV_DO_EMPTY + it % PL::V_STAGES));   // dY(it) was last read by this product
        if (it + 1 < n) {
          ok = wait_q(it + 1);
          if (!ok) break;
          tc_fence_after();
          issue_st(it + 1);
        }
        // dK += dS^T Q
        ok = __all_sync(0xffffffffu, mbar_wait(bar(KV_DST_READY), (uint32_t)(it & 1), p.status, 223, it));
        if (!ok) break;
        tc_fence_after();
        issue_acc(C_DK, C_DPT, q_addr, it == 0);
        umma_commit_if(leader, bar(KV_Q_EMPTY + it % PL::K_STAGES));
        umma_commit_if(leader, bar(KV_ACC_DONE));
        if (it + 1 < n) {
          ok = wait_do(it + 1);
          if (!ok) break;
          tc_fence_after();
          issue_dpt(it + 1);
        }
      }
      umma_commit_if(leader, bar(KV_DRAIN));
      mbar_wait(bar(KV_DRAIN), 0, p.status, 227, 0);
    }
  } else {
    // ------------------------------------------------------------------ element-wise warps
    const int qtr = warp >> 2, lane_base = (warp & 3) * 32, row = lane_base + lane;
    const int kj = k0 + row;               // this thread's key
    constexpr int OC = HD / 4;
    const uint32_t t_row = tmem_base + ((uint32_t)lane_base << 16);
    const bool key_ok = kj < T;
    // The query-dependent terms (minus log-sum-exp, minus delta x scale) are the same for every key row: the first 256
    // element-wise threads fetch one value each a step ahead and stage them in shared memory, so that the
    // inner loop reads them as broadcasts instead of 64 global loads per thread.  Rows beyond T get
    // lse = +inf, which makes their probabilities exactly zero.
    float (*s_nlse)[BLK] = reinterpret_cast<float (*)[BLK]>(smem_gen + PL::OFF_STAGE_KV);
    float (*s_del)[BLK] = s_nlse + 2;
    // split mode: S^T and dP^T carry the pre-pass's scales; dS^T is kept in the units of dP' x 2^-19 and P^T 2^10 larger
    const float sl2 = SPLIT ? p.scale_log2 * __ldg(p.fac + split::FAC_INV_QK) : p.scale_log2;
    const float dmul = SPLIT ? DS_SHIFT : p.scale;
    const float del_mul = SPLIT ? __ldg(p.fac + split::FAC_DYV) * DS_SHIFT : p.scale;
    auto fetch = [&](int it) -> float {
      const int qi = (i_begin + it) * BLK + (tid & (BLK - 1));
      if (tid >= 2 * BLK || it >= n || qi >= T) return tid < BLK ? -INFINITY : 0.f;
      return tid < BLK ? -__ldg(p.lse + (int64_t)bh * T + qi) : -__ldg(p.delta + (int64_t)bh * T + qi) * del_mul;
    };
    auto stage = [&](int it, float v) {
      if (tid < BLK) s_nlse[it & 1][tid] = v;
      else if (tid < 2 * BLK) s_del[it & 1][tid - BLK] = v;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(KV_LD_READY));
    };
    if (n > 0) stage(0, fetch(0));
    for (int it = 0; it < n && ok; ++it) {
      const int q_local = qtr * 32;                         // first of this thread's 32 queries within the tile
      const int q_base = (i_begin + it) * BLK + q_local;
      const float next = fetch(it + 1);                     // in flight while this step is processed
      ok = __all_sync(0xffffffffu, mbar_wait(bar(KV_LD_READY), (uint32_t)(it & 1), p.status, 231, it));
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(KV_ST_FULL), (uint32_t)(it & 1), p.status, 230, it));
      if (!ok) break;
      tc_fence_after();
      const float* nlse_s = s_nlse[it & 1] + q_local;
      const float* del_s = s_del[it & 1] + q_local;
      const bool diag = p.causal && (i_begin + it) * BLK < k0 + BLK;   // only the diagonal tile needs the causal test
      uint32_t mw = 0xffffffffu;          // keep-bits of this thread's key against its 32 queries of the step
      if constexpr (MASKED) {
        if (p.mask_bits_t != nullptr)
          mw = __ldg(p.mask_bits_t + (int64_t)min(kj, T - 1) * p.mask_row_stride + 4 * (i_begin + it) + qtr);
        else
          mw = ((__ldg(p.mask_bits + (int64_t)bi * p.mask_batch_stride + (min(kj, T - 1) >> 5)) >> (kj & 31)) & 1u) ? 0xffffffffu : 0u;
      }
      // pass 1: P^T = 2^(S^T scale - lse), kept in fp32 for pass 2, packed to bf16 over S^T (fp32 pairs)
      const float2 sc2 = make_float2(sl2, sl2), ps2 = make_float2(dmul, dmul);
      const float2 zero2 = make_float2(0.f, 0.f);
      uint32_t s[32], pk[16];
      uint32_t pk_lo[SPLIT ? 16 : 1];
      tmem_ld32(t_row + C_ST + qtr * 32, s);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const float4 nl = *reinterpret_cast<const float4*>(nlse_s + i);
        const float nls[4] = {nl.x, nl.y, nl.z, nl.w};
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
          const float2 x = ffma2(make_float2(__uint_as_float(s[i + e]), __uint_as_float(s[i + e + 1])), sc2,
                                 make_float2(nls[e], nls[e + 1]));
          float v0 = fast_exp2(x.x), v1 = fast_exp2(x.y);
          if constexpr (MASKED) {
            // a masked entry: 0, or 1 / T in a fully masked row (staged -lse = -inf; rows beyond T are staged the same
            // way and stay 0)
            if (((mw >> (i + e)) & 1u) == 0u) v0 = (nls[e] == -INFINITY && q_base + i + e < T) ? p.inv_T : 0.f;
            if (((mw >> (i + e + 1)) & 1u) == 0u) v1 = (nls[e + 1] == -INFINITY && q_base + i + e + 1 < T) ? p.inv_T : 0.f;
          }
          if (!key_ok || (diag && kj > q_base + i + e)) v0 = 0.f;
          if (!key_ok || (diag && kj > q_base + i + e + 1)) v1 = 0.f;
          s[i + e] = __float_as_uint(v0);
          s[i + e + 1] = __float_as_uint(v1);
        }
        if constexpr (SPLIT) {
          split_pack(__uint_as_float(s[i]) * PT_SHIFT, __uint_as_float(s[i + 1]) * PT_SHIFT, pk[i / 2], pk_lo[i / 2]);
          split_pack(__uint_as_float(s[i + 2]) * PT_SHIFT, __uint_as_float(s[i + 3]) * PT_SHIFT, pk[i / 2 + 1], pk_lo[i / 2 + 1]);
        } else {
          pk[i / 2] = pack_bf16(__uint_as_float(s[i]), __uint_as_float(s[i + 1]));
          pk[i / 2 + 1] = pack_bf16(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
        }
      }
      tmem_st16(t_row + C_ST + qtr * 32, pk);
      if constexpr (SPLIT) tmem_st16(t_row + C_ST + qtr * 32 + 16, pk_lo);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(KV_PT_READY));
      // pass 2: dS^T = P^T o (dP^T - delta) scale, packed to bf16 over dP^T
      ok = __all_sync(0xffffffffu, mbar_wait(bar(KV_DPT_FULL), (uint32_t)(it & 1), p.status, 233, it));
      if (!ok) break;
      tc_fence_after();
      uint32_t dp[32];
      tmem_ld32(t_row + C_DPT + qtr * 32, dp);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const float4 de = *reinterpret_cast<const float4*>(del_s + i);
        const float des[4] = {de.x, de.y, de.z, de.w};
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
          // (dP - delta) scale as one fused pair operation, then times P
          const float2 g = ffma2(make_float2(__uint_as_float(dp[i + e]), __uint_as_float(dp[i + e + 1])), ps2,
                                 make_float2(des[e], des[e + 1]));
          const float2 d = ffma2(make_float2(__uint_as_float(s[i + e]), __uint_as_float(s[i + e + 1])), g, zero2);
          if constexpr (SPLIT) split_pack(d.x, d.y, pk[(i + e) / 2], pk_lo[(i + e) / 2]);
          else pk[(i + e) / 2] = pack_bf16(d.x, d.y);
        }
      }
      if (it + 1 < n) stage(it + 1, next);
      tmem_st16(t_row + C_DPT + qtr * 32, pk);
      if constexpr (SPLIT) tmem_st16(t_row + C_DPT + qtr * 32 + 16, pk_lo);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(KV_DST_READY));
    }
    if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar(KV_ACC_DONE), (uint32_t)((n - 1) & 1), p.status, 232, n));
    constexpr int ESZ = SPLIT ? 4 : 2, PR = HD * ESZ / 16;
    uint8_t* tile_k = smem_gen + PL::OFF_RES0;         // the K and V tiles: every product has finished with them
    uint8_t* tile_v = smem_gen + PL::OFF_RES1;
    const bool fin = ok && n > 0;
    if (fin) {
      tc_fence_after();
      const float mul_k = SPLIT ? p.scale * DS_UNSHIFT * __ldg(p.fac + split::FAC_INV_DYVQ) : 1.0f;
      const float mul_v = SPLIT ? PT_UNSHIFT * __ldg(p.fac + split::FAC_INV_DY) : 1.0f;
      stage_columns<PR, OC, SPLIT>(tile_k, row, qtr, t_row + C_DK + qtr * OC, mul_k);
      stage_columns<PR, OC, SPLIT>(tile_v, row, qtr, t_row + C_DV + qtr * OC, mul_v);
    }
    ew_bar_sync();
    if (fin) {
      const int64_t off0 = (int64_t)bi * p.os.b + (int64_t)hi * p.os.h + (int64_t)k0 * p.os.t;
      store_staged_rows<PR, ESZ>(tile_k, warp, lane, p.out0, off0, p.os.t, min(BLK, T - k0));
      store_staged_rows<PR, ESZ>(tile_v, warp, lane, p.out1, off0, p.os.t, min(BLK, T - k0));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// delta[row] = sum_c dY[row][c] * Y[row][c]  (bf16 inputs, fp32 result).  D / 8 lanes share a row (16-byte loads), so a
// warp covers 256 / D rows.
__global__ void bwd_delta_bf16_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ y,
                                      int64_t rows, int H, int T, int D, const McaStrides ys, float* __restrict__ delta) {
  mca_pdl_launch_dependents();
  mca_pdl_wait();   // dy and y are earlier kernels' output
  const int lane = threadIdx.x & 31, g = D / 8, rpw = 32 / g;        // g in {8, 16}
  const int64_t row = ((int64_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5)) * rpw + lane / g;
  float acc = 0.f;
  if (row < rows) {
    const unsigned bh = (unsigned)(row / T), bi = bh / (unsigned)H;
    const int64_t off = (int64_t)bi * ys.b + (int64_t)(bh - bi * H) * ys.h + (row - (int64_t)bh * T) * ys.t + (lane % g) * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(dy + off);       // y and dy share the output layout
    const uint4 b = *reinterpret_cast<const uint4*>(y + off);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
      const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[i]));
      acc = fmaf(fa.x, fb.x, fmaf(fa.y, fb.y, acc));
    }
  }
  for (int o = g / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (row < rows && lane % g == 0) delta[row] = acc;
}

// Both kernels of one backward, with or without the caller's mask.
template <int HD, bool SPLIT, bool MASKED>
int launch_bwd_pair(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo, BwdParams p,
                    void* dq, void* dk, void* dv, int B, int H, int T, cudaStream_t st) {
  using PL = BwdPlan<SPLIT ? 128 : HD>;
  const size_t smem_kv = PL::BYTES_KV, smem_dq = PL::BYTES_DQ;
  MCA_CUDA_TRY(cudaFuncSetAttribute(sdpa_bwd_dkdv_tc_kernel<HD, SPLIT, MASKED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv));
  MCA_CUDA_TRY(cudaFuncSetAttribute(sdpa_bwd_dq_tc_kernel<HD, SPLIT, MASKED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq));
  dim3 grid(mca_ceil_div(T, BLK), B * H);
  p.out0 = dk; p.out1 = dv;
  int e = mca_launch_pdl(sdpa_bwd_dkdv_tc_kernel<HD, SPLIT, MASKED>, grid, dim3(BW_THREADS), smem_kv, st, mq, mk, mv, mdo, p);
  if (e) return e;
  p.out0 = dq; p.out1 = nullptr;
  return mca_launch_pdl(sdpa_bwd_dq_tc_kernel<HD, SPLIT, MASKED>, grid, dim3(BW_THREADS), smem_dq, st, mq, mk, mv, mdo, p);
}

void set_mask(BwdParams& p, const McaMaskBits* mask, int T) {
  p.mask_bits = mask ? mask->bits : nullptr;
  p.mask_bits_t = mask ? mask->bits_t : nullptr;
  p.mask_batch_stride = mask ? mask->batch_stride : 0;
  p.mask_row_stride = mask ? mask->row_stride : 0;
  p.inv_T = 1.0f / (float)T;
}

template <int HD>
int launch_bwd(const void* q, const void* k, const void* v, const void* dy, const float* lse, const float* delta,
               int causal, int B, int H, int T, void* dq, void* dk, void* dv, int* status, int layout, cudaStream_t st,
               const McaMaskBits* mask = nullptr) {
  if (mask != nullptr && causal) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  CUtensorMap mq, mk, mv, mdo;
  int e;
  const McaStrides sin = mca_in_strides(layout, H, T, HD), sout = mca_out_strides(layout, H, T, HD);
  if ((e = make_map_bf16(&mq, q, B, H, T, HD, sin)) || (e = make_map_bf16(&mk, k, B, H, T, HD, sin)) ||
      (e = make_map_bf16(&mv, v, B, H, T, HD, sin)) || (e = make_map_bf16(&mdo, dy, B, H, T, HD, sout)))
    return e;
  BwdParams p;
  p.fac = nullptr;
  p.lse = lse; p.delta = delta; p.status = status; p.T = T; p.causal = causal; p.H = H;
  {
    // Q, K, V, dY of one (batch, head): keep a group's set under about 64 MB of the 126 MB L2
    const int64_t g = (64ll << 20) / ((int64_t)4 * T * HD * 2);
    p.group = causal ? (int)std::max<int64_t>(1, std::min<int64_t>(g, (int64_t)B * H)) : 1;
  }
  p.os = sin;
  p.scale = 1.0f / sqrtf((float)HD);
  p.scale_log2 = p.scale * 1.4426950408889634f;
  set_mask(p, mask, T);
  if (mask != nullptr) return launch_bwd_pair<HD, false, true>(mq, mk, mv, mdo, p, dq, dk, dv, B, H, T, st);
  return launch_bwd_pair<HD, false, false>(mq, mk, mv, mdo, p, dq, dk, dv, B, H, T, st);
}

// Split-operand backward for fp32 callers.  The workspace still holds the fp16 halves of q, k, v the forward's pre-pass
// wrote; dY is split here.
template <int HD>
int launch_bwd_split(const float* dy, const float* y_copy, const float* lse, float* delta, int causal, int B, int H, int T,
                     float* dq, float* dk, float* dv, void* workspace, int* status, int layout, cudaStream_t st,
                     const McaMaskBits* mask = nullptr) {
  if (mask != nullptr && causal) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  const int64_t rows = (int64_t)B * H * T;
  const split::Workspace w = split::carve(workspace, rows);
  const McaStrides sin = mca_in_strides(layout, H, T, HD), sout = mca_out_strides(layout, H, T, HD);
  split::Job job;
  job.src[0] = dy; job.dst[0] = w.tensor[split::TENSOR_DY]; job.slot[0] = split::TENSOR_DY;
  job.src[1] = job.src[2] = nullptr; job.dst[1] = job.dst[2] = nullptr; job.slot[1] = job.slot[2] = 0;
  // the kernel that splits dY also forms delta = rowsum(dY o Y) from the elements it holds
  int e = split::run<HD>(job, 1, sout, H, T, rows, w, true, st, y_copy, delta);
  if (e) return e;
  CUtensorMap mq, mk, mv, mdo;
  const McaStrides sp{(int64_t)H * T * 128, (int64_t)T * 128, 128};
  const CUtensorMap* maps[4] = {&mq, &mk, &mv, &mdo};
  for (int i = 0; i < 4; ++i)
    if ((e = make_map_4d(const_cast<CUtensorMap*>(maps[i]), w.tensor[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, B, H, T, 128, sp,
                         CU_TENSOR_MAP_SWIZZLE_128B)))
      return e;
  BwdParams p;
  p.fac = w.fac;
  p.lse = lse; p.delta = delta; p.status = status; p.T = T; p.causal = causal; p.H = H;
  {
    const int64_t g = (64ll << 20) / ((int64_t)4 * T * 256);
    p.group = causal ? (int)std::max<int64_t>(1, std::min<int64_t>(g, (int64_t)B * H)) : 1;
  }
  p.os = sin;
  p.scale = 1.0f / sqrtf((float)HD);
  p.scale_log2 = p.scale * 1.4426950408889634f;
  set_mask(p, mask, T);
  if (mask != nullptr) return launch_bwd_pair<HD, true, true>(mq, mk, mv, mdo, p, dq, dk, dv, B, H, T, st);
  return launch_bwd_pair<HD, true, false>(mq, mk, mv, mdo, p, dq, dk, dv, B, H, T, st);
}

}  // namespace

int mca_sdpa_backward_tc(const void* q, const void* k, const void* v, const void* y, const void* dy, const float* lse,
                         float* delta_scratch, int dtype, int causal, int B, int H, int T, int D, void* dq, void* dk,
                         void* dv, int* status, void* stream) {
  return mca_sdpa_backward_tc_layout(q, k, v, y, dy, lse, delta_scratch, dtype, causal, B, H, T, D, dq, dk, dv, status,
                                     MCA_LAYOUT_BHTD, stream);
}

int mca_sdpa_backward_tc_layout(const void* q, const void* k, const void* v, const void* y, const void* dy,
                                const float* lse, float* delta_scratch, int dtype, int causal, int B, int H, int T, int D,
                                void* dq, void* dk, void* dv, int* status, int layout, void* stream) {
  return mca_sdpa_backward_tc_masked(q, k, v, y, dy, lse, delta_scratch, dtype, causal, B, H, T, D, dq, dk, dv, status, layout,
                                     nullptr, nullptr, MCA_MASK_NONE, stream);
}

int mca_sdpa_backward_tc_masked(const void* q, const void* k, const void* v, const void* y, const void* dy, const float* lse,
                                float* delta_scratch, int dtype, int causal, int B, int H, int T, int D, void* dq, void* dk,
                                void* dv, int* status, int layout, const uint32_t* mask_bits, const uint32_t* mask_bits_t,
                                int mask_mode, void* stream) {
  McaMaskBits mb;
  const McaMaskBits* mask = nullptr;
  int me = mca_mask_bits_view(mask_bits, mask_bits_t, mask_mode, T, true, &mb, &mask);
  if (me) return me;
  if (layout != MCA_LAYOUT_BHTD && layout != MCA_LAYOUT_PACKED) return ERROR_PARAM_OUT_OF_RANGE;
  if (!q || !k || !v || !y || !dy || !lse || !delta_scratch || !dq || !dk || !dv || !status) return ERROR_PARAM_NULL;
  if (B <= 0 || H <= 0 || T <= 0 || (int64_t)B * H > 65535) return ERROR_PARAM_OUT_OF_RANGE;
  if (dtype != MCA_DTYPE_BF16) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
       reinterpret_cast<uintptr_t>(dv)) & 15)
    return ERROR_PARAM_OUT_OF_RANGE;
  if (D != 64 && D != 128) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows = (int64_t)B * H * T;
  int e;
  {
    const int64_t rows_per_block = 8 * (256 / D);   // eight warps, 256 / D rows each
    e = mca_launch_pdl(bwd_delta_bf16_kernel, dim3((unsigned)((rows + rows_per_block - 1) / rows_per_block)), dim3(256), 0, st,
                       (const __nv_bfloat16*)dy, (const __nv_bfloat16*)y, rows, H, T, D, mca_out_strides(layout, H, T, D), delta_scratch);
  }
  if (e) return e;
  if (D == 128) return launch_bwd<128>(q, k, v, dy, lse, delta_scratch, causal, B, H, T, dq, dk, dv, status, layout, st, mask);
  return launch_bwd<64>(q, k, v, dy, lse, delta_scratch, causal, B, H, T, dq, dk, dv, status, layout, st, mask);
}

int mca_sdpa_backward_f32_tc(const float* dy, const float* y_copy, const float* lse, float* delta_scratch, int causal, int B,
                             int H, int T, int D, float* dq, float* dk, float* dv, void* workspace, int64_t workspace_bytes,
                             int* status, int layout, void* stream) {
  return mca_sdpa_backward_f32_tc_masked(dy, y_copy, lse, delta_scratch, causal, B, H, T, D, dq, dk, dv, workspace, workspace_bytes,
                                         status, layout, nullptr, nullptr, MCA_MASK_NONE, stream);
}

int mca_sdpa_backward_f32_tc_masked(const float* dy, const float* y_copy, const float* lse, float* delta_scratch, int causal,
                                    int B, int H, int T, int D, float* dq, float* dk, float* dv, void* workspace,
                                    int64_t workspace_bytes, int* status, int layout, const uint32_t* mask_bits,
                                    const uint32_t* mask_bits_t, int mask_mode, void* stream) {
  McaMaskBits mb;
  const McaMaskBits* mask = nullptr;
  int me = mca_mask_bits_view(mask_bits, mask_bits_t, mask_mode, T, true, &mb, &mask);
  if (me) return me;
  if (layout != MCA_LAYOUT_BHTD && layout != MCA_LAYOUT_PACKED) return ERROR_PARAM_OUT_OF_RANGE;
  if (!dy || !y_copy || !lse || !delta_scratch || !dq || !dk || !dv || !workspace || !status) return ERROR_PARAM_NULL;
  if (B <= 0 || H <= 0 || T <= 0 || (int64_t)B * H > 65535) return ERROR_PARAM_OUT_OF_RANGE;
  if (!mca_sdpa_backward_f32_tc_supported(D)) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  if (workspace_bytes < mca_sdpa_forward_f32_tc_workspace_bytes(B, H, T)) return ERROR_ATTN_SCRATCH_TOO_SMALL;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
       reinterpret_cast<uintptr_t>(dv) | reinterpret_cast<uintptr_t>(workspace)) & 15)
    return ERROR_PARAM_OUT_OF_RANGE;
  cudaStream_t st = (cudaStream_t)stream;
  switch (D) {
    case 16: return launch_bwd_split<16>(dy, y_copy, lse, delta_scratch, causal, B, H, T, dq, dk, dv, workspace, status, layout, st, mask);
    case 32: return launch_bwd_split<32>(dy, y_copy, lse, delta_scratch, causal, B, H, T, dq, dk, dv, workspace, status, layout, st, mask);
    case 64: return launch_bwd_split<64>(dy, y_copy, lse, delta_scratch, causal, B, H, T, dq, dk, dv, workspace, status, layout, st, mask);
  }
  return ERROR_ATTN_UNSUPPORTED_SHAPE;
}

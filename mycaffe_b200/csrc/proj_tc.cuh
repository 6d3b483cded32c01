// Decode projections for more than eight sequences: one pass over the weights, on the tensor cores.
//
// The streaming kernel of gemv.cu shares a pass over the weights between at most eight sequences; sixteen to
// sixty-four sequences (the batched decode configurations) would take two to eight passes.  Here the product
// Y[b, r] = sum_k W[r, k] X[b, k] is a tcgen05 contraction with the weights as the M = 128 operand and the sequences
// as N, so every weight byte leaves HBM once whatever the batch, and the kernel is bound by that stream.
// Replaces the per-sequence cublasSgemv calls of the reference's decode step (CudaExtension.llm32.llama2/Files/
// primitives.cu:322-340) with the arithmetic of its CPU twin (llama2_cpu.cpp:189-202,224-237) kept to fp32 accuracy:
//   * fp32 weights: a tile of 128 rows x 64 k arrives by TMA as fp32; eight warps rewrite it in place as two fp16
//     tiles hi = 16 w cut to fp16's mantissa, lo = fp16(16 w - hi) in the 128-byte-swizzled K-major layout the MMA reads
//     (in place: a tile costs 32 KB of shared memory, not 64, and what a tile costs in shared-memory traffic -- the TMA
//     write, the converters' read and write, the MMAs' operand reads -- is what bounds the kernel); the activations are
//     split the same way by a small pre-pass (after RMSNorm and a per-sequence power-of-two scale), and the product is
//     the three MMAs hi.hi + hi.lo + lo.hi into one fp32 accumulator in TMEM (the dropped lo.lo term is 2^-22);
//   * bf16 weights: the TMA tile is the MMA operand itself, the activations are two bf16 pieces (16 mantissa bits; the
//     weights themselves carry 8), two MMAs per k16.
// Work items are (tile of 128 rows, slice of K): matrices with few rows (Wo, W2) are cut along K so that every SM
// streams; a slice leaves its fp32 partial sums in a scratch array and the slice that arrives last (a ticket per
// tile and quarter of its rows) adds all of them in slice order, so the result does not depend on timing.  The gated
// pair W1/W3 of the feed-forward block is one item with two accumulators and silu(a) * b in the epilogue.
// Roles of a CTA (480 threads, one CTA per SM, persistent over items): warps 0-7 convert, 8-11 epilogue (TMEM lanes
// 32 (w - 8) ..), warp 12 TMA producer of the weights, warp 13 MMA issuer and TMEM owner, warp 14 TMA producer of the
// activation pieces.  The weight ring (five 32 KB slots for fp32, eight 16 KB slots for bf16) and the activation ring
// have their own barriers.  Every wait is bounded.
// The activation pieces, per-sequence scales, partial sums and tickets live in arrays that are part of the library
// image (about 24 MB per device): nothing is allocated, but two of these products must not overlap on one device.
#pragma once
#include "tc_common.cuh"

namespace proj {
using namespace tc;

constexpr int ROWS = 128;          // weight rows per tile (MMA M)
constexpr int KC = 64;             // k per stage: one 128-byte row of 16-bit operands
constexpr int MAX_B = 64;          // sequences (MMA N, rounded up to 16)
constexpr int MAX_N = 16384;       // longest contraction
constexpr int MAX_ITEMS = 296;     // (tile, slice) items when K is cut
constexpr int MAX_TILES = 2048;
constexpr int CONV_WARPS = 8, EPI_WARPS = 4;
constexpr int WARP_EPI0 = CONV_WARPS, WARP_TMA = CONV_WARPS + EPI_WARPS, WARP_MMA = WARP_TMA + 1, WARP_TMA_X = WARP_MMA + 1;
constexpr int THREADS = (WARP_TMA_X + 1) * 32;
constexpr float W_SCALE = 16.f;    // fp32 weights are split after this exact scaling (keeps the low halves normal)
constexpr uint32_t TMEM_ALLOC = 256, ACC_COLS = 128;

__device__ __align__(1024) uint16_t g_x_pieces[2 * MAX_B * MAX_N];
__device__ float g_x_scale[MAX_B];
__device__ float g_partials[(size_t)MAX_ITEMS * ROWS * 2 * MAX_B];
__device__ unsigned int g_tickets[MAX_TILES * EPI_WARPS];
__device__ int g_status[4];

template <typename WT> struct Plan;
template <> struct Plan<float> {
  static constexpr bool CONVERT = true;
#ifndef MCA_PROJ_SW
#define MCA_PROJ_SW 5
#endif
#ifndef MCA_PROJ_SX
#define MCA_PROJ_SX 3
#endif
  static constexpr int SW = MCA_PROJ_SW, SX = MCA_PROJ_SX, PIECES = 2, FMT = 0;   // weight / activation ring depths; fp16 operands
  static constexpr uint32_t W_BYTES = ROWS * KC * 4;                    // a slot: the fp32 tile, then hi | lo in its place
  static constexpr uint32_t X_BYTES = PIECES * MAX_B * 128;
  static constexpr uint32_t OP_BYTES = ROWS * KC * 2;                   // one fp16 operand tile (half a slot)
  static constexpr uint32_t OFF_W = 0, OFF_X = OFF_W + SW * W_BYTES, OFF_OP = OFF_X + SX * X_BYTES;
  static constexpr uint32_t OFF_BAR = OFF_OP;
};
template <> struct Plan<__nv_bfloat16> {
  static constexpr bool CONVERT = false;
  static constexpr int SW = 8, SX = 3, PIECES = 2, FMT = 1;            // bf16 operands
  static constexpr uint32_t W_BYTES = ROWS * KC * 2;
  static constexpr uint32_t X_BYTES = PIECES * MAX_B * 128;
  static constexpr uint32_t OP_BYTES = 0;
  static constexpr uint32_t OFF_W = 0, OFF_X = OFF_W + SW * W_BYTES, OFF_OP = OFF_X + SX * X_BYTES;
  static constexpr uint32_t OFF_BAR = OFF_OP;
};
// barriers: wfull[SW] wempty[SW] xfull[SX] xempty[SX] convdone[SW] accfull[2] accfree[2], then the TMEM address
constexpr uint32_t BAR_BYTES = 512;
template <typename WT> constexpr size_t smem_bytes() { return Plan<WT>::OFF_BAR + BAR_BYTES + EPI_WARPS * MAX_B * 4 + 1024; }

struct Params {
  float* out[3];
  int rows[3];
  int tile0[4];        // first tile of each matrix (not gated); tile0[n_mats] = tiles
  int n_mats, B, Bp, n, accumulate, swiglu, slices, tiles, kchunks;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Barrier 1 over the converter warps, returning the AND of their predicates.
__device__ __forceinline__ bool conv_bar_and(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\t"
      "barrier.cta.red.and.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "n"(CONV_WARPS * 32)
      : "memory");
  return r != 0;
}

__device__ __forceinline__ float block_sum(float v, float* red) {   // 256 threads
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) t += red[w];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) t = fmaxf(t, red[w]);
  return t;
}

// Activations of sequence b -> 16-bit pieces (row p * Bp + b of a (pieces * Bp, n) array): RMSNorm as the CPU twin
// orders it, o[j] = w[j] * (s * x[j]) with s = 1 / sqrt(sum(x^2) / n + eps) (llama2_cpu.cpp:189-202), then
//   BF16 = false: v / 2^e with 2^e chosen so that the row's largest magnitude lands in [2^13, 2^14), as fp16 hi + lo;
//   BF16 = true:  v as two bf16 pieces, hi = bf16(v), lo = bf16(v - hi): 16 mantissa bits, two hundred times finer than
//                 the bf16 weights they multiply.
// Rows from B up to Bp are written as zeros.  One CTA of 256 threads per row.
template <bool BF16>
__global__ void __launch_bounds__(256) x_pieces_kernel(const float* __restrict__ x, const float* __restrict__ norm_w, float eps,
                                                       int n, int B, int Bp, uint16_t* __restrict__ pieces,
                                                       float* __restrict__ xscale) {
  __shared__ float red[8];
  extern __shared__ float xrow[];                       // the row, read from global memory once
  const int b = blockIdx.x, tid = threadIdx.x;
  mca_pdl_launch_dependents();                          // the contraction kernel may start fetching weights
  mca_pdl_wait();                                       // launched ahead of the kernels before it: their results (x, and the
                                                        // previous contraction's last reads of the pieces) come first
  const size_t piece_stride = (size_t)Bp * n;
  uint16_t* dst = pieces + (size_t)b * n;
  if (b >= B) {
    for (int k = tid; k < n; k += 256) {
      dst[k] = 0; dst[piece_stride + k] = 0;
    }
    return;
  }
  const float* xr = x + (size_t)b * n;
  float ss = 0.f;
  for (int k = tid; k < n; k += 256) { const float v = xr[k]; xrow[k] = v; ss = fmaf(v, v, ss); }
  float s = 1.f;
  if (norm_w != nullptr) {
    ss = block_sum(ss, red);
    s = 1.0f / sqrtf(ss / (float)n + eps);
  }
  float amax = 0.f;
  for (int k = tid; k < n; k += 256) {                  // a thread revisits only the elements it wrote itself
    const float v = norm_w != nullptr ? __ldg(norm_w + k) * (s * xrow[k]) : xrow[k];
    xrow[k] = v;
    amax = fmaxf(amax, fabsf(v));
  }
  if (BF16) {
    for (int k = tid; k < n; k += 256) {
      const float v = xrow[k];
      const __nv_bfloat16 h = __float2bfloat16_rn(v);
      const __nv_bfloat16 l = __float2bfloat16_rn(v - __bfloat162float(h));
      dst[k] = __bfloat16_as_ushort(h);
      dst[piece_stride + k] = __bfloat16_as_ushort(l);
    }
    if (tid == 0) xscale[b] = 1.f;
    return;
  }
  amax = block_max(amax, red);
  int e = 0;
  if (amax > 0.f && amax < INFINITY) { frexpf(amax, &e); e -= 14; }
  const float down = ldexpf(1.f, -e);
  for (int k = tid; k < n; k += 256) {
    const float v = xrow[k] * down;
    const __half h = __float2half_rn(v);
    const __half l = __float2half_rn(v - __half2float(h));
    dst[k] = __half_as_ushort(h);
    dst[piece_stride + k] = __half_as_ushort(l);
  }
  if (tid == 0) xscale[b] = ldexpf(1.f, e) / W_SCALE;
}

template <typename WT>
__global__ void __launch_bounds__(THREADS, 1) proj_tc_kernel(const __grid_constant__ CUtensorMap mw0,
                                                             const __grid_constant__ CUtensorMap mw1,
                                                             const __grid_constant__ CUtensorMap mw2,
                                                             const __grid_constant__ CUtensorMap mx, const Params p) {
  using PL = Plan<WT>;
  constexpr int SW = PL::SW, SX = PL::SX;
  extern __shared__ unsigned char pj_smem_raw[];
  const uint32_t raw = smem_u32(pj_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gen = pj_smem_raw + (base - raw);
  const uint32_t bar0 = base + PL::OFF_BAR;
  auto wfull = [&](int s) { return bar0 + 8u * s; };
  auto wempty = [&](int s) { return bar0 + 8u * (SW + s); };
  auto xfull = [&](int s) { return bar0 + 8u * (2 * SW + s); };
  auto xempty = [&](int s) { return bar0 + 8u * (2 * SW + SX + s); };
  constexpr int NB0 = 2 * SW + 2 * SX;
  auto convdone = [&](int c) { return bar0 + 8u * (NB0 + c); };        // [SW]: slot c holds the converted tiles
  auto accfull = [&](int a) { return bar0 + 8u * (NB0 + SW + a); };
  auto accfree = [&](int a) { return bar0 + 8u * (NB0 + SW + 2 + a); };
  static_assert(8 * (NB0 + SW + 4) + 8 <= BAR_BYTES, "barriers fit their block");
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + PL::OFF_BAR + 8 * (NB0 + SW + 4));
  float* cs = reinterpret_cast<float*>(gen + PL::OFF_BAR + BAR_BYTES);   // per-sequence output scales, one copy per epilogue warp
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int* status = g_status;

  if (tid == 0) {
    for (int s = 0; s < SW; ++s) {
      mbar_init(wfull(s), 1);
      mbar_init(wempty(s), 1);                              // the MMA has read the slot
      mbar_init(convdone(s), CONV_WARPS);
    }
    for (int s = 0; s < SX; ++s) {
      mbar_init(xfull(s), 1);
      mbar_init(xempty(s), 1);
    }
    for (int c = 0; c < 2; ++c) {
      mbar_init(accfull(c), 1);
      mbar_init(accfree(c), EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == WARP_MMA) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_ALLOC);
    tmem_relinquish();
  }
  if (warp == WARP_TMA && lane == 0) {
    prefetch_tensormap(&mw0);
    if (p.n_mats > 1) prefetch_tensormap(&mw1);
    if (p.n_mats > 2) prefetch_tensormap(&mw2);
    prefetch_tensormap(&mx);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  mca_pdl_launch_dependents();   // a dependent launch may take the SMs as this kernel's CTAs leave them
  const int items = p.tiles * p.slices;
  const int nacc = p.swiglu ? 2 : 1;
  // k chunks of slice j: [j * kchunks / slices, (j + 1) * kchunks / slices)
  auto slice_lo = [&](int j) { return (int)(((int64_t)j * p.kchunks) / p.slices); };
  const uint32_t x_piece_bytes = (uint32_t)p.Bp * 128u;
  bool ok = true;

  if (warp == WARP_TMA) {
    // ------------------------------------------------------------------ weight producer
    // The weights depend on nothing this stream computes: their tiles are requested from the first instruction on, also
    // while the pre-pass that this launch may have overtaken is still running.  A slot is free again as soon as the
    // converters have read it (fp32) or the MMA has (bf16).
    if (lane == 0) {
      int g = 0;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int u = item / p.slices, j = item - u * p.slices;
        const int k0 = slice_lo(j), k1 = slice_lo(j + 1);
        for (int mi = 0; mi < nacc && ok; ++mi) {
          int m = mi, row0 = u * ROWS;
          if (!p.swiglu) {
            m = 0;
            if (p.n_mats > 1 && u >= p.tile0[1]) m = 1;
            if (p.n_mats > 2 && u >= p.tile0[2]) m = 2;
            row0 = (u - p.tile0[m]) * ROWS;
          }
          const CUtensorMap* mw = m == 0 ? &mw0 : (m == 1 ? &mw1 : &mw2);
          for (int kc = k0; kc < k1; ++kc, ++g) {
            const int s = g % SW;
            ok = mbar_wait(wempty(s), (uint32_t)(((g / SW) & 1) ^ 1), status, 1, g);
            if (!ok) break;
            mbar_expect_tx(wfull(s), PL::W_BYTES);
            tma_load_2d(base + PL::OFF_W + s * PL::W_BYTES, mw, wfull(s), kc * KC, row0);
          }
        }
      }
    }
  } else if (warp == WARP_TMA_X) {
    // ------------------------------------------------------------------ activation producer
    if (lane == 0) {
      mca_pdl_wait();                                     // the pieces are the pre-pass's output
      int g = 0;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int u = item / p.slices, j = item - u * p.slices;
        const int k0 = slice_lo(j), k1 = slice_lo(j + 1);
        for (int mi = 0; mi < nacc && ok; ++mi) {
          for (int kc = k0; kc < k1; ++kc, ++g) {
            const int s = g % SX;
            ok = mbar_wait(xempty(s), (uint32_t)(((g / SX) & 1) ^ 1), status, 8, g);
            if (!ok) break;
            mbar_expect_tx(xfull(s), PL::PIECES * x_piece_bytes);
#pragma unroll
            for (int pc = 0; pc < PL::PIECES; ++pc)
              tma_load_2d(base + PL::OFF_X + s * PL::X_BYTES + pc * x_piece_bytes, &mx, xfull(s), kc * KC, pc * p.Bp);
          }
        }
      }
    }
  } else if (warp == WARP_MMA) {
    // ------------------------------------------------------------------ MMA issuer (one lane)
    if (lane == 0) {
      const uint32_t idesc = make_idesc_fmt(ROWS, p.Bp, 0, 0, PL::FMT);
      int g = 0, it = 0;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++it) {
        const int u = item / p.slices, j = item - u * p.slices;
        const int k0 = slice_lo(j), k1 = slice_lo(j + 1);
        const int a = it & 1;
        ok = mbar_wait(accfree(a), (uint32_t)(((it >> 1) & 1) ^ 1), status, 2, it);
        if (!ok) break;
        tc_fence_after();
        for (int mi = 0; mi < nacc && ok; ++mi) {
          const uint32_t d_tmem = tmem_base + (uint32_t)a * ACC_COLS + (uint32_t)(mi * p.Bp);
          for (int kc = k0; kc < k1; ++kc, ++g) {
            const int sw = g % SW, sx = g % SX;
            // fp32 weights: the slot holds the converted hi | lo tiles once all converter warps have arrived
            ok = mbar_wait(PL::CONVERT ? convdone(sw) : wfull(sw), (uint32_t)((g / SW) & 1), status, 3, g);
            if (!ok) break;
            const uint32_t a_hi = base + PL::OFF_W + sw * PL::W_BYTES, a_lo = a_hi + PL::OP_BYTES;
            ok = mbar_wait(xfull(sx), (uint32_t)((g / SX) & 1), status, 9, g);
            if (!ok) break;
            tc_fence_after();
            const uint32_t xs = base + PL::OFF_X + sx * PL::X_BYTES;
#pragma unroll
            for (int kk = 0; kk < KC / 16; ++kk) {
              const uint32_t first = (kc == k0 && kk == 0) ? 0u : 1u;
              const uint64_t dx0 = make_desc(xs + kk * 32, 16, 1024);
              const uint64_t dx1 = make_desc(xs + x_piece_bytes + kk * 32, 16, 1024);
              const uint64_t da = make_desc(a_hi + kk * 32, 16, 1024);
              if constexpr (PL::CONVERT) {
                const uint64_t dl = make_desc(a_lo + kk * 32, 16, 1024);
                umma_ss(d_tmem, da, dx0, idesc, first);     // hi . hi
                umma_ss(d_tmem, da, dx1, idesc, 1u);        // hi . lo
                umma_ss(d_tmem, dl, dx0, idesc, 1u);        // lo . hi
              } else {
                umma_ss(d_tmem, da, dx0, idesc, first);     // W . x_hi
                umma_ss(d_tmem, da, dx1, idesc, 1u);        // W . x_lo
              }
            }
            umma_commit(wempty(sw));
            umma_commit(xempty(sx));
          }
        }
        if (ok) umma_commit(accfull(a));
      }
    }
  } else if (warp < CONV_WARPS) {
    // ------------------------------------------------------------------ converters (fp32 weights)
    if constexpr (PL::CONVERT) {
      int g = 0;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int u = item / p.slices, j = item - u * p.slices;
        const int steps = nacc * (slice_lo(j + 1) - slice_lo(j));
        for (int t = 0; t < steps; ++t, ++g) {
          const int s = g % SW;
          const bool mine = __all_sync(0xffffffffu, mbar_wait(wfull(s), (uint32_t)((g / SW) & 1), status, 5, g));
          // The tile is rewritten in place: hi over the first half of the slot, lo over the second.  A lane takes the
          // sixteen rows of its warp into registers (k = 2 lane, 2 lane + 1: 8-byte reads, no bank conflicts); nobody
          // writes before all eight warps have read.  The barrier also carries the vote on the wait's outcome, so that
          // either every converter warp goes on or none does.
          float2 v[ROWS / CONV_WARPS];
          const float* wst = reinterpret_cast<const float*>(gen + PL::OFF_W + s * PL::W_BYTES);
          if (mine) {
#pragma unroll
            for (int rr = 0; rr < ROWS / CONV_WARPS; ++rr)
              v[rr] = *reinterpret_cast<const float2*>(wst + (warp * (ROWS / CONV_WARPS) + rr) * KC + 2 * lane);
          }
          ok = conv_bar_and(mine);
          if (!ok) break;
          unsigned char* ohi = gen + PL::OFF_W + s * PL::W_BYTES;
          unsigned char* olo = ohi + PL::OP_BYTES;
#pragma unroll
          for (int rr = 0; rr < ROWS / CONV_WARPS; ++rr) {
            const int r = warp * (ROWS / CONV_WARPS) + rr;
            // hi = the scaled weight cut to fp16's mantissa (exact in fp16), lo = the rest (exact in fp32, rounded once)
            const float a0 = v[rr].x * W_SCALE, a1 = v[rr].y * W_SCALE;
            const float h0 = __uint_as_float(__float_as_uint(a0) & 0xffffe000u), h1 = __uint_as_float(__float_as_uint(a1) & 0xffffe000u);
            uint32_t h, l;
            asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(h) : "f"(h1), "f"(h0));
            asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(l) : "f"(a1 - h1), "f"(a0 - h0));
            const uint32_t off = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u + (uint32_t)(((lane >> 2) ^ (r & 7)) << 4) +
                                 (uint32_t)(lane & 3) * 4u;
            *reinterpret_cast<uint32_t*>(ohi + off) = h;
            *reinterpret_cast<uint32_t*>(olo + off) = l;
          }
          fence_proxy_async();          // the MMA reads these tiles through the asynchronous proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(convdone(s));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int e = warp - WARP_EPI0;                       // TMEM lanes 32 e .. 32 e + 31
    const int r = e * 32 + lane;                          // row of the tile
    // per-sequence output scales, written by the pre-pass this launch may have overtaken: every warp keeps a copy
    mca_pdl_wait();
    cs += e * MAX_B;
    cs[lane] = lane < p.B ? __ldcg(g_x_scale + lane) : 0.f;
    cs[lane + 32] = lane + 32 < p.B ? __ldcg(g_x_scale + lane + 32) : 0.f;
    __syncwarp();
    const int ncols = nacc * p.Bp;
    int it = 0;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++it) {
      const int u = item / p.slices, j = item - u * p.slices;
      const int a = it & 1;
      int m = 0, row0 = u * ROWS;
      if (!p.swiglu) {
        if (p.n_mats > 1 && u >= p.tile0[1]) m = 1;
        if (p.n_mats > 2 && u >= p.tile0[2]) m = 2;
        row0 = (u - p.tile0[m]) * ROWS;
      }
      float* outm = m == 0 ? p.out[0] : (m == 1 ? p.out[1] : p.out[2]);
      const int rows_m = m == 0 ? p.rows[0] : (m == 1 ? p.rows[1] : p.rows[2]);
      const int row = row0 + r;
      ok = __all_sync(0xffffffffu, mbar_wait(accfull(a), (uint32_t)((it >> 1) & 1), status, 7, it));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + ((uint32_t)(e * 32) << 16) + (uint32_t)a * ACC_COLS;
      // sixteen output elements of this thread's row: the products scaled back, gated if asked, added to the residual
      // if asked (all sixteen residuals are requested before any is used)
      auto finish16 = [&](int c0, const float (&va)[16], const float (&vb)[16]) {
        if (row >= rows_m) return;
        float res[16];
        float* dst = outm + (size_t)c0 * rows_m + row;
#pragma unroll
        for (int i = 0; i < 16; ++i) res[i] = (p.accumulate && c0 + i < p.B) ? __ldcg(dst + (size_t)i * rows_m) : 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (c0 + i < p.B) {
            const float sc = cs[c0 + i];
            float y = va[i] * sc;
            if (p.swiglu) {
              y *= (1.0f / (1.0f + expf(-y)));          // silu, llama2_cpu.cpp:360-365
              y *= vb[i] * sc;
            }
            dst[(size_t)i * rows_m] = y + res[i];
          }
        }
      };
      if (p.slices == 1) {
        for (int c0 = 0; c0 < p.Bp; c0 += 16) {
          uint32_t va[16], vb[16];
          float fa[16], fb[16];
          tmem_ld16(t_acc + c0, va);
          if (p.swiglu) tmem_ld16(t_acc + p.Bp + c0, vb);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) { fa[i] = __uint_as_float(va[i]); fb[i] = p.swiglu ? __uint_as_float(vb[i]) : 0.f; }
          finish16(c0, fa, fb);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(accfree(a));
      } else {
        float* part = g_partials + ((size_t)(u * p.slices + j) * ncols) * ROWS + r;
        for (int c0 = 0; c0 < ncols; c0 += 16) {
          uint32_t v[16];
          tmem_ld16(t_acc + c0, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) __stcg(part + (size_t)(c0 + i) * ROWS, __uint_as_float(v[i]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(accfree(a));
        // a ticket per (tile, quarter of its rows): the warp that arrives last for its quarter adds up all slices
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          const unsigned int old = atomicAdd(&g_tickets[u * EPI_WARPS + e], 1u);
          last = old == (unsigned int)(p.slices - 1);
          if (last) g_tickets[u * EPI_WARPS + e] = 0;    // ready for the next launch
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          const float* p0 = g_partials + ((size_t)(u * p.slices) * ncols) * ROWS + r;
          // Sixteen columns at a time, two slices per round: 32 loads are in flight together, and the sums are taken in
          // slice order whoever arrived last.
          auto gather = [&](int col0, float (&acc)[16]) {
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = 0.f;
            for (int s0 = 0; s0 < p.slices; s0 += 2) {
              float t[2][16];
#pragma unroll
              for (int q = 0; q < 2; ++q)
#pragma unroll
                for (int i = 0; i < 16; ++i)
                  t[q][i] = s0 + q < p.slices ? __ldcg(p0 + ((size_t)(s0 + q) * ncols + col0 + i) * ROWS) : 0.f;
#pragma unroll
              for (int q = 0; q < 2; ++q)
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] += t[q][i];
            }
          };
          for (int c0 = 0; c0 < p.Bp; c0 += 16) {
            float va[16], vb[16];
            gather(c0, va);
            if (p.swiglu) gather(p.Bp + c0, vb);
            if (!p.swiglu) {
#pragma unroll
              for (int i = 0; i < 16; ++i) vb[i] = 0.f;
            }
            finish16(c0, va, vb);
          }
        }
      }
    }
  }
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_ALLOC);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
inline int make_map_2d(CUtensorMap* map, const void* basep, CUtensorMapDataType type, int elt, int64_t rows, int64_t cols,
                       int box_cols, int box_rows, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * elt};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, type, 2, const_cast<void*>(basep), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : ERROR_ATTN_UNSUPPORTED_SHAPE;
}

inline bool& enabled() { static bool on = true; return on; }

// K slices for `tiles` row tiles of `kchunks` stages each on `sms` SMs: the count that fills whole waves best, with at
// least four stages per slice and at most MAX_ITEMS items.
inline int pick_slices(int tiles, int kchunks, int sms) {
  int best = 1;
  double best_eff = (double)tiles / ((double)((tiles + sms - 1) / sms) * sms);
  for (int s = 2; s <= 8; ++s) {
    if (kchunks / s < 4 || tiles * s > MAX_ITEMS) break;
    const int items = tiles * s;
    const double eff = (double)items / ((double)((items + sms - 1) / sms) * sms);
    if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
  }
  return best;
}

}  // namespace proj

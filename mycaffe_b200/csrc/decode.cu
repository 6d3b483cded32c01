// Split-KV flash decoding for the llama2 KV-cache path.
//
// Replaces the reference's decode attention for one new token
// (Primitives::attention / multi_head_attention_kernel, CudaExtension.llm32.llama2/Files/
// primitives.cu:158-202,391-403, CPU twin llama2_cpu.cpp:304-342) together with the steps
// the reference runs as separate launches before it: RoPE on the new q/k (rope_kernel,
// primitives.cu:99-116) and the append of k,v to the cache (llama2_gpu.cpp:67-72).
//
// The reference launches one CTA per head and lets each thread walk a whole K row, so its
// cache reads are uncoalesced and 32 CTAs cannot fill the machine.  Here the keys of every
// (sequence, kv-head) are cut into splits; a CTA streams its split once with 128-bit loads
// in which the lanes of a group cover one contiguous cache row, reduces dot products with
// warp shuffles, keeps an online-softmax state per lane group, and writes one partial
// (max, sum, weighted V) per head.  A second small kernel combines the partials.  The work
// is bound by HBM traffic: every cache byte is read exactly once.
#include <algorithm>
#include <mutex>

#include <cstdint>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

// Scratch of the no-allocation entry point (mca_decode_attention_static): the split partials
// live in this fixed array instead of caller-provided memory.  Every GPU that loads the library
// holds these 8 MiB until the process exits.  In host code the symbol is only a stand-in; the
// device address is obtained once per device with cudaGetSymbolAddress.
constexpr int64_t MCA_STATIC_SCRATCH_FLOATS = 2 * 1024 * 1024;
static __device__ __align__(256) float g_static_decode_scratch[MCA_STATIC_SCRATCH_FLOATS];

namespace {

constexpr int DEC_THREADS = 256;
constexpr int DEC_WARPS = DEC_THREADS / 32;

// Cache elements one lane holds of a row.  A group of G = HS / EPL lanes (a power of two) covers one contiguous
// cache row with 128-bit loads, so EPL is a multiple of 4 (fp32) or 8 (bf16) elements: 16 for head sizes that are
// 16 x a power of two, 12 (fp32) or 24 (bf16) for 48 and 96.
template <typename CT, int HS> struct Epl {
  static constexpr int VEC = 16 / (int)sizeof(CT);
  static constexpr int value = (HS % 48 == 0) ? (VEC == 4 ? 12 : 24) : 16;
};

// Status words of the decode kernels: [0] number of sequences whose position was outside [0, max_len) since the
// last read, [1] the first such sequence, [2] its position.  Such a sequence is not attended and its output is zero.
__device__ int g_decode_status[4];

struct DecodeParams {
  const float* q;        // (B, n_heads*HS): projection of the new token (before RoPE when fr != null)
  const float* k_new;    // (B, kv_dim) or null: new key (before RoPE); appended to the cache at pos[b]
  const float* v_new;    // (B, kv_dim) or null
  void* k_cache;         // (B, seq_len, kv_dim) cache element type
  void* v_cache;
  const int* pos;        // (B): index of the new token; keys 0..pos[b] are attended
  const float* fr;       // (seq_len, HS/2) cos table or null (no RoPE)
  const float* fi;       // (seq_len, HS/2) sin table
  float* part_acc;       // (B, n_heads, nsplit, HS)
  float* part_ml;        // (B, n_heads, nsplit, 2)
  float* out;            // (B, n_heads*HS)
  int64_t cache_batch_stride;  // elements between sequences in the caches
  int n_heads, n_kv_heads, kv_mul, seq_len, split_len, nsplit;
  int pos_limit;         // positions must lie in [0, pos_limit): the planned splits and the cache cover no more
};

template <typename CT, int EPL> struct RowSlice;
template <int EPL> struct RowSlice<float, EPL> {
  static constexpr int NV = EPL / 4;
  // chunk c of lane gl covers elements (c*G + gl)*4 .. +3
  template <int G> static __device__ __forceinline__ void load(const float* row, int gl, float (&x)[EPL]) {
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const float4 t = __ldcs(reinterpret_cast<const float4*>(row) + c * G + gl);
      x[c * 4 + 0] = t.x; x[c * 4 + 1] = t.y; x[c * 4 + 2] = t.z; x[c * 4 + 3] = t.w;
    }
  }
  template <int G> static __device__ __forceinline__ void store(float* row, int gl, const float (&x)[EPL]) {
#pragma unroll
    for (int c = 0; c < NV; ++c)
      reinterpret_cast<float4*>(row)[c * G + gl] = make_float4(x[c * 4], x[c * 4 + 1], x[c * 4 + 2], x[c * 4 + 3]);
  }
  template <int G> static __device__ __forceinline__ int elem(int gl, int i) { return ((i >> 2) * G + gl) * 4 + (i & 3); }
};
template <int EPL> struct RowSlice<__nv_bfloat16, EPL> {
  static constexpr int NV = EPL / 8;
  // chunk c of lane gl covers elements (c*G + gl)*8 .. +7
  template <int G> static __device__ __forceinline__ void load(const __nv_bfloat16* row, int gl, float (&x)[EPL]) {
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const uint4 t = __ldcs(reinterpret_cast<const uint4*>(row) + c * G + gl);
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[c * 8 + 2 * i] = __uint_as_float(w[i] << 16);
        x[c * 8 + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    }
  }
  template <int G> static __device__ __forceinline__ void store(__nv_bfloat16* row, int gl, const float (&x)[EPL]) {
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(x[c * 8 + 2 * i], x[c * 8 + 2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
      reinterpret_cast<uint4*>(row)[c * G + gl] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  template <int G> static __device__ __forceinline__ int elem(int gl, int i) { return ((i >> 3) * G + gl) * 8 + (i & 7); }
};

// bf16 caches stream through a per-warp ring in shared memory filled by cp.async: a bf16 row is half the bytes of
// an fp32 one, so twice the rows have to be outstanding to cover the HBM latency, and asynchronous copies keep them
// in flight without holding them in registers.  Every lane copies exactly the 4 x 16 bytes it consumes itself
// (NV vectors of the K row, NV of the V row; NV = 2, or 3 for head sizes 48 and 96), so no synchronisation other than
// its own wait_group is needed.  Row steps in flight per warp: six (96 KB per CTA: two CTAs per SM overlap their
// ramps), four with three vectors per row.
template <int NV> struct DecRing {
  static constexpr int STAGES = NV <= 2 ? 6 : 4;
  static constexpr size_t BYTES = (size_t)DEC_WARPS * STAGES * 2 * NV * 32 * sizeof(uint4);   // per CTA
};
__device__ __forceinline__ void unpack_bf16x8(const uint4& t, float* x) {
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// Load 16 elements of a float vector in the lane's element order, optionally rotating
// adjacent pairs by the RoPE angle of this position (rope, llama2_cpu.cpp:239-262).
template <typename CT, int G, int EPL>
__device__ __forceinline__ void load_vec_rope(const float* __restrict__ src, int gl, const float* __restrict__ cr,
                                              const float* __restrict__ ci, float (&x)[EPL]) {
#pragma unroll
  for (int i = 0; i < EPL; i += 2) {
    const int e = RowSlice<CT, EPL>::template elem<G>(gl, i);  // even
    const float x0 = src[e], x1 = src[e + 1];
    if (cr != nullptr) {
      const float c = cr[e >> 1], s = ci[e >> 1];
      x[i] = x0 * c - x1 * s;
      x[i + 1] = x0 * s + x1 * c;
    } else {
      x[i] = x0; x[i + 1] = x1;
    }
  }
}

template <typename CT, int HS, int KVM>
__global__ void __launch_bounds__(DEC_THREADS, KVM == 1 ? 2 : 1) decode_split_kernel(const DecodeParams p) {   // one query head per kv head: two CTAs per SM (at most 128 registers)
  constexpr int EPL = Epl<CT, HS>::value;
  using Row = RowSlice<CT, EPL>;
  constexpr int G = HS / EPL;     // lanes per cache row
  constexpr int RPW = 32 / G;     // rows per warp per step
  constexpr int U = 2;            // steps in flight
  __shared__ float s_acc[DEC_WARPS][KVM][HS];
  __shared__ float s_ml[DEC_WARPS][KVM][2];

  mca_pdl_launch_dependents();   // a projection kernel that follows may start fetching its weights
  mca_pdl_wait();                // launched ahead of the kernels before it: q is their output, and the scratch theirs to read
  const int b = blockIdx.z;
  const int h0 = blockIdx.y * KVM;          // first query head of this CTA
  const int kvh = h0 / p.kv_mul;
  const int split = blockIdx.x;
  const int pos = p.pos[b];
  if (pos < 0 || pos >= p.pos_limit) {
    // A position outside the cache (or beyond the planned splits) is not followed: nothing of this sequence is
    // read or appended, its output is zero, and the status words say which sequence it was.
    if (split == 0) {
      if (blockIdx.y == 0 && threadIdx.x == 0 && atomicAdd(&g_decode_status[0], 1) == 0) {
        g_decode_status[1] = b;
        g_decode_status[2] = pos;
      }
      if (p.nsplit == 1)
        for (int i = threadIdx.x; i < KVM * HS; i += DEC_THREADS) p.out[(int64_t)b * p.n_heads * HS + (int64_t)h0 * HS + i] = 0.f;
    }
    return;
  }
  const int L = pos + 1;
  const int r_begin = split * p.split_len;
  if (r_begin >= L) return;
  const int r_end = min(L, r_begin + p.split_len);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gl = lane % G, g = lane / G;
  const int kv_dim = p.n_kv_heads * HS;
  const int dim = p.n_heads * HS;
  CT* kc = reinterpret_cast<CT*>(p.k_cache) + (int64_t)b * p.cache_batch_stride + (int64_t)kvh * HS;
  CT* vc = reinterpret_cast<CT*>(p.v_cache) + (int64_t)b * p.cache_batch_stride + (int64_t)kvh * HS;
  const float* cr = p.fr ? p.fr + (int64_t)pos * (HS / 2) : nullptr;
  const float* ci = p.fi ? p.fi + (int64_t)pos * (HS / 2) : nullptr;
  const float inv_div = sqrtf((float)HS);

  float q[KVM][EPL];
#pragma unroll
  for (int x = 0; x < KVM; ++x) load_vec_rope<CT, G, EPL>(p.q + (int64_t)b * dim + (int64_t)(h0 + x) * HS, gl, cr, ci, q[x]);

  float m[KVM], l[KVM], acc[KVM][EPL];
#pragma unroll
  for (int x = 0; x < KVM; ++x) {
    m[x] = -INFINITY; l[x] = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) acc[x][i] = 0.f;
  }

  const bool has_new = (p.k_new != nullptr);
  if constexpr (sizeof(CT) == 2) {
    // ---- bf16 cache: cp.async ring
    constexpr int NV = Row::NV;                 // 16-byte vectors of a K (or V) row per lane
    constexpr int DEC_RING = DecRing<NV>::STAGES;
    extern __shared__ __align__(16) uint4 dec_ring[];
    uint4* my_ring = dec_ring + (size_t)warp * DEC_RING * 2 * NV * 32;     // [stage][vector][lane]
    const uint32_t my_ring_s = (uint32_t)__cvta_generic_to_shared(my_ring);
    const __nv_bfloat16* kcb = reinterpret_cast<const __nv_bfloat16*>(kc);
    const __nv_bfloat16* vcb = reinterpret_cast<const __nv_bfloat16*>(vc);
    const int first = r_begin + warp * RPW;
    const int stride = DEC_WARPS * RPW;
    const int n_steps = first < r_end ? (r_end - first + stride - 1) / stride : 0;
    auto issue = [&](int t) {
      if (t < n_steps) {
        const int row = first + t * stride + g;
        if (row < r_end && !(has_new && row == pos)) {
          const uint32_t dst = my_ring_s + (uint32_t)(((t % DEC_RING) * 2 * NV * 32 + lane) * sizeof(uint4));
          const uint4* ks = reinterpret_cast<const uint4*>(kcb + (int64_t)row * kv_dim);
          const uint4* vs = reinterpret_cast<const uint4*>(vcb + (int64_t)row * kv_dim);
#pragma unroll
          for (int c = 0; c < NV; ++c) {
            mca_cp_async16(dst + (uint32_t)(c * 32 * sizeof(uint4)), ks + c * G + gl);
            mca_cp_async16(dst + (uint32_t)((NV + c) * 32 * sizeof(uint4)), vs + c * G + gl);
          }
        }
      }
      mca_cp_async_commit();   // one group per step, also when it is empty, so that the group count is the step count
    };
#pragma unroll
    for (int t = 0; t < DEC_RING - 1; ++t) issue(t);
    for (int t = 0; t < n_steps; ++t) {
      issue(t + DEC_RING - 1);     // its slot was read in the previous iteration
      mca_cp_async_wait<DEC_RING - 1>();
      const int row = first + t * stride + g;
      const bool valid = row < r_end;
      float kx[EPL], vx[EPL];
      if (valid && has_new && row == pos) {
        // the new token: take k,v from the projections, rotate k, append both to the cache, and attend to what a
        // later step will read back from the cache
        load_vec_rope<CT, G, EPL>(p.k_new + (int64_t)b * kv_dim + (int64_t)kvh * HS, gl, cr, ci, kx);
        load_vec_rope<CT, G, EPL>(p.v_new + (int64_t)b * kv_dim + (int64_t)kvh * HS, gl, nullptr, nullptr, vx);
        if (h0 % p.kv_mul == 0) {
          Row::template store<G>(kc + (int64_t)row * kv_dim, gl, kx);
          Row::template store<G>(vc + (int64_t)row * kv_dim, gl, vx);
        }
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          kx[i] = __bfloat162float(__float2bfloat16_rn(kx[i]));
          vx[i] = __bfloat162float(__float2bfloat16_rn(vx[i]));
        }
      } else if (valid) {
        const uint4* src = my_ring + (size_t)(t % DEC_RING) * 2 * NV * 32 + lane;
#pragma unroll
        for (int c = 0; c < NV; ++c) {
          unpack_bf16x8(src[c * 32], kx + 8 * c);
          unpack_bf16x8(src[(NV + c) * 32], vx + 8 * c);
        }
      } else {
#pragma unroll
        for (int i = 0; i < EPL; ++i) { kx[i] = 0.f; vx[i] = 0.f; }
      }
#pragma unroll
      for (int x = 0; x < KVM; ++x) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) s = fmaf(q[x][i], kx[i], s);
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (valid) {
          s = s / inv_div;  // score /= sqrtf(head_size), llama2_cpu.cpp:322
          if (s > m[x]) {   // the running maximum moves (rare once it has settled): rescale what was accumulated
            const float corr = __expf(m[x] - s);
            l[x] *= corr;
#pragma unroll
            for (int i = 0; i < EPL; ++i) acc[x][i] *= corr;
            m[x] = s;
          }
          const float pw = __expf(s - m[x]);
          l[x] += pw;
#pragma unroll
          for (int i = 0; i < EPL; ++i) acc[x][i] = fmaf(pw, vx[i], acc[x][i]);
        }
      }
    }
    mca_cp_async_wait<0>();
  } else {
  for (int base = r_begin + warp * RPW; base < r_end; base += DEC_WARPS * RPW * U) {
    float kx[U][EPL], vx[U][EPL];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int row = base + u * DEC_WARPS * RPW + g;
      valid[u] = row < r_end;
      if (valid[u]) {
        if (has_new && row == pos) {
          // the new token: take k,v from the projections, rotate k, and append both to the cache
          load_vec_rope<CT, G, EPL>(p.k_new + (int64_t)b * kv_dim + (int64_t)kvh * HS, gl, cr, ci, kx[u]);
          load_vec_rope<CT, G, EPL>(p.v_new + (int64_t)b * kv_dim + (int64_t)kvh * HS, gl, nullptr, nullptr, vx[u]);
          if (h0 % p.kv_mul == 0) {
            Row::template store<G>(kc + (int64_t)row * kv_dim, gl, kx[u]);
            Row::template store<G>(vc + (int64_t)row * kv_dim, gl, vx[u]);
          }
          if (sizeof(CT) == 2) {  // attend to what a later step will read back from the cache
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
              kx[u][i] = __bfloat162float(__float2bfloat16_rn(kx[u][i]));
              vx[u][i] = __bfloat162float(__float2bfloat16_rn(vx[u][i]));
            }
          }
        } else {
          Row::template load<G>(kc + (int64_t)row * kv_dim, gl, kx[u]);
          Row::template load<G>(vc + (int64_t)row * kv_dim, gl, vx[u]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int x = 0; x < KVM; ++x) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) s = fmaf(q[x][i], kx[u][i], s);
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (valid[u]) {
          s = s / inv_div;  // score /= sqrtf(head_size), llama2_cpu.cpp:322
          if (s > m[x]) {   // the running maximum moves (rare once it has settled): rescale what was accumulated
            const float corr = __expf(m[x] - s);
            l[x] *= corr;
#pragma unroll
            for (int i = 0; i < EPL; ++i) acc[x][i] *= corr;
            m[x] = s;
          }
          const float pw = __expf(s - m[x]);
          l[x] += pw;
#pragma unroll
          for (int i = 0; i < EPL; ++i) acc[x][i] = fmaf(pw, vx[u][i], acc[x][i]);
        }
      }
    }
  }

  }

  // merge the lane groups of a warp, then the warps of the CTA
#pragma unroll
  for (int x = 0; x < KVM; ++x) {
    float m_all = m[x];
#pragma unroll
    for (int o = G; o < 32; o <<= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, o));
    const float f = (m[x] == -INFINITY) ? 0.f : __expf(m[x] - m_all);
    float lsum = l[x] * f;
#pragma unroll
    for (int o = G; o < 32; o <<= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      float a = acc[x][i] * f;
#pragma unroll
      for (int o = G; o < 32; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      if (g == 0) s_acc[warp][x][Row::template elem<G>(gl, i)] = a;
    }
    if (lane == 0) { s_ml[warp][x][0] = m_all; s_ml[warp][x][1] = lsum; }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < KVM * HS; idx += DEC_THREADS) {
    const int x = idx / HS, e = idx % HS;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, s_ml[w][x][0]);
    float lsum = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float mw = s_ml[w][x][0];
      const float f = (mw == -INFINITY) ? 0.f : __expf(mw - M);
      lsum += s_ml[w][x][1] * f;
      a += s_acc[w][x][e] * f;
    }
    const int h = h0 + x;
    if (p.nsplit == 1) {
      p.out[(int64_t)b * dim + (int64_t)h * HS + e] = a / lsum;
    } else {
      const int64_t slot = ((int64_t)b * p.n_heads + h) * p.nsplit + split;
      p.part_acc[slot * HS + e] = a;
      if (e == 0) { p.part_ml[slot * 2] = M; p.part_ml[slot * 2 + 1] = lsum; }
    }
  }
}

// Combine pass: out[b,h,:] = sum_s exp(m_s - M) acc_s / sum_s exp(m_s - M) l_s.
template <int HS>
__global__ void __launch_bounds__(HS) decode_combine_kernel(const float* __restrict__ part_acc,
                                                            const float* __restrict__ part_ml,
                                                            const int* __restrict__ pos, int n_heads, int nsplit,
                                                            int split_len, int pos_limit, float* __restrict__ out) {
  mca_pdl_launch_dependents();
  const int h = blockIdx.x, b = blockIdx.y, e = threadIdx.x;
  const int pb = pos[b];
  mca_pdl_wait();   // the partials are the split kernel's output
  if (pb < 0 || pb >= pos_limit) { out[((int64_t)b * n_heads + h) * HS + e] = 0.f; return; }
  const int n_valid = min(nsplit, (pb + split_len) / split_len);  // ceil((pos+1)/split_len)
  const int64_t slot0 = ((int64_t)b * n_heads + h) * nsplit;
  float M = -INFINITY;
  for (int s = 0; s < n_valid; ++s) M = fmaxf(M, part_ml[(slot0 + s) * 2]);
  float lsum = 0.f, a = 0.f;
  for (int s = 0; s < n_valid; ++s) {
    const float f = __expf(part_ml[(slot0 + s) * 2] - M);
    lsum += part_ml[(slot0 + s) * 2 + 1] * f;
    a += part_acc[(slot0 + s) * HS + e] * f;
  }
  out[((int64_t)b * n_heads + h) * HS + e] = a / lsum;
}

// ---------------------------------------------------------------------------------------------
// Exchange of the head outputs between the GPUs that share the heads (one process per GPU), in place of an all-gather
// per layer-step: every rank stores its (B, dim/N) slice into the (B, dim) buffer of every rank (plain 16-byte stores
// to peer memory mapped into this process; this GPU's own buffer is one of the destinations), then raises its flag
// in every rank's flag array and waits until all ranks' flags in its own array have reached this exchange's
// generation.  When the kernel has finished, this rank's buffer holds every rank's slice.
// The wait is bounded: if a peer never arrives the kernel records it in the status words and returns.
// ---------------------------------------------------------------------------------------------
struct ExchangeParams {
  const float* src;        // (B, dim_local) this rank's head outputs
  float* dst[8];           // the (B, dim_total) buffer of every rank, this rank's own included
  int* flag_dst[8];        // the flag array of every rank (int[8]); this rank raises entry `rank` in each
  const int* flag_local;   // this rank's own flag array
  int* counter;            // local ticket of the CTAs that have finished storing (returns to 0)
  int* status;             // [0] != 0: gave up; [1] the rank waited for, [2] its flag, [3] the generation
  int n, rank, B, dim_local, dim_total, col0, generation;
  unsigned long long limit_ns;
};

__global__ void __launch_bounds__(256) decode_exchange_kernel(const ExchangeParams p) {
  mca_pdl_launch_dependents();
  mca_pdl_wait();          // src is the output of the kernel before
  const int v_per_row = p.dim_local / 4;
  const int total = p.B * v_per_row;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int b = idx / v_per_row, c = idx - b * v_per_row;
    const float4 v = *reinterpret_cast<const float4*>(p.src + (int64_t)b * p.dim_local + c * 4);
    const int64_t off = (int64_t)b * p.dim_total + p.col0 + c * 4;
#pragma unroll
    for (int d = 0; d < 8; ++d)   // constant indices: the parameter block stays in constant memory
      if (d < p.n) *reinterpret_cast<float4*>(p.dst[d] + off) = v;
  }
  __threadfence_system();          // this thread's peer stores are ordered before what follows
  __syncthreads();
  if (threadIdx.x != 0) return;
  const int ticket = atomicAdd(p.counter, 1);
  if (ticket != (int)gridDim.x - 1) return;
  // last CTA: every store of this rank has been issued and fenced
  *p.counter = 0;
  __threadfence_system();
#pragma unroll
  for (int d = 0; d < 8; ++d)
    if (d < p.n) asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.flag_dst[d] + p.rank), "r"(p.generation) : "memory");
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (int r = 0; r < p.n; ++r) {
    int f;
    unsigned polls = 0;
    for (;;) {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(f) : "l"(p.flag_local + r) : "memory");
      if (f - p.generation >= 0) break;           // generations only grow (wrap-safe comparison)
      if ((++polls & 63u) == 0) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > p.limit_ns) {
          if (atomicCAS(p.status, 0, 3) == 0) { p.status[1] = r; p.status[2] = f; p.status[3] = p.generation; }
          return;
        }
      }
    }
  }
}

template <typename CT, int HS>
int launch_decode(const DecodeParams& p, int B, cudaStream_t st) {
  const int kvmt = p.kv_mul >= 4 ? 4 : p.kv_mul;
  dim3 grid(p.nsplit, p.n_heads / kvmt, B);
  const size_t smem = sizeof(CT) == 2 ? DecRing<Epl<CT, HS>::value / 8>::BYTES : 0;   // the bf16 path's cp.async ring
  if (smem) {
    MCA_CUDA_TRY(cudaFuncSetAttribute(decode_split_kernel<CT, HS, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MCA_CUDA_TRY(cudaFuncSetAttribute(decode_split_kernel<CT, HS, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MCA_CUDA_TRY(cudaFuncSetAttribute(decode_split_kernel<CT, HS, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  // Up to eight sequences the kernel is launched ahead of the one before it (resident and waiting when that one
  // finishes: the step is short and the launch latency shows, + 6 % at one sequence).  With more sequences the
  // kernels either side of it in a decode step are the tensor-core projections, and the whole step measured 15-25 %
  // slower with the attention launched ahead of them: an ordinary launch.
  int e;
  if (B <= 8) {
    switch (kvmt) {
      case 1: e = mca_launch_pdl(decode_split_kernel<CT, HS, 1>, grid, dim3(DEC_THREADS), smem, st, p); break;
      case 2: e = mca_launch_pdl(decode_split_kernel<CT, HS, 2>, grid, dim3(DEC_THREADS), smem, st, p); break;
      case 4: e = mca_launch_pdl(decode_split_kernel<CT, HS, 4>, grid, dim3(DEC_THREADS), smem, st, p); break;
      default: return ERROR_ATTN_UNSUPPORTED_SHAPE;
    }
  } else {
    switch (kvmt) {
      case 1: decode_split_kernel<CT, HS, 1><<<grid, DEC_THREADS, smem, st>>>(p); break;
      case 2: decode_split_kernel<CT, HS, 2><<<grid, DEC_THREADS, smem, st>>>(p); break;
      case 4: decode_split_kernel<CT, HS, 4><<<grid, DEC_THREADS, smem, st>>>(p); break;
      default: return ERROR_ATTN_UNSUPPORTED_SHAPE;
    }
    e = mca_launch_status();
  }
  if (e) return e;
  if (p.nsplit > 1) {
    // programmatic dependent launch: the combine pass is resident and waiting when the last split finishes
    e = mca_launch_pdl(decode_combine_kernel<HS>, dim3(p.n_heads, B), dim3(HS), 0, st, (const float*)p.part_acc,
                       (const float*)p.part_ml, p.pos, p.n_heads, p.nsplit, p.split_len, p.pos_limit, p.out);
  }
  return e;
}

}  // namespace

int mca_decode_plan(int B, int n_heads, int n_kv_heads, int head_size, int max_len, int* split_len, int* nsplit,
                    int64_t* scratch_floats) {
  if (B <= 0 || n_heads <= 0 || n_kv_heads <= 0 || max_len <= 0 || n_heads % n_kv_heads != 0)
    return ERROR_PARAM_OUT_OF_RANGE;
  // Aim for about two waves of CTAs over 148 SMs x 2 resident CTAs (short splits pay their set-up and the combine
  // pass again; fewer waves leave ragged lengths unbalanced), with at least 128 keys each.
  const int64_t rows = (int64_t)B * n_kv_heads * max_len;
  int64_t sl = rows / (148 * 2 * 2);
  sl = (sl + 127) / 128 * 128;
  if (sl < 128) sl = 128;
  if (sl > 1024) sl = 1024;
  const int64_t groups = (int64_t)B * n_kv_heads;       // CTAs per split
  if (groups * ((max_len + 127) / 128) <= 4 * 296) {
    // Few CTAs (one sequence, or a handful): a partly filled last wave costs as much as a full one, so the split
    // count is chosen by whole waves over the 296 resident CTAs -- time ~ waves x (set-up, about 64 keys' worth, + keys
    // per split) -- instead of by a fixed length.  One sequence of 2339 keys and 32 heads: 9 splits of 260 keys in one
    // wave, where 128-key splits give 608 CTAs, i.e. two waves and sixteen stragglers.
    int64_t best_cost = INT64_MAX;
    int best_n = 1;
    for (int n = 1; n <= std::max(1, max_len / 128); ++n) {   // splits of at least 128 keys; up to 255 keys: one split, no scratch
      const int64_t len = ((max_len + n - 1) / n + 15) / 16 * 16;
      const int64_t waves = (groups * n + 295) / 296;
      const int64_t cost = waves * (64 + len);
      if (cost < best_cost) { best_cost = cost; best_n = n; }
    }
    sl = (((int64_t)max_len + best_n - 1) / best_n + 15) / 16 * 16;
  }
  {
    // tuning aid: MCA_DECODE_SPLIT_LEN=<keys> (a multiple of 16) overrides the planned split length for every call of
    // the process; read once
    static const int forced = [] {
      const char* e = getenv("MCA_DECODE_SPLIT_LEN");
      const int v = e ? atoi(e) : 0;
      return (v >= 16 && v % 16 == 0) ? v : 0;
    }();
    if (forced) sl = forced;
  }
  *split_len = (int)sl;
  *nsplit = (max_len + (int)sl - 1) / (int)sl;
  *scratch_floats = (int64_t)B * n_heads * (*nsplit) * (head_size + 2);
  return 0;
}

int64_t mca_decode_static_scratch_floats(void) { return MCA_STATIC_SCRATCH_FLOATS; }

int mca_decode_attention_static(const float* q, const float* k_new, const float* v_new, void* k_cache, void* v_cache,
                                int cache_is_bf16, int64_t cache_batch_stride, const int* pos, int B, int n_heads,
                                int n_kv_heads, int head_size, int seq_len, int max_len, const float* freq_real,
                                const float* freq_imag, float* out, void* stream) {
  // Device address of the static scratch, looked up once per device with that device current.
  static std::mutex lock;
  static float* dev_ptr[64] = {nullptr};
  int dev = -1;
  MCA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ERROR_PARAM_OUT_OF_RANGE;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> g(lock);
    if (dev_ptr[dev] == nullptr) {
      void* p = nullptr;
      MCA_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_decode_scratch));
      dev_ptr[dev] = static_cast<float*>(p);
    }
    scratch = dev_ptr[dev];
  }
  int split_len = 0, nsplit = 0;
  int64_t need = 0;
  int e = mca_decode_plan(B, n_heads, n_kv_heads, head_size, max_len, &split_len, &nsplit, &need);
  if (e) return e;
  if (nsplit > 1 && need > MCA_STATIC_SCRATCH_FLOATS) return ERROR_ATTN_STATIC_SCRATCH_EXCEEDED;
  return mca_decode_attention(q, k_new, v_new, k_cache, v_cache, cache_is_bf16, cache_batch_stride, pos, B, n_heads,
                              n_kv_heads, head_size, seq_len, max_len, freq_real, freq_imag, scratch,
                              MCA_STATIC_SCRATCH_FLOATS, out, stream);
}

int mca_decode_attention(const float* q, const float* k_new, const float* v_new, void* k_cache, void* v_cache,
                         int cache_is_bf16, int64_t cache_batch_stride, const int* pos, int B, int n_heads,
                         int n_kv_heads, int head_size, int seq_len, int max_len, const float* freq_real,
                         const float* freq_imag, float* scratch, int64_t scratch_floats, float* out, void* stream) {
  if (!q || !k_cache || !v_cache || !pos || !out) return ERROR_PARAM_NULL;
  if ((k_new == nullptr) != (v_new == nullptr)) return ERROR_PARAM_NULL;
  if ((freq_real == nullptr) != (freq_imag == nullptr)) return ERROR_PARAM_NULL;
  if (!mca_decode_head_size_supported(head_size)) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  if (max_len <= 0 || max_len > seq_len || B > 65535) return ERROR_PARAM_OUT_OF_RANGE;
  {
    // The kernels read and write cache rows as 16-byte vectors: base addresses must be 16-byte aligned and the
    // distance between sequences a whole number of vectors (rows are: kv_dim is a multiple of 16 elements).
    const int vec = cache_is_bf16 ? 8 : 4;
    if (((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) != 0) return ERROR_PARAM_OUT_OF_RANGE;
    if (cache_batch_stride % vec != 0 || cache_batch_stride < (int64_t)max_len * n_kv_heads * head_size) return ERROR_PARAM_OUT_OF_RANGE;
    if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(k_new) |
          reinterpret_cast<uintptr_t>(v_new) | reinterpret_cast<uintptr_t>(pos)) & 3) != 0)
      return ERROR_PARAM_OUT_OF_RANGE;
  }
  DecodeParams p;
  int64_t need = 0;
  int e = mca_decode_plan(B, n_heads, n_kv_heads, head_size, max_len, &p.split_len, &p.nsplit, &need);
  if (e) return e;
  if (p.nsplit > 1 && (scratch == nullptr || scratch_floats < need)) return ERROR_ATTN_SCRATCH_TOO_SMALL;
  p.q = q; p.k_new = k_new; p.v_new = v_new; p.k_cache = k_cache; p.v_cache = v_cache; p.pos = pos;
  p.fr = freq_real; p.fi = freq_imag; p.out = out;
  p.part_acc = scratch;
  p.part_ml = scratch ? scratch + (int64_t)B * n_heads * p.nsplit * head_size : nullptr;
  p.cache_batch_stride = cache_batch_stride;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.kv_mul = n_heads / n_kv_heads; p.seq_len = seq_len;
  p.pos_limit = max_len;   // <= seq_len, and the planned splits cover [0, max_len)
  if (p.kv_mul > 4 && p.kv_mul % 4 != 0) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  if (p.kv_mul == 3) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  switch (head_size) {
#define MCA_DECODE_CASE(HS_) \
    case HS_: return cache_is_bf16 ? launch_decode<__nv_bfloat16, HS_>(p, B, st) : launch_decode<float, HS_>(p, B, st);
    MCA_DECODE_CASE(32) MCA_DECODE_CASE(48) MCA_DECODE_CASE(64) MCA_DECODE_CASE(96) MCA_DECODE_CASE(128)
#undef MCA_DECODE_CASE
  }
  return ERROR_ATTN_UNSUPPORTED_SHAPE;
}

int mca_decode_head_size_supported(int head_size) {
  return head_size == 32 || head_size == 48 || head_size == 64 || head_size == 96 || head_size == 128;
}

int mca_decode_status(int* status3) {
  if (!status3) return ERROR_PARAM_NULL;
  int st[4] = {0, 0, 0, 0};
  MCA_CUDA_TRY(cudaMemcpyFromSymbol(st, g_decode_status, sizeof(st)));
  if (st[0] != 0) {
    const int zero[4] = {0, 0, 0, 0};
    MCA_CUDA_TRY(cudaMemcpyToSymbol(g_decode_status, zero, sizeof(zero)));
  }
  status3[0] = st[0]; status3[1] = st[1]; status3[2] = st[2];
  return 0;
}

int mca_decode_exchange(const float* src, float* const* dst, int* const* flag_dst, const int* flag_local, int* counter,
                        int* status, int n, int rank, int B, int dim_local, int dim_total, int col0, int generation,
                        int limit_ms, void* stream) {
  if (!src || !dst || !flag_dst || !flag_local || !counter || !status) return ERROR_PARAM_NULL;
  if (n < 1 || n > 8 || rank < 0 || rank >= n || B <= 0 || dim_local <= 0 || dim_local % 4 || dim_total % 4 || col0 % 4 ||
      col0 < 0 || col0 + dim_local > dim_total || limit_ms <= 0 || limit_ms > 10000)
    return ERROR_PARAM_OUT_OF_RANGE;
  ExchangeParams p;
  uintptr_t bits = reinterpret_cast<uintptr_t>(src);
  for (int i = 0; i < 8; ++i) {
    p.dst[i] = i < n ? dst[i] : nullptr;
    p.flag_dst[i] = i < n ? flag_dst[i] : nullptr;
    if (i < n) {
      if (!dst[i] || !flag_dst[i]) return ERROR_PARAM_NULL;
      bits |= reinterpret_cast<uintptr_t>(dst[i]);
    }
  }
  if (bits & 15) return ERROR_PARAM_OUT_OF_RANGE;
  p.src = src; p.flag_local = flag_local; p.counter = counter; p.status = status;
  p.n = n; p.rank = rank; p.B = B; p.dim_local = dim_local; p.dim_total = dim_total; p.col0 = col0; p.generation = generation;
  p.limit_ns = (unsigned long long)limit_ms * 1000000ull;
  const int total = B * (dim_local / 4);
  const int blocks = std::max(1, std::min(148, (total + 255) / 256));
  return mca_launch_pdl(decode_exchange_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, p);
}

// CPU oracle for the MyCaffe attention hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, on the CPU, the arithmetic that the reference performs on
// its attention path.  Nothing in the shipped library links, loads or calls it:
// only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
// may use it, and only as the checker.
//
// Parity status: PINNED for the GPT scaled-dot-product forward/backward by the
// reference's in-tree golden vectors
// (MyCaffe.test/test_data/data/text/gpt/gpt-pico-csa{,3,B,3B}); the decode
// restatement is pinned against the reference's own CPU twin compiled from its
// source (CudaExtension.llm32.llama2/Files/llama2_cpu.cpp).  The TFT and RoPE
// restatements have no golden data in the tree ("parity unpinned": they follow
// the cited source lines only).
//
// Every function cites the reference file:line it follows (paths relative to
// the reference project root).  `ACC` selects the accumulation type: float
// reproduces the reference's fp32 arithmetic, double is the error yardstick.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// Value the reference writes over masked logits (finite, not -inf):
// CudaDnnDLL/Cuda Files/attn.cu:302-329 (fInf = -1e+29f).
constexpr float kMaskedLogit = -1e29f;

// Row softmax, max-subtracted, as cuDNN SOFTMAX_ACCURATE / llama2_cpu.cpp:204-222.
template <typename ACC>
inline void softmax_row(const ACC* s, int n, ACC* p) {
  ACC m = s[0];
  for (int j = 1; j < n; ++j) m = std::max(m, s[j]);
  ACC sum = 0;
  for (int j = 0; j < n; ++j) { p[j] = std::exp(s[j] - m); sum += p[j]; }
  for (int j = 0; j < n; ++j) p[j] /= sum;
}

// attnHandle<T>::Forward, CudaDnnDLL/Cuda Files/attn.cu:518-602:
//   S = (1/sqrt(D)) * Q K^T   (scale is the GEMM alpha, attn.cu:567)
//   S[masked] = -1e29         (attn.cu:571-583; mask kernels math.cu:2994-3057)
//   P = softmax_row(S)        (attn.cu:587)
//   Y = P V                   (attn.cu:598)
// mask_mode 0: none; 1: (T,T) mask, masked where mask==0 (apply_mask);
// 2: (B,T) key mask, masked where mask==0 (apply_mask_batch); 3: the lower-triangular mask of
// fillMask (CausalSelfAttentionLayer.cs:276-291) generated on the fly (same result as mode 1 with
// tril(ones), without holding a T x T array).
// q_begin/q_step select a strided subset of query rows (used to bound the
// work at very long T); rows not selected are left untouched.
template <typename ACC, typename OUT>
void sdpa_forward(const float* Q, const float* K, const float* V, const float* mask, int mask_mode,
                  int B, int H, int T, int D, OUT* Y, OUT* P_out, int q_begin, int q_step) {
  const ACC scale = ACC(1.0 / std::sqrt((double)D));
  const int64_t BH = (int64_t)B * H;
#pragma omp parallel
  {
    std::vector<ACC> s(T), p(T), y(D);
#pragma omp for collapse(2) schedule(dynamic, 4)
    for (int64_t bh = 0; bh < BH; ++bh) {
      for (int i = q_begin; i < T; i += q_step) {
        const int b = (int)(bh / H);
        const float* q = Q + (bh * T + i) * D;
        for (int j = 0; j < T; ++j) {
          const float* k = K + (bh * T + j) * D;
          ACC acc = 0;
          for (int d = 0; d < D; ++d) acc += ACC(q[d]) * ACC(k[d]);
          acc *= scale;
          if (mask_mode == 1 && mask[(int64_t)i * T + j] == 0.0f) acc = ACC(kMaskedLogit);
          if (mask_mode == 2 && mask[(int64_t)b * T + j] == 0.0f) acc = ACC(kMaskedLogit);
          if (mask_mode == 3 && j > i) acc = ACC(kMaskedLogit);
          s[j] = acc;
        }
        softmax_row<ACC>(s.data(), T, p.data());
        for (int d = 0; d < D; ++d) y[d] = 0;
        for (int j = 0; j < T; ++j) {
          const float* v = V + (bh * T + j) * D;
          const ACC pj = p[j];
          for (int d = 0; d < D; ++d) y[d] += pj * ACC(v[d]);
        }
        OUT* yo = Y + (bh * T + i) * D;
        for (int d = 0; d < D; ++d) yo[d] = OUT(y[d]);
        if (P_out) {
          OUT* po = P_out + (bh * T + i) * (int64_t)T;
          for (int j = 0; j < T; ++j) po[j] = OUT(p[j]);
        }
      }
    }
  }
}

// attnHandle<T>::Backward, CudaDnnDLL/Cuda Files/attn.cu:608-661 with
// blob<T>::matmulgrad attn.cu:380-397:
//   dP = dY V^T ; dV = P^T dY
//   dS = P o (dP - rowsum(dP o P))        (cuDNN softmax backward)
//   dS *= 1/sqrt(D)
//   dQ = dS K ; dK = dS^T Q
// The reference uses the probabilities saved by Forward and does not re-apply
// the mask (masked entries have P == 0 exactly, so their dS is 0).  Here P is
// recomputed with the same mask.
template <typename ACC, typename OUT>
void sdpa_backward(const float* Q, const float* K, const float* V, const float* dY, const float* mask,
                   int mask_mode, int B, int H, int T, int D, OUT* dQ, OUT* dK, OUT* dV) {
  const ACC scale = ACC(1.0 / std::sqrt((double)D));
  const int64_t BH = (int64_t)B * H;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t bh = 0; bh < BH; ++bh) {
    const int b = (int)(bh / H);
    std::vector<ACC> s(T), p(T), dp(T), ds(T), dq(D);
    std::vector<ACC> dk((size_t)T * D, 0), dv((size_t)T * D, 0);
    for (int i = 0; i < T; ++i) {
      const float* q = Q + (bh * T + i) * D;
      const float* dy = dY + (bh * T + i) * D;
      for (int j = 0; j < T; ++j) {
        const float* k = K + (bh * T + j) * D;
        ACC acc = 0;
        for (int d = 0; d < D; ++d) acc += ACC(q[d]) * ACC(k[d]);
        acc *= scale;
        if (mask_mode == 1 && mask[(int64_t)i * T + j] == 0.0f) acc = ACC(kMaskedLogit);
        if (mask_mode == 2 && mask[(int64_t)b * T + j] == 0.0f) acc = ACC(kMaskedLogit);
        if (mask_mode == 3 && j > i) acc = ACC(kMaskedLogit);
        s[j] = acc;
      }
      softmax_row<ACC>(s.data(), T, p.data());
      ACC dot = 0;
      for (int j = 0; j < T; ++j) {
        const float* v = V + (bh * T + j) * D;
        ACC acc = 0;
        for (int d = 0; d < D; ++d) acc += ACC(dy[d]) * ACC(v[d]);
        dp[j] = acc;
        dot += acc * p[j];
        for (int d = 0; d < D; ++d) dv[(size_t)j * D + d] += p[j] * ACC(dy[d]);
      }
      for (int d = 0; d < D; ++d) dq[d] = 0;
      for (int j = 0; j < T; ++j) {
        ds[j] = p[j] * (dp[j] - dot) * scale;
        const float* k = K + (bh * T + j) * D;
        for (int d = 0; d < D; ++d) {
          dq[d] += ds[j] * ACC(k[d]);
          dk[(size_t)j * D + d] += ds[j] * ACC(q[d]);
        }
      }
      OUT* dqo = dQ + (bh * T + i) * D;
      for (int d = 0; d < D; ++d) dqo[d] = OUT(dq[d]);
    }
    for (int64_t x = 0; x < (int64_t)T * D; ++x) {
      dK[bh * T * D + x] = OUT(dk[x]);
      dV[bh * T * D + x] = OUT(dv[x]);
    }
  }
}

// RopeDataCpu<T>::Initialize, CudaDnnDLL/Cuda Files/rope.cu:143-207 (the GPU
// twin rope.cu:501-553 builds the same table): freq_i = 1/powf(theta, 2i/D),
// cos/sin(pos*freq_i) evaluated with cosf/sinf in fp32.
void rope_tables(int T, int D, float theta, float* cos_t, float* sin_t) {
  const int half = D / 2;
  std::vector<float> freq(half);
  for (int i = 0, idx = 0; i < D; i += 2, ++idx) {
    float power = (float)(i / (float)D);
    power = powf(theta, power);
    freq[idx] = 1.0f / power;
  }
  for (int pos = 0; pos < T; ++pos)
    for (int i = 0; i < half; ++i) {
      const float f = freq[i] * pos;
      cos_t[(int64_t)pos * half + i] = cosf(f);
      sin_t[(int64_t)pos * half + i] = sinf(f);
    }
}

// RopeDataGpu<T>::Forward/Backward, rope.cu:724-864: x is (B,T,H,D); pair p =
// (x[2p], x[2p+1]); position = (p % (T*H*D/2)) / (H*D/2), frequency = p % (D/2);
// forward rotates by +angle, backward by -angle.  freq_offset > 0 shifts the
// table start (rope.cu:812-818), used by the KV-cache decode path.
void rope_apply(const float* x, float* y, int64_t n, int T, int H, int D, const float* cos_t,
                const float* sin_t, int freq_offset, bool backward) {
  const int half = D / 2;
  const int64_t full = (int64_t)half * H;
  const float* c = cos_t + (freq_offset > 0 ? freq_offset : 0);
  const float* s = sin_t + (freq_offset > 0 ? freq_offset : 0);
  for (int64_t p = 0; p < n / 2; ++p) {
    const int64_t base = p % ((int64_t)T * full);
    const int64_t idx = (base / full) * half + base % half;
    const float fc = c[idx], fs = s[idx];
    const float xr = x[2 * p], xi = x[2 * p + 1];
    if (!backward) { y[2 * p] = xr * fc - xi * fs; y[2 * p + 1] = xr * fs + xi * fc; }
    else           { y[2 * p] = xr * fc + xi * fs; y[2 * p + 1] = -xr * fs + xi * fc; }
  }
}

// MultiHeadAttentionInterpLayer<T>.forward attention block,
// MyCaffe.layers.tft/layers.tft/MultiHeadAttentionInterpLayer.cs:728-759:
//   S_h = Q_h K_h^T / sqrt(d_model) (:732-733); S[mask==1] = -1e29 (:743);
//   P_h = softmax(S_h) (:748); O_h = P_h V (V shared by all heads, :706-710,:751);
//   out = mean_h O_h, attn = mean_h P_h (:758-759, :244-264).
// Q: (B,H,Nq,d)  K: (B,H,Nk,d)  V: (B,Nk,d)  mask: (Nq,Nk) or null.
template <typename ACC, typename OUT>
void tft_forward(const float* Q, const float* K, const float* V, const float* mask, int B, int H, int Nq,
                 int Nk, int d, OUT* out, OUT* attn) {
  const ACC scale = ACC(1.0 / std::sqrt((double)d));
#pragma omp parallel
  {
    std::vector<ACC> s(Nk), p(Nk), pm(Nk), o(d), om(d);
#pragma omp for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
      for (int i = 0; i < Nq; ++i) {
        std::fill(pm.begin(), pm.end(), ACC(0));
        std::fill(om.begin(), om.end(), ACC(0));
        for (int h = 0; h < H; ++h) {
          const float* q = Q + (((int64_t)b * H + h) * Nq + i) * d;
          for (int j = 0; j < Nk; ++j) {
            const float* k = K + (((int64_t)b * H + h) * Nk + j) * d;
            ACC acc = 0;
            for (int x = 0; x < d; ++x) acc += ACC(q[x]) * ACC(k[x]);
            acc *= scale;
            if (mask && mask[(int64_t)i * Nk + j] == 1.0f) acc = ACC(kMaskedLogit);
            s[j] = acc;
          }
          softmax_row<ACC>(s.data(), Nk, p.data());
          std::fill(o.begin(), o.end(), ACC(0));
          for (int j = 0; j < Nk; ++j) {
            const float* v = V + ((int64_t)b * Nk + j) * d;
            for (int x = 0; x < d; ++x) o[x] += p[j] * ACC(v[x]);
          }
          // channel mean = running sum over heads then one scale by 1/H (:255-263)
          for (int j = 0; j < Nk; ++j) pm[j] += p[j];
          for (int x = 0; x < d; ++x) om[x] += o[x];
        }
        const ACC inv = ACC(1.0 / H);
        for (int x = 0; x < d; ++x) out[((int64_t)b * Nq + i) * d + x] = OUT(om[x] * inv);
        for (int j = 0; j < Nk; ++j) attn[((int64_t)b * Nq + i) * Nk + j] = OUT(pm[j] * inv);
      }
  }
}

// Backward of the block above, MultiHeadAttentionInterpLayer.cs:780-859 (same
// algebra as attn.cu:608-661 per head, plus the two head-means and the shared V):
// d_out (B,Nq,d), d_attn (B,Nq,Nk, may be null) -> dQ (B,H,Nq,d), dK (B,H,Nk,d), dV (B,Nk,d).
template <typename ACC, typename OUT>
void tft_backward(const float* Q, const float* K, const float* V, const float* mask, const float* d_out,
                  const float* d_attn, int B, int H, int Nq, int Nk, int d, OUT* dQ, OUT* dK, OUT* dV) {
  const ACC scale = ACC(1.0 / std::sqrt((double)d));
  const ACC inv = ACC(1.0 / H);
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    std::vector<ACC> s(Nk), p(Nk), dp(Nk);
    std::vector<ACC> dv((size_t)Nk * d, 0), dk((size_t)Nk * d), dq(d);
    for (int h = 0; h < H; ++h) {
      std::fill(dk.begin(), dk.end(), ACC(0));
      for (int i = 0; i < Nq; ++i) {
        const float* q = Q + (((int64_t)b * H + h) * Nq + i) * d;
        const float* go = d_out + ((int64_t)b * Nq + i) * d;
        for (int j = 0; j < Nk; ++j) {
          const float* k = K + (((int64_t)b * H + h) * Nk + j) * d;
          ACC acc = 0;
          for (int x = 0; x < d; ++x) acc += ACC(q[x]) * ACC(k[x]);
          acc *= scale;
          if (mask && mask[(int64_t)i * Nk + j] == 1.0f) acc = ACC(kMaskedLogit);
          s[j] = acc;
        }
        softmax_row<ACC>(s.data(), Nk, p.data());
        ACC dot = 0;
        for (int j = 0; j < Nk; ++j) {
          const float* v = V + ((int64_t)b * Nk + j) * d;
          ACC acc = 0;
          for (int x = 0; x < d; ++x) acc += ACC(go[x]) * inv * ACC(v[x]);
          if (d_attn) acc += ACC(d_attn[((int64_t)b * Nq + i) * Nk + j]) * inv;
          dp[j] = acc;
          dot += acc * p[j];
          for (int x = 0; x < d; ++x) dv[(size_t)j * d + x] += p[j] * ACC(go[x]) * inv;
        }
        std::fill(dq.begin(), dq.end(), ACC(0));
        for (int j = 0; j < Nk; ++j) {
          const ACC ds = p[j] * (dp[j] - dot) * scale;
          const float* k = K + (((int64_t)b * H + h) * Nk + j) * d;
          for (int x = 0; x < d; ++x) {
            dq[x] += ds * ACC(k[x]);
            dk[(size_t)j * d + x] += ds * ACC(q[x]);
          }
        }
        for (int x = 0; x < d; ++x) dQ[(((int64_t)b * H + h) * Nq + i) * d + x] = OUT(dq[x]);
      }
      for (int64_t x = 0; x < (int64_t)Nk * d; ++x) dK[((int64_t)b * H + h) * Nk * d + x] = OUT(dk[x]);
    }
    for (int64_t x = 0; x < (int64_t)Nk * d; ++x) dV[(int64_t)b * Nk * d + x] = OUT(dv[x]);
  }
}

// precompute_freqs_cis, CudaExtension.llm32.llama2/Files/llama2_cpu.cpp:388-414
// (theta fixed at 10000 there; parameterised here).
void llama_freqs(int head_size, int64_t seq_len, float theta, float* fr, float* fi) {
  std::vector<float> f(head_size / 2);
  for (int i = 0; i < head_size; i += 2) {
    float val = i / (float)head_size;
    float div = powf(theta, val);
    f[i / 2] = (div == 0.0f) ? 0 : 1.0f / div;
  }
  for (int64_t i = 0; i < seq_len; ++i)
    for (int j = 0; j < head_size / 2; ++j) {
      fr[i * head_size / 2 + j] = cosf(i * f[j]);
      fi[i * head_size / 2 + j] = sinf(i * f[j]);
    }
}

// rmsnorm, llama2_cpu.cpp:189-202.
void rmsnorm(float* o, const float* x, const float* w, int n, float eps) {
  float ss = 0.0f;
  for (int j = 0; j < n; ++j) ss += x[j] * x[j];
  ss /= n;
  ss += eps;
  ss = 1.0f / sqrtf(ss);
  for (int j = 0; j < n; ++j) o[j] = w[j] * (ss * x[j]);
}

// One decode step of the attention block for a batch of independent sequences,
// TransformerCpu::forward llama2_cpu.cpp:290-342 (rope :239-262, cache append
// :293-298, attention :304-342).  q: (B, n_heads*hs) and k,v: (B, kv_dim) are
// the projections for the new token BEFORE RoPE; caches are
// (B, seq_len, kv_dim) and are updated in place at row pos[b]; out: (B, dim).
// The reference rotates k with the q-head loop bound (llama2_cpu.cpp:244), which
// is only in range when n_kv_heads == n_heads; here k is rotated per kv head.
void llama_decode(float* q, float* k, const float* v, float* kc, float* vc, const int* pos, int B,
                  int n_heads, int n_kv_heads, int hs, int seq_len, const float* fr, const float* fi,
                  float* out, float* att_out) {
  const int kv_dim = n_kv_heads * hs, dim = n_heads * hs, kv_mul = n_heads / n_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int b = 0; b < B; ++b)
    for (int kvh = 0; kvh < n_kv_heads; ++kvh) {
      const int p = pos[b];
      const float* cr = fr + (int64_t)p * hs / 2;
      const float* ci = fi + (int64_t)p * hs / 2;
      float* kb = k + (int64_t)b * kv_dim + kvh * hs;
      for (int i = 0; i < hs; i += 2) {
        const float k0 = kb[i], k1 = kb[i + 1];
        kb[i] = k0 * cr[i / 2] - k1 * ci[i / 2];
        kb[i + 1] = k0 * ci[i / 2] + k1 * cr[i / 2];
      }
      float* kcb = kc + (int64_t)b * seq_len * kv_dim;
      float* vcb = vc + (int64_t)b * seq_len * kv_dim;
      memcpy(kcb + (int64_t)p * kv_dim + kvh * hs, kb, hs * sizeof(float));
      memcpy(vcb + (int64_t)p * kv_dim + kvh * hs, v + (int64_t)b * kv_dim + kvh * hs, hs * sizeof(float));
      std::vector<float> att(p + 1);
      for (int h = kvh * kv_mul; h < (kvh + 1) * kv_mul; ++h) {
        float* qh = q + (int64_t)b * dim + h * hs;
        for (int i = 0; i < hs; i += 2) {
          const float q0 = qh[i], q1 = qh[i + 1];
          qh[i] = q0 * cr[i / 2] - q1 * ci[i / 2];
          qh[i + 1] = q0 * ci[i / 2] + q1 * cr[i / 2];
        }
        for (int t = 0; t <= p; ++t) {
          const float* kk = kcb + (int64_t)t * kv_dim + kvh * hs;
          float score = 0.0f;
          for (int i = 0; i < hs; ++i) score += qh[i] * kk[i];
          score /= sqrtf((float)hs);
          att[t] = score;
        }
        softmax_row<float>(att.data(), p + 1, att.data());
        float* xb = out + (int64_t)b * dim + h * hs;
        memset(xb, 0, hs * sizeof(float));
        for (int t = 0; t <= p; ++t) {
          const float* vv = vcb + (int64_t)t * kv_dim + kvh * hs;
          const float a = att[t];
          for (int i = 0; i < hs; ++i) xb[i] += a * vv[i];
        }
        if (att_out) memcpy(att_out + ((int64_t)b * n_heads + h) * seq_len, att.data(), (p + 1) * sizeof(float));
      }
    }
}

// matmul, llama2_cpu.cpp:224-237: W (d,n) @ x (n) -> out (d).
void gemv(float* out, const float* x, const float* w, int n, int d) {
#pragma omp parallel for
  for (int i = 0; i < d; ++i) {
    float val = 0.0f;
    for (int j = 0; j < n; ++j) val += w[(int64_t)i * n + j] * x[j];
    out[i] = val;
  }
}

}  // namespace

extern "C" {

int oracle_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// The OpenMP team size of this process (the compiled reference twin shares the same runtime).  A launcher may
// export OMP_NUM_THREADS=1 for its workers; the CPU legs of the benchmark set the size they report explicitly.
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

void oracle_sdpa_forward_f32(const float* Q, const float* K, const float* V, const float* mask, int mask_mode,
                             int B, int H, int T, int D, float* Y, float* P) {
  sdpa_forward<float, float>(Q, K, V, mask, mask_mode, B, H, T, D, Y, P, 0, 1);
}
void oracle_sdpa_forward_f64(const float* Q, const float* K, const float* V, const float* mask, int mask_mode,
                             int B, int H, int T, int D, double* Y, double* P) {
  sdpa_forward<double, double>(Q, K, V, mask, mask_mode, B, H, T, D, Y, P, 0, 1);
}
// Strided subset of query rows (rows q_begin, q_begin+q_step, ...); other rows of Y untouched.
void oracle_sdpa_forward_rows_f32(const float* Q, const float* K, const float* V, const float* mask,
                                  int mask_mode, int B, int H, int T, int D, float* Y, int q_begin,
                                  int q_step) {
  sdpa_forward<float, float>(Q, K, V, mask, mask_mode, B, H, T, D, Y, nullptr, q_begin, q_step);
}
void oracle_sdpa_backward_f32(const float* Q, const float* K, const float* V, const float* dY,
                              const float* mask, int mask_mode, int B, int H, int T, int D, float* dQ,
                              float* dK, float* dV) {
  sdpa_backward<float, float>(Q, K, V, dY, mask, mask_mode, B, H, T, D, dQ, dK, dV);
}
void oracle_sdpa_backward_f64(const float* Q, const float* K, const float* V, const float* dY,
                              const float* mask, int mask_mode, int B, int H, int T, int D, double* dQ,
                              double* dK, double* dV) {
  sdpa_backward<double, double>(Q, K, V, dY, mask, mask_mode, B, H, T, D, dQ, dK, dV);
}
void oracle_rope_tables(int T, int D, float theta, float* cos_t, float* sin_t) {
  rope_tables(T, D, theta, cos_t, sin_t);
}
void oracle_rope_apply(const float* x, float* y, int64_t n, int T, int H, int D, const float* cos_t,
                       const float* sin_t, int freq_offset, int backward) {
  rope_apply(x, y, n, T, H, D, cos_t, sin_t, freq_offset, backward != 0);
}
void oracle_tft_forward_f32(const float* Q, const float* K, const float* V, const float* mask, int B, int H,
                            int Nq, int Nk, int d, float* out, float* attn) {
  tft_forward<float, float>(Q, K, V, mask, B, H, Nq, Nk, d, out, attn);
}
void oracle_tft_forward_f64(const float* Q, const float* K, const float* V, const float* mask, int B, int H,
                            int Nq, int Nk, int d, double* out, double* attn) {
  tft_forward<double, double>(Q, K, V, mask, B, H, Nq, Nk, d, out, attn);
}
void oracle_tft_backward_f64(const float* Q, const float* K, const float* V, const float* mask,
                             const float* d_out, const float* d_attn, int B, int H, int Nq, int Nk, int d,
                             double* dQ, double* dK, double* dV) {
  tft_backward<double, double>(Q, K, V, mask, d_out, d_attn, B, H, Nq, Nk, d, dQ, dK, dV);
}
void oracle_tft_backward_f32(const float* Q, const float* K, const float* V, const float* mask,
                             const float* d_out, const float* d_attn, int B, int H, int Nq, int Nk, int d,
                             float* dQ, float* dK, float* dV) {
  tft_backward<float, float>(Q, K, V, mask, d_out, d_attn, B, H, Nq, Nk, d, dQ, dK, dV);
}
void oracle_llama_freqs(int head_size, int64_t seq_len, float theta, float* fr, float* fi) {
  llama_freqs(head_size, seq_len, theta, fr, fi);
}
void oracle_rmsnorm(float* o, const float* x, const float* w, int n, float eps) { rmsnorm(o, x, w, n, eps); }
void oracle_gemv(float* out, const float* x, const float* w, int n, int d) { gemv(out, x, w, n, d); }
void oracle_llama_decode(float* q, float* k, const float* v, float* kc, float* vc, const int* pos, int B,
                         int n_heads, int n_kv_heads, int hs, int seq_len, const float* fr, const float* fi,
                         float* out, float* att_out) {
  llama_decode(q, k, v, kc, vc, pos, B, n_heads, n_kv_heads, hs, seq_len, fr, fi, out, att_out);
}

// ---- LayerNorm, operation by operation as LayerNormData<T>::Forward / Backward issue them
// (CudaDnnDLL/Cuda Files/layernorm.cu:291-333, :340-384).  channel_mean accumulates a row in
// double and rounds the mean to float (math.cu:6817-6831); everything else is float arithmetic.
void oracle_layernorm_fwd(const float* x, float* y, float* stdev, int64_t rows, int inner, float eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * inner;
    double acc = 0;
    for (int j = 0; j < inner; ++j) acc += (double)xr[j];
    const float mean = (float)(acc / (double)inner);
    acc = 0;
    for (int j = 0; j < inner; ++j) {
      const float xmu = xr[j] - mean;
      const float sq = xmu * xmu;          // powx(.., 2)
      acc += (double)sq;
    }
    const float var = (float)(acc / (double)inner);
    const float sd = sqrtf(var + eps);     // scale, add_scalar, sqrt
    stdev[r] = sd;
    for (int j = 0; j < inner; ++j) y[r * inner + j] = (xr[j] - mean) / sd;
  }
}
void oracle_layernorm_bwd(const float* y, const float* dy, const float* stdev, float* dx, int64_t rows, int inner, float eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float *yr = y + r * inner, *dyr = dy + r * inner;
    double a1 = 0, a2 = 0;
    for (int j = 0; j < inner; ++j) { a1 += (double)(yr[j] * dyr[j]); a2 += (double)dyr[j]; }
    const float m1 = (float)(a1 / (double)inner), m2 = (float)(a2 / (double)inner);
    for (int j = 0; j < inner; ++j) {
      float work = yr[j] * m1;
      work = work + m2;
      work = dyr[j] - work;
      // add_scalar(outer*channels, eps, stdevfull) touches the first `rows` elements of the
      // count-sized broadcast tensor only (layernorm.cu:377)
      const int64_t flat = r * inner + j;
      const float denom = flat < rows ? stdev[r] + eps : stdev[r];
      dx[flat] = work / denom;
    }
  }
}

// ---- RMSNorm layer, operation by operation as RMSNormLayer<T>.forward / backward issue them
// (MyCaffe.layers.gpt/layers.gpt/RMSNormLayer.cs:156-179, :190-231).  w may be null
// (enable_weights false).  dw sums over all rows (for outerNum == 1 this is the reference's channel_sum).
void oracle_rmsnorm_layer_fwd(const float* x, const float* w, float* y, float* inv_rms, int64_t rows, int inner, float eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * inner;
    double acc = 0;
    for (int j = 0; j < inner; ++j) acc += (double)(xr[j] * xr[j]);       // powx, channel_mean
    const float rms = sqrtf((float)(acc / (double)inner) + eps);          // sqrt(x + eps)
    const float inv = rms == 0.f ? 0.f : 1.0f / rms;                      // invert
    if (inv_rms) inv_rms[r] = inv;
    for (int j = 0; j < inner; ++j) {
      const float out = xr[j] * inv;
      y[r * inner + j] = w ? w[j] * out : out;
    }
  }
}
void oracle_rmsnorm_layer_bwd(const float* x, const float* w, const float* dy, float* dx, float* dw, int64_t rows, int inner,
                              float eps) {
  std::vector<double> dwacc(inner, 0.0);
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * inner, *dyr = dy + r * inner;
    double acc = 0;
    for (int j = 0; j < inner; ++j) acc += (double)(xr[j] * xr[j]);
    const float rms = sqrtf((float)(acc / (double)inner) + eps);
    const float inv = rms == 0.f ? 0.f : 1.0f / rms;
    double dinv_acc = 0;
    for (int j = 0; j < inner; ++j) {
      const float out = xr[j] * inv;
      if (w) dwacc[j] += (double)(dyr[j] * out);
      const float g = w ? dyr[j] * w[j] : dyr[j];
      dinv_acc += (double)(g * xr[j]);                                    // mul, channel_sumEx
    }
    const float dinv = (float)dinv_acc;
    const float rms2 = rms * rms;                                         // powx(rms, 2)
    const float neg_inv2 = rms2 == 0.f ? 0.f : -1.0f / rms2;              // invert(.., numerator -1)
    const float drms = dinv * neg_inv2;
    const float half_inv = rms == 0.f ? 0.f : 1.0f / (rms * 2.0f);        // invert(.., 1, 2)
    float dmean = half_inv * drms;
    dmean = dmean * (float)(1.0 / (double)inner);                         // channel_duplicate, scal(1/inner)
    for (int j = 0; j < inner; ++j) {
      const float g = w ? dyr[j] * w[j] : dyr[j];
      const float dxa = g * inv;
      float dxb = 2.0f * xr[j];                                           // scale(2, x)
      dxb = dxb * dmean;
      dx[r * inner + j] = dxb + dxa;                                      // add
    }
  }
  if (dw) for (int j = 0; j < inner; ++j) dw[j] = (float)dwacc[j];
}

}  // extern "C"

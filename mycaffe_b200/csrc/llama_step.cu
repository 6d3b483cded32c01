// One decode step of the whole llama2 transformer for B independent sequences: token -> logits.
// Replaces TransformerGpu::forward (CudaExtension.llm32.llama2/Files/llama2_gpu.cpp:32-111), which
// issues per layer rmsnorm, three cublasSgemv, rope, two cache copies, the attention kernel, the Wo
// cublasSgemv, add, rmsnorm, two cublasSgemv, siglu, cublasSgemv, add -- about 16 launches, several
// of them with a host synchronisation -- and is limited to one sequence.  Here a layer is five
// launches (six with the split-KV combine pass) on one stream and nothing touches the host:
//   1. RMSNorm + [Wq;Wk;Wv]            (mca_decode_qkv_rmsnorm)
//   2. RoPE + cache append + attention (mca_decode_attention, plus its combine pass)
//   3. Wo + residual                   (mca_decode_out_proj)
//   4. RMSNorm + W1/W3 + SwiGLU        (mca_decode_ffn, first launch)
//   5. W2 + residual                   (mca_decode_ffn, second launch)
// then the final RMSNorm + classifier.  The arithmetic follows the CPU twin
// (TransformerCpu::forward, llama2_cpu.cpp:264-386).  The call only enqueues work: it can be
// captured into a CUDA graph and replayed per token, since tokens and positions are read from
// device memory.
#include "common.cuh"
#include "kernels.h"

namespace {

// x[b, :] = table[token[b], :] (llama2_gpu.cpp:45-47).  A token outside the vocabulary reads row 0
// of the table instead of memory outside it.
__global__ void embed_rows_kernel(const float* __restrict__ table, const int* __restrict__ tokens, int vocab, int dim,
                                  float* __restrict__ x) {
  mca_pdl_launch_dependents();
  const int b = blockIdx.y;
  int t = tokens[b];
  if (t < 0 || t >= vocab) t = 0;
  const float4* src = reinterpret_cast<const float4*>(table + (int64_t)t * dim);
  float4* dst = reinterpret_cast<float4*>(x + (int64_t)b * dim);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim / 4; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

inline int64_t round4(int64_t n) { return (n + 3) / 4 * 4; }

struct Carve {
  int64_t x, q, k, v, att, h, scratch, total, scratch_floats;
};

int carve(const McaLlamaConfig& c, int B, int max_len, Carve* out) {
  if (c.dim <= 0 || c.hidden_dim <= 0 || c.n_layers <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 ||
      c.vocab_size <= 0 || c.seq_len <= 0 || B <= 0 || max_len <= 0 || max_len > c.seq_len)
    return ERROR_PARAM_OUT_OF_RANGE;
  if (c.dim % c.n_heads != 0 || c.n_heads % c.n_kv_heads != 0) return ERROR_PARAM_OUT_OF_RANGE;
  const int hs = c.dim / c.n_heads;
  const int64_t kv_dim = (int64_t)c.n_kv_heads * hs;
  int sl = 0, ns = 0;
  int64_t need = 0;
  int e = mca_decode_plan(B, c.n_heads, c.n_kv_heads, hs, max_len, &sl, &ns, &need);
  if (e) return e;
  Carve w;
  int64_t o = 0;
  w.x = o; o += round4((int64_t)B * c.dim);
  w.q = o; o += round4((int64_t)B * c.dim);
  w.k = o; o += round4(B * kv_dim);
  w.v = o; o += round4(B * kv_dim);
  w.att = o; o += round4((int64_t)B * c.dim);
  w.h = o; o += round4((int64_t)B * c.hidden_dim);
  w.scratch = o; o += round4(need);
  w.scratch_floats = need;
  w.total = o;
  *out = w;
  return 0;
}

}  // namespace

int64_t mca_llama_workspace_floats(const McaLlamaConfig* cfg, int B, int max_len) {
  Carve w;
  if (!cfg || carve(*cfg, B, max_len, &w)) return -1;
  return w.total;
}

int mca_llama_forward(const McaLlamaConfig* cfg, const McaLlamaWeights* wt, const McaLlamaState* st, const int* tokens,
                      const int* pos, int B, int max_len, float* logits, void* stream) {
  if (!cfg || !wt || !st || !tokens || !pos || !logits) return ERROR_PARAM_NULL;
  if (!wt->token_embedding_table || !wt->rms_att_weight || !wt->rms_ffn_weight || !wt->rms_final_weight || !wt->wq ||
      !wt->wk || !wt->wv || !wt->wo || !wt->w1 || !wt->w2 || !wt->w3 || !wt->wcls)
    return ERROR_PARAM_NULL;
  if (!st->key_cache || !st->value_cache || !st->freq_real || !st->freq_imag || !st->workspace) return ERROR_PARAM_NULL;
  Carve w;
  int e = carve(*cfg, B, max_len, &w);
  if (e) return e;
  if (st->workspace_floats < w.total) return ERROR_ATTN_SCRATCH_TOO_SMALL;
  if ((reinterpret_cast<uintptr_t>(st->workspace) & 15) != 0 || cfg->dim % 8 != 0 || cfg->hidden_dim % 8 != 0)
    return ERROR_PARAM_OUT_OF_RANGE;
  if ((reinterpret_cast<uintptr_t>(wt->token_embedding_table) & 15) != 0) return ERROR_PARAM_OUT_OF_RANGE;
  const int dim = cfg->dim, hidden = cfg->hidden_dim, hs = dim / cfg->n_heads;
  const int kv_dim = cfg->n_kv_heads * hs;
  const float eps = 1e-5f;  // rmsnorm, llama2_cpu.cpp:196
  cudaStream_t s = (cudaStream_t)stream;
  float* ws = st->workspace;
  float *x = ws + w.x, *q = ws + w.q, *k = ws + w.k, *v = ws + w.v, *att = ws + w.att, *h = ws + w.h;
  const size_t wb = wt->weights_bf16 ? 2 : 4, cb = st->cache_is_bf16 ? 2 : 4;
  auto mat = [&](const void* base, int64_t layer, int64_t rows, int64_t cols) -> const void* {
    return static_cast<const char*>(base) + (size_t)(layer * rows * cols) * wb;
  };

  embed_rows_kernel<<<dim3(mca_ceil_div(dim / 4, 256), B), 256, 0, s>>>(wt->token_embedding_table, tokens,
                                                                       cfg->vocab_size, dim, x);
  if ((e = mca_launch_status())) return e;

  const int64_t layer_cache = (int64_t)B * cfg->seq_len * kv_dim;   // caches are (layer, B, seq_len, kv_dim)
  for (int l = 0; l < cfg->n_layers; ++l) {
    e = mca_decode_qkv_rmsnorm(x, wt->rms_att_weight + (int64_t)l * dim, eps, mat(wt->wq, l, dim, dim),
                               mat(wt->wk, l, kv_dim, dim), mat(wt->wv, l, kv_dim, dim), wt->weights_bf16, B, dim,
                               kv_dim, q, k, v, stream);
    if (e) return e;
    void* kc = static_cast<char*>(st->key_cache) + (size_t)(l * layer_cache) * cb;
    void* vc = static_cast<char*>(st->value_cache) + (size_t)(l * layer_cache) * cb;
    e = mca_decode_attention(q, k, v, kc, vc, st->cache_is_bf16, (int64_t)cfg->seq_len * kv_dim, pos, B, cfg->n_heads,
                             cfg->n_kv_heads, hs, cfg->seq_len, max_len, st->freq_real, st->freq_imag,
                             ws + w.scratch, w.scratch_floats, att, stream);
    if (e) return e;
    e = mca_decode_out_proj(att, mat(wt->wo, l, dim, dim), wt->weights_bf16, B, dim, x, stream);
    if (e) return e;
    e = mca_decode_ffn(wt->rms_ffn_weight + (int64_t)l * dim, eps, mat(wt->w1, l, hidden, dim),
                       mat(wt->w2, l, dim, hidden), mat(wt->w3, l, hidden, dim), wt->weights_bf16, B, dim, hidden, h,
                       x, stream);
    if (e) return e;
  }
  return mca_decode_logits(x, wt->rms_final_weight, eps, wt->wcls, wt->weights_bf16, B, dim, cfg->vocab_size, logits,
                           stream);
}

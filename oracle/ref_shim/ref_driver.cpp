// C entry points around the reference's own TransformerCpu
// (CudaExtension.llm32.llama2/Files/llama2_cpu.cpp, class in llama2_cpu.h:71-95),
// compiled from the reference tree where it lies.  TEST INFRASTRUCTURE ONLY: the
// shipped library never loads this.  It lets the tests and the CPU-baseline leg
// of the benchmark run the reference's decode math and read its RunState.
#include "llama2_cpu.h"

extern "C" {

void* ref_llama_create(const char* checkpoint_path, long* err) {
  TransformerCpu* t = new TransformerCpu();
  long e = t->build(checkpoint_path);
  if (err) *err = e;
  if (e) { t->fd = -1; t->data = (float*)MAP_FAILED; return nullptr; }
  return t;
}

void ref_llama_config(void* h, int* out7) {
  Config* c = &((TransformerCpu*)h)->m_config;
  out7[0] = c->dim; out7[1] = c->hidden_dim; out7[2] = c->n_layers; out7[3] = c->n_heads;
  out7[4] = c->n_kv_heads; out7[5] = c->vocab_size; out7[6] = c->seq_len;
}

// Runs TransformerCpu::forward(token, pos) (llama2_cpu.cpp:264-386).
float* ref_llama_forward(void* h, int token, int pos) { return ((TransformerCpu*)h)->forward(token, pos); }

// which: 0 x, 1 xb, 2 xb2, 3 q, 4 k, 5 v, 6 att, 7 logits, 8 key_cache, 9 value_cache,
// 10 freq_real, 11 freq_imag  (RunState, llama2_cpu.h:50-69).
float* ref_llama_state(void* h, int which) {
  RunState* s = &((TransformerCpu*)h)->m_state;
  switch (which) {
    case 0: return s->x;    case 1: return s->xb;  case 2: return s->xb2; case 3: return s->q;
    case 4: return s->k;    case 5: return s->v;   case 6: return s->att; case 7: return s->logits;
    case 8: return s->key_cache; case 9: return s->value_cache;
    case 10: return s->freq_real; case 11: return s->freq_imag;
  }
  return nullptr;
}

void ref_llama_destroy(void* h) { delete (TransformerCpu*)h; }

// The reference's free functions, exposed for direct checks.
void ref_softmax(float* x, int size) { softmax(x, size); }
void ref_precompute_freqs_cis(int dim, size_t seq_len, float* fr, float* fi) {
  precompute_freqs_cis(dim, seq_len, fr, fi);
}

}  // extern "C"

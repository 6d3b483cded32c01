// The extension ABI of the llama2 route: the three entry points a parent CudaDnnDLL resolves in an
// extension library (CudaDnnDLL/Cuda Files/extension.cu:18-83) and the function ids
// CudaExtension.llm32.llama2 answers behind them (CudaExtension.llm32.cpp:20-26,91-268).
//
// What is here: CREATE / DESTROY / LOAD / QUERYSTATUS / ABORT with the reference's packing, and one
// added id (MCA_LLM_EXTENSION_FORWARD) that runs TransformerGpu::forward(token, pos) of the loaded
// model and returns the logits.  LOAD reads an 'ak42' version-1 checkpoint the way read_checkpoint
// and memory_map_weights do (Files/llama2_gpu.cpp:234-333: magic, version, Config, shared-classifier
// byte, weights from byte 256 in the fixed order), uploads it in one piece and allocates the caches,
// RoPE tables and workspace once; FORWARD is one mca_llama_forward call on the default stream.
// GENERATE and QUERYRESPONSE need the tokenizer and sampler, which are not part of this library:
// they answer ERROR_NOT_SUPPORTED with a message, like any id the reference does not know.
#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace {

// Windows codes the reference returns on this route.
constexpr MCA_LONG WIN_ERROR_INVALID_PARAMETER = 87;
constexpr MCA_LONG WIN_ERROR_NOT_SUPPORTED = 50;
constexpr MCA_LONG WIN_ERROR_FILE_INVALID = 1006;
constexpr MCA_LONG WIN_PEER_E_NOT_INITIALIZED = (MCA_LONG)0x80630001u;
// Files/llm.h:16-20
constexpr MCA_LONG ERROR_LLM_LOAD_MODEL = 10001;
constexpr MCA_LONG ERROR_LLM_LOAD_MODEL_MISSING_MODEL_FILE = 10002;

constexpr int kHeaderBytes = 256;
constexpr int kMaxSeqLen = 20480;  // read_checkpoint clamps seq_len (llama2_gpu.cpp:299-300)

typedef MCA_LONG (*InvokeFloatFn)(MCA_LONG, MCA_LONG, float*, MCA_LONG, float**, MCA_LONG*, MCA_LPTSTR, MCA_LONG);
typedef MCA_LONG (*AllocHostFn)(MCA_LONG, MCA_LONG, float**, float*, bool);

InvokeFloatFn g_parent_invoke = nullptr;
AllocHostFn g_parent_alloc_host = nullptr;
MCA_LONG g_parent_kernel = 0;

struct Llm {
  float temperature = 1.0f, topp = 0.9f;
  long seed = 0;
  std::atomic<bool> cancel{false}, busy{false};
  bool loaded = false;
  int device = 0;
  McaLlamaConfig cfg{};
  float* slab = nullptr;  // every weight of the checkpoint, in file order
  McaLlamaWeights w{};
  McaLlamaState st{};
  float* logits = nullptr;
  int* tok_pos = nullptr;  // device {token, pos}

  void release() {
    cudaFree(slab); cudaFree(st.key_cache); cudaFree(st.value_cache); cudaFree(const_cast<float*>(st.freq_real));
    cudaFree(const_cast<float*>(st.freq_imag)); cudaFree(st.workspace); cudaFree(logits); cudaFree(tok_pos);
    slab = nullptr; logits = nullptr; tok_pos = nullptr;
    st = McaLlamaState{};
    w = McaLlamaWeights{};
    loaded = false;
  }
  ~Llm() { release(); }
};

std::map<long, Llm*> g_llm;
std::mutex g_llm_lock;
long g_next_llm = 1;

Llm* find_llm(long h) {
  std::lock_guard<std::mutex> lock(g_llm_lock);
  auto it = g_llm.find(h);
  return it == g_llm.end() ? nullptr : it->second;
}

void message(MCA_LPTSTR szErr, MCA_LONG max, const char* text) {
  if (!szErr || max <= 0) return;
  strncpy(szErr, text, (size_t)max - 1);
  szErr[max - 1] = 0;
}

// "model.bin;tokenizer.bin" -> the model path (LLMData<T>::Load splits the same way, Files/llm.cpp:107-127).
std::string model_path_of(const char* input) {
  std::string s(input ? input : "");
  const size_t semi = s.find(';');
  if (semi != std::string::npos) s.resize(semi);
  return s;
}

MCA_LONG load_checkpoint(Llm* m, const std::string& path, MCA_LPTSTR szErr, MCA_LONG max) {
  m->release();
  const int fd = open(path.c_str(), O_RDONLY);
  if (fd < 0) return ERROR_LLM_LOAD_MODEL_MISSING_MODEL_FILE;
  struct stat sb;
  if (fstat(fd, &sb) != 0 || sb.st_size < kHeaderBytes) { close(fd); return WIN_ERROR_FILE_INVALID; }
  void* map = mmap(nullptr, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (map == MAP_FAILED) return WIN_ERROR_FILE_INVALID;
  struct Unmap { void* p; size_t n; ~Unmap() { munmap(p, n); } } unmap{map, (size_t)sb.st_size};
  const unsigned char* head = static_cast<const unsigned char*>(map);
  uint32_t magic;
  int32_t version, c[7];
  memcpy(&magic, head, 4);
  memcpy(&version, head + 4, 4);
  memcpy(c, head + 8, sizeof(c));
  const int shared_classifier = head[8 + sizeof(c)];
  if (magic != 0x616b3432u || version != 1) return WIN_ERROR_FILE_INVALID;
  McaLlamaConfig cfg{c[0], c[1], c[2], c[3], c[4], c[5], c[6]};
  if (cfg.seq_len > kMaxSeqLen) cfg.seq_len = kMaxSeqLen;
  if (cfg.dim <= 0 || cfg.hidden_dim <= 0 || cfg.n_layers <= 0 || cfg.n_heads <= 0 || cfg.n_kv_heads <= 0 ||
      cfg.vocab_size <= 0 || cfg.seq_len <= 0 || cfg.dim % cfg.n_heads || cfg.n_heads % cfg.n_kv_heads)
    return WIN_ERROR_FILE_INVALID;
  const int64_t L = cfg.n_layers, dim = cfg.dim, hid = cfg.hidden_dim, hs = dim / cfg.n_heads;
  const int64_t kv = (int64_t)cfg.n_kv_heads * hs, vocab = cfg.vocab_size;
  // memory_map_weights, llama2_gpu.cpp:242-259
  const int64_t sizes[12] = {L * dim, L * dim, dim, vocab * dim, L * dim * dim, L * kv * dim, L * kv * dim, L * dim * dim,
                             L * hid * dim, L * dim * hid, L * hid * dim, shared_classifier ? 0 : vocab * dim};
  int64_t off[13] = {0};
  for (int i = 0; i < 12; ++i) off[i + 1] = off[i] + sizes[i];
  if ((int64_t)sb.st_size < kHeaderBytes + off[12] * 4) return WIN_ERROR_FILE_INVALID;
  if (mca_llama_workspace_floats(&cfg, 1, cfg.seq_len) < 0) {
    message(szErr, max, "llama2 extension: this model shape has no decode kernel");
    return ERROR_ATTN_UNSUPPORTED_SHAPE;
  }

  if (cudaMalloc(&m->slab, (size_t)off[12] * 4) != cudaSuccess) { cudaGetLastError(); m->release(); return ERROR_MEMORY_OUT; }
  cudaError_t ce = cudaMemcpy(m->slab, head + kHeaderBytes, (size_t)off[12] * 4, cudaMemcpyHostToDevice);
  if (ce != cudaSuccess) { m->release(); return (MCA_LONG)ce; }
  const float* s = m->slab;
  m->w.rms_att_weight = s + off[0]; m->w.rms_ffn_weight = s + off[1]; m->w.rms_final_weight = s + off[2];
  m->w.token_embedding_table = s + off[3];
  m->w.wq = s + off[4]; m->w.wk = s + off[5]; m->w.wv = s + off[6]; m->w.wo = s + off[7];
  m->w.w1 = s + off[8]; m->w.w2 = s + off[9]; m->w.w3 = s + off[10];
  m->w.wcls = shared_classifier ? m->w.token_embedding_table : s + off[11];
  m->w.weights_bf16 = 0;

  const size_t cache_bytes = (size_t)(L * cfg.seq_len * kv) * 4;
  const size_t table = (size_t)cfg.seq_len * (hs / 2);
  const int64_t ws = mca_llama_workspace_floats(&cfg, 1, cfg.seq_len);
  float *fr = nullptr, *fi = nullptr;
  if (cudaMalloc(&m->st.key_cache, cache_bytes) != cudaSuccess || cudaMalloc(&m->st.value_cache, cache_bytes) != cudaSuccess ||
      cudaMalloc(&fr, table * 4) != cudaSuccess || cudaMalloc(&fi, table * 4) != cudaSuccess ||
      cudaMalloc(&m->st.workspace, (size_t)ws * 4) != cudaSuccess ||
      cudaMalloc(&m->logits, (size_t)vocab * 4) != cudaSuccess || cudaMalloc(&m->tok_pos, 2 * sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(fr); cudaFree(fi);
    m->release();
    return ERROR_MEMORY_OUT;
  }
  m->st.freq_real = fr; m->st.freq_imag = fi;
  m->st.cache_is_bf16 = 0;
  m->st.workspace_floats = ws;
  cudaMemset(m->st.key_cache, 0, cache_bytes);     // calloc in the reference (malloc_run_state)
  cudaMemset(m->st.value_cache, 0, cache_bytes);
  std::vector<float> c_t(table), s_t(table);
  mca_rope_tables_host(cfg.seq_len, (int)hs, 10000.0f, c_t.data(), s_t.data());  // precompute_freqs_cis, theta 10000
  cudaMemcpy(fr, c_t.data(), table * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(fi, s_t.data(), table * 4, cudaMemcpyHostToDevice);
  m->cfg = cfg;
  m->loaded = true;
  return 0;
}

MCA_LONG forward(Llm* m, int token, int pos, float** ppOutput, MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG max) {
  if (!m->loaded) { message(szErr, max, "llama2 extension: no model loaded"); return ERROR_LLM_LOAD_MODEL; }
  if (!ppOutput || !plOutput) return ERROR_PARAM_NULL;
  if (pos < 0 || pos >= m->cfg.seq_len || token < 0 || token >= m->cfg.vocab_size) return ERROR_PARAM_OUT_OF_RANGE;
  cudaError_t ce = cudaSetDevice(m->device);
  if (ce != cudaSuccess) return (MCA_LONG)ce;
  const int tp[2] = {token, pos};
  if ((ce = cudaMemcpyAsync(m->tok_pos, tp, sizeof(tp), cudaMemcpyHostToDevice, 0)) != cudaSuccess) return (MCA_LONG)ce;
  int e = mca_llama_forward(&m->cfg, &m->w, &m->st, m->tok_pos, m->tok_pos + 1, 1, pos + 1, m->logits, nullptr);
  if (e) return e;
  if ((ce = cudaStreamSynchronize(0)) != cudaSuccess) return (MCA_LONG)ce;
  // results travel in memory the parent allocates (and frees through its FREEMEM id)
  MCA_LONG le = g_parent_alloc_host(g_parent_kernel, m->cfg.vocab_size, ppOutput, m->logits, true);
  if (le) return le;
  *plOutput = m->cfg.vocab_size;
  return 0;
}

MCA_LONG small_result(const float* vals, int n, float** ppOutput, MCA_LONG* plOutput) {
  if (!ppOutput || !plOutput) return ERROR_PARAM_NULL;
  MCA_LONG e = g_parent_alloc_host(g_parent_kernel, n, ppOutput, const_cast<float*>(vals), false);
  if (e) return e;
  *plOutput = n;
  return 0;
}

}  // namespace

extern "C" {

MCA_LONG DLL_InitFloatCustomExtension(void* hParent, MCA_LONG lKernelIdx) {
  if (!hParent) return WIN_ERROR_INVALID_PARAMETER;
  InvokeFloatFn inv = (InvokeFloatFn)dlsym(hParent, "DLL_InvokeFloat");               // SZFN_INTERNAL_INVOKEFLOAT
  AllocHostFn alloc = (AllocHostFn)dlsym(hParent, "Internal_AllocHostFloat");         // SZFN_INTERNAL_ALLOCHOSTFLT
  if (!inv || !alloc) return WIN_ERROR_INVALID_PARAMETER;
  g_parent_invoke = inv;
  g_parent_alloc_host = alloc;
  g_parent_kernel = lKernelIdx;
  return 0;
}

MCA_LONG DLL_InvokeFloatCustomExtension(MCA_LONG lfnIdx, float* pInput, MCA_LONG lInput, float** ppOutput,
                                        MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG lErrMax) {
  if (!g_parent_invoke) return WIN_PEER_E_NOT_INITIALIZED;
  switch (lfnIdx) {
    case LLM_CUDA_EXTENSION_CREATE: {
      Llm* m = new Llm();
      if (lInput > 0 && pInput) m->temperature = pInput[0];
      if (lInput > 1 && pInput) m->topp = pInput[1];
      if (lInput > 2 && pInput) m->seed = (long)pInput[2];
      cudaGetDevice(&m->device);  // the parent's kernel made its device current
      long h;
      {
        std::lock_guard<std::mutex> lock(g_llm_lock);
        h = g_next_llm++;
        g_llm[h] = m;
      }
      const float v = (float)h;
      MCA_LONG e = small_result(&v, 1, ppOutput, plOutput);
      if (e) {
        std::lock_guard<std::mutex> lock(g_llm_lock);
        g_llm.erase(h);
        delete m;
      }
      return e;
    }
    case LLM_CUDA_EXTENSION_DESTROY: {
      if (lInput < 1 || !pInput) return WIN_ERROR_INVALID_PARAMETER;
      Llm* m = nullptr;
      {
        std::lock_guard<std::mutex> lock(g_llm_lock);
        auto it = g_llm.find((long)pInput[0]);
        if (it != g_llm.end()) { m = it->second; g_llm.erase(it); }
      }
      if (m) {
        m->cancel.store(true);
        for (int i = 0; i < 12 && m->busy.load(); ++i) usleep(250000);  // up to 3 s, as the reference waits
        if (!m->busy.load()) { cudaSetDevice(m->device); delete m; }
      }
      return 0;
    }
    case LLM_CUDA_EXTENSION_ABORT: {
      if (lInput < 1 || !pInput) return WIN_ERROR_INVALID_PARAMETER;
      if (Llm* m = find_llm((long)pInput[0])) m->cancel.store(true);
      return 0;
    }
    case LLM_CUDA_EXTENSION_QUERYSTATUS: {
      if (lInput < 1 || !pInput) return WIN_ERROR_INVALID_PARAMETER;
      Llm* m = find_llm((long)pInput[0]);
      if (!m) return WIN_ERROR_INVALID_PARAMETER;
      const float v[2] = {m->loaded ? 1.0f : 0.0f, m->loaded ? 1.0f : 0.0f};  // LLMData<T>::QueryStatus, llm.cpp:161-177
      return small_result(v, 2, ppOutput, plOutput);
    }
    case MCA_LLM_EXTENSION_FORWARD: {
      if (lInput < 3 || !pInput) return WIN_ERROR_INVALID_PARAMETER;
      Llm* m = find_llm((long)pInput[0]);
      if (!m) return WIN_ERROR_INVALID_PARAMETER;
      m->busy.store(true);
      MCA_LONG e = forward(m, (int)pInput[1], (int)pInput[2], ppOutput, plOutput, szErr, lErrMax);
      m->busy.store(false);
      return e;
    }
  }
  message(szErr, lErrMax, "The function specified is not supported.");
  return WIN_ERROR_NOT_SUPPORTED;
}

MCA_LONG DLL_InvokeFloatCustomExtensionEx(MCA_LONG lfnIdx, float* pInput, MCA_LONG lInput, float** ppOutput,
                                          MCA_LONG* plOutput, MCA_LPTSTR szInput, MCA_LPTSTR szOutput,
                                          MCA_LONG lOutputMax, MCA_LPTSTR szErr, MCA_LONG lErrMax) {
  (void)ppOutput; (void)plOutput; (void)szOutput; (void)lOutputMax;
  if (!g_parent_invoke) return WIN_PEER_E_NOT_INITIALIZED;
  switch (lfnIdx) {
    case LLM_CUDA_EXTENSION_LOAD: {
      if (lInput < 1 || !pInput) return WIN_ERROR_INVALID_PARAMETER;
      Llm* m = find_llm((long)pInput[0]);
      if (!m) return 0;  // the reference ignores an unknown handle here (CudaExtension.llm32.cpp:224-235)
      m->busy.store(true);
      cudaSetDevice(m->device);
      MCA_LONG e = load_checkpoint(m, model_path_of(szInput), szErr, lErrMax);
      m->busy.store(false);
      return e;
    }
    case LLM_CUDA_EXTENSION_GENERATE:
    case LLM_CUDA_EXTENSION_QUERYRESPONSE:
      message(szErr, lErrMax, "llama2 extension: text generation (tokenizer, sampler) is not provided; "
                              "use MCA_LLM_EXTENSION_FORWARD for the logits of one (token, pos).");
      return WIN_ERROR_NOT_SUPPORTED;
  }
  message(szErr, lErrMax, "The function specified is not supported.");
  return WIN_ERROR_NOT_SUPPORTED;
}

MCA_LONG DLL_InitDoubleCustomExtension(void*, MCA_LONG) { return ERROR_NOT_IMPLEMENTED; }

MCA_LONG DLL_InvokeDoubleCustomExtension(MCA_LONG, double*, MCA_LONG, double**, MCA_LONG*, MCA_LPTSTR szErr, MCA_LONG lErrMax) {
  message(szErr, lErrMax, "llama2 extension: the double base type is not implemented");
  return ERROR_NOT_IMPLEMENTED;
}

MCA_LONG DLL_InvokeDoubleCustomExtensionEx(MCA_LONG, double*, MCA_LONG, double**, MCA_LONG*, MCA_LPTSTR, MCA_LPTSTR, MCA_LONG,
                                           MCA_LPTSTR szErr, MCA_LONG lErrMax) {
  message(szErr, lErrMax, "llama2 extension: the double base type is not implemented");
  return ERROR_NOT_IMPLEMENTED;
}

}  // extern "C"

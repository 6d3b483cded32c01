// The reference's dispatch ABI for the attention path: kernel table, memory-handle table,
// function-id switch.  Mirrors CudaDnnDLL/CudaDnnDLL.cpp (exports), Cuda Files/main.cu
// (Kernel<T>::Run switch) and Cuda Files/device.h / device.cu (argument unpacking) for the
// ids listed in mycaffe_attn.h, and nothing else of that DLL.
#include <dlfcn.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int kMaxKernels = 2048;  // Cuda Files/main.h:21

struct MemItem {
  void* ptr = nullptr;
  int64_t count = 0;
  bool bf16 = false;
  size_t bytes() const { return (size_t)count * (bf16 ? 2 : 4); }
};

struct AttnHandle {
  bool configured = false;
  int B = 0, block = 0, H = 0, D = 0, dtype = MCA_DTYPE_F32, flags = 0;
  bool training = false;
  float dropout = 0.f;
  // owned device buffers, sized at Set for the configured block size
  float *row_max = nullptr, *row_sum = nullptr, *y_copy = nullptr, *delta = nullptr, *lse = nullptr;
  void* split_ws = nullptr;    // fp16 halves of q, k, v for the split-operand tensor-core forward of fp32 handles
  int64_t split_ws_bytes = 0;
  float* mask_ws = nullptr;    // fp32 copies for a bf16 handle that is given a (T,T) or batch mask (allocated on first use)
  size_t mask_ws_floats = 0;
  uint32_t *mask_bits = nullptr, *mask_bits_t = nullptr;   // keep-bits of a (T,T) or batch mask for the tensor-core kernels
  size_t mask_bits_words = 0;
  int* causal_flag = nullptr;  // [0] mask classification, [1..4] kernel status words, [6..7] the classification's scratch
  // A (T,T) mask is classified on every Forward, and the host has to know the class to choose the kernel.  In
  // synchronous mode the call ends with a blocking read of the status words anyway: the class is read with them, and
  // the kernels are chosen beforehand on the class the last verified call found.  A wrong guess that matters (taken
  // for the lower triangle, is not) is found by that read and the Forward runs again with the class known; nothing
  // unverified is ever returned.
  int spec_class = -1;         // what the last verified classification found (1 lower triangle, 0 other), -1 none yet
  int spec_assumed = 0;
  bool spec_pending = false;   // this call's kernels were chosen on spec_class; the read at its end checks it
  bool spec_allowed = true;
  // state of the last forward, consumed by backward
  bool have_fwd = false;
  int fwd_T = 0, fwd_mask_mode = 0, fwd_layout = 0;
  long fwd_mask_handle = 0;   // memory handle of the forward's mask (0: none); resolved again by Backward
  bool fwd_batch_mask = false;
  bool fwd_split = false;       // the forward was the split-operand tensor-core kernel: its workspace holds q, k, v halves
  bool status_pending = false;  // a tensor-core launch was made in asynchronous mode and its status words are unread
  void release() {
    cudaFree(row_max); cudaFree(row_sum); cudaFree(y_copy); cudaFree(delta); cudaFree(lse); cudaFree(causal_flag);
    cudaFree(split_ws); cudaFree(mask_ws); cudaFree(mask_bits); cudaFree(mask_bits_t);
    split_ws = nullptr; split_ws_bytes = 0;
    mask_ws = nullptr; mask_ws_floats = 0;
    mask_bits = mask_bits_t = nullptr; mask_bits_words = 0;
    row_max = row_sum = y_copy = delta = lse = nullptr;
    causal_flag = nullptr;
    configured = have_fwd = false;
    fwd_mask_handle = 0;
  }
};

struct RopeHandle {
  int B = 0, T = 0, H = 0, D = 0, shared_index = 0, refs = 1;
  float *cos_t = nullptr, *sin_t = nullptr;
};

struct DecodeHandle {
  int B = 0, n_heads = 0, n_kv_heads = 0, hs = 0, seq_len = 0;
  bool bf16 = false;
  float *fr = nullptr, *fi = nullptr, *scratch = nullptr;
  int64_t scratch_floats = 0;
};

struct LayerNormHandle {
  int64_t rows = 0;
  int inner = 0;
  float eps = 0.f;
  float* stdev = nullptr;   // (rows) from the last forward
  bool have_fwd = false;
};

// An extension library loaded through CUDA_FN_CREATE_EXTENSION (extensionHandle<T>, Cuda Files/extension.h:57-90).
typedef MCA_LONG (*ExtInitFn)(void*, MCA_LONG);
typedef MCA_LONG (*ExtInvokeFn)(MCA_LONG, float*, MCA_LONG, float**, MCA_LONG*, MCA_LPTSTR, MCA_LONG);
typedef MCA_LONG (*ExtInvokeExFn)(MCA_LONG, float*, MCA_LONG, float**, MCA_LONG*, MCA_LPTSTR, MCA_LPTSTR, MCA_LONG, MCA_LPTSTR,
                                  MCA_LONG);
struct ExtensionHandle {
  void* lib = nullptr;       // dlopen handle (null: the extension entry points of this library itself)
  ExtInvokeFn run = nullptr;
  ExtInvokeExFn run_ex = nullptr;
};

struct CallCounter {
  long calls = 0, errors = 0;
  double gpu_ms_last = 0.0, gpu_ms_total = 0.0;
};

struct Kernel {
  int device = 0;
  bool async = false;
  bool timing = false;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::map<long, CallCounter> counters;
  std::unordered_map<long, ExtensionHandle> extensions;
  long next_handle = 1;
  std::unordered_map<long, MemItem> mem;
  std::unordered_map<long, AttnHandle> attn;
  std::unordered_map<long, RopeHandle> rope;
  std::unordered_map<long, DecodeHandle> decode;
  std::unordered_map<long, LayerNormHandle> layernorm;
  float* norm_scratch = nullptr;   // grow-only: dW partials of the RMSNorm backward
  int64_t norm_scratch_floats = 0;
  std::unordered_map<long, int> cudnn;
  std::vector<void*> host_bufs;
  std::string last_detail;
  float* stage = nullptr;  // grow-only fp32 staging buffer for float <-> bf16 transfers
  size_t stage_count = 0;
  int* h_answer = nullptr; // eight pinned words for small device answers the host has to wait for (a mask's class in
                           // [0], an attention handle's class + status words in [2..6])
  int* answer_words() {
    if (h_answer == nullptr && cudaMallocHost((void**)&h_answer, 8 * sizeof(int)) != cudaSuccess) {
      cudaGetLastError();
      h_answer = nullptr;
    }
    return h_answer;
  }

  float* staging(size_t count) {
    if (count > stage_count) {
      cudaFree(stage);
      stage = nullptr;
      stage_count = 0;
      if (cudaMalloc(&stage, count * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
      stage_count = count;
    }
    return stage;
  }

  MemItem* get(long h) {
    auto it = mem.find(h);
    return it == mem.end() ? nullptr : &it->second;
  }
};

Kernel* g_kernels[kMaxKernels];
std::mutex g_table_lock;

const char* error_name(long e) {
  switch (e) {
    case ERROR_DLL_NOT_INIT: return "DLL not initialized";
    case ERROR_PARAM_OUT_OF_RANGE: return "parameter out of range";
    case ERROR_PARAM_NULL: return "parameter null";
    case ERROR_MEMORY_OUT: return "out of memory";
    case ERROR_NOT_IMPLEMENTED: return "not implemented";
    case ERROR_MEMORY_RANGE_EXCEEDED: return "memory range exceeded";
    case ERROR_MEMORY_MIXED_HALF_TYPES: return "memory handle has the wrong element type";
    case ERROR_MEMORY_NOT_FOUND: return "memory handle not found";
    case ERROR_MEMORY_TOO_SMALL: return "memory too small";
    case ERROR_ROPE_NOT_INITIALIZED: return "rope not initialized";
    case ERROR_LAYERNORM_NOT_INITIALIZED: return "layernorm not initialized";
    case ERROR_ATTN_NOT_INITIALIZED: return "attn not initialized";
    case ERROR_ATTN + 3: return "attn missing descriptor";
    case ERROR_ATTN_INCOMPATIBLE_BLOB_SIZE: return "attn incompatible blob size";
    case ERROR_ATTN_INVALID_BLOCK_SIZE: return "attn invalid block size";
    case ERROR_ATTN_UNSUPPORTED_SHAPE: return "attn: no sm_100a kernel for this head size / dtype / mask";
    case ERROR_ATTN_KERNEL_TIMEOUT: return "attn: a bounded device-side wait gave up";
    case ERROR_ATTN_BACKWARD_WITHOUT_FORWARD: return "attn: backward needs a training-mode forward at the configured block size on the same handle";
    case ERROR_ATTN_NOT_B200: return "attn: device is not compute capability 10.x";
    case ERROR_ATTN_SCRATCH_TOO_SMALL: return "attn: scratch too small";
    case ERROR_ATTN_STATIC_SCRATCH_EXCEEDED: return "attn: problem too large for the library's built-in decode scratch";
  }
  return nullptr;
}

// getError, CudaDnnDLL.cpp:1727-1745: copy a message for the code into the caller's buffer.
void get_error(long err, MCA_LPTSTR szErr, MCA_LONG max, const Kernel* k = nullptr) {
  if (!szErr || max <= 0) return;
  const char* name = error_name(err);
  char buf[512];
  if (name) snprintf(buf, sizeof(buf), "MyCaffe attn (%ld): %s", err, name);
  else if (err > 0 && err < 2000) snprintf(buf, sizeof(buf), "CUDA (%ld): %s", err, cudaGetErrorString((cudaError_t)err));
  else snprintf(buf, sizeof(buf), "error %ld", err);
  if (k && !k->last_detail.empty()) {
    size_t n = strlen(buf);
    snprintf(buf + n, sizeof(buf) - n, " [%s]", k->last_detail.c_str());
  }
  strncpy(szErr, buf, (size_t)max - 1);
  szErr[max - 1] = 0;
}

long verify_in(long n, const void* p, long lo, long hi) {  // Device<T>::verifyInput, device.h:710-740
  if (n < lo || n > hi) return ERROR_PARAM_OUT_OF_RANGE;
  if (lo == 0 && hi == 0) return 0;
  if (p == nullptr) return ERROR_PARAM_NULL;
  return 0;
}
long verify_out(MCA_LONG* plOutput, float** ppOutput) {  // device.h:742-752
  if (!plOutput || !ppOutput) return ERROR_PARAM_NULL;
  return 0;
}
long set_out(float v, MCA_LONG* plOutput, float** ppOutput) {
  *plOutput = 1;
  (*ppOutput)[0] = v;
  return 0;
}

long finish(Kernel* k, long err) {
  if (err) return err;
  if (!k->async) return (long)cudaStreamSynchronize(0);  // the reference blocks after every op (attn.cu:601)
  return 0;
}

long check_f32(Kernel* k, long h, int64_t need, float** out) {
  MemItem* m = k->get(h);
  if (!m) return ERROR_MEMORY_NOT_FOUND;
  if (m->bf16) return ERROR_MEMORY_MIXED_HALF_TYPES;
  if (m->count < need) return ERROR_MEMORY_TOO_SMALL;
  *out = (float*)m->ptr;
  return 0;
}
long check_any(Kernel* k, long h, int64_t need, bool want_bf16, void** out) {
  MemItem* m = k->get(h);
  if (!m) return ERROR_MEMORY_NOT_FOUND;
  if (m->bf16 != want_bf16) return ERROR_MEMORY_MIXED_HALF_TYPES;
  if (m->count < need) return ERROR_MEMORY_TOO_SMALL;
  *out = m->ptr;
  return 0;
}

// ---- memory ids -------------------------------------------------------------------------

long alloc_mem(Kernel* k, long lInput, float* pf, long llInput, MCA_LONGLONG* pl, MCA_LONG* plOutput,
               float** ppOutput, bool bf16) {
  long e;
  if ((e = verify_in(llInput, pl, 1, 2))) return e;
  if ((e = verify_out(plOutput, ppOutput))) return e;
  const int64_t count = pl[0];
  if (count <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  const float* src = nullptr;
  if (lInput > 1) {  // Device<T>::AllocMemory, device.cu:854-899
    if (!pf) return ERROR_PARAM_NULL;
    if (lInput == count + 1) src = pf + 1;
    else if (lInput == count + 2) src = pf + 2;
    else return ERROR_PARAM_OUT_OF_RANGE;
  }
  MemItem m;
  m.count = count;
  m.bf16 = bf16;
  cudaError_t ce = cudaMalloc(&m.ptr, m.bytes());
  if (ce != cudaSuccess) { cudaGetLastError(); return ce == cudaErrorMemoryAllocation ? ERROR_MEMORY_OUT : (long)ce; }
  if (src) {
    if (!bf16) {
      if ((ce = cudaMemcpy(m.ptr, src, m.bytes(), cudaMemcpyHostToDevice)) != cudaSuccess) { cudaFree(m.ptr); return ce; }
    } else {
      float* tmp = nullptr;
      if ((ce = cudaMalloc(&tmp, count * 4)) != cudaSuccess) { cudaFree(m.ptr); return ce; }
      cudaMemcpy(tmp, src, count * 4, cudaMemcpyHostToDevice);
      mca_convert_f32_to_bf16(tmp, m.ptr, count, 0);
      cudaStreamSynchronize(0);
      cudaFree(tmp);
    }
  } else {
    cudaMemsetAsync(m.ptr, 0, m.bytes(), 0);
  }
  const long h = k->next_handle++;
  k->mem[h] = m;
  return set_out((float)h, plOutput, ppOutput);
}

long free_mem(Kernel* k, long llInput, MCA_LONGLONG* pl) {
  long e;
  if ((e = verify_in(llInput, pl, 1, 1))) return e;
  auto it = k->mem.find((long)pl[0]);
  if (it == k->mem.end()) return ERROR_MEMORY_NOT_FOUND;
  cudaFree(it->second.ptr);
  k->mem.erase(it);
  return 0;
}

long alloc_host(Kernel* k, int64_t count, float** dst) {
  cudaError_t ce = cudaMallocHost((void**)dst, (size_t)count * sizeof(float));
  if (ce != cudaSuccess) { cudaGetLastError(); return ERROR_MEMORY_OUT; }
  k->host_bufs.push_back(*dst);
  return 0;
}

long copy_to_host(Kernel* k, const MemItem* m, int64_t count, float* dst) {
  if (!m->bf16) return (long)cudaMemcpy(dst, m->ptr, (size_t)count * 4, cudaMemcpyDeviceToHost);
  float* tmp = k->staging((size_t)count);
  if (!tmp) return ERROR_MEMORY_OUT;
  long e = mca_convert_bf16_to_f32(m->ptr, tmp, count, 0);
  if (!e) e = (long)cudaMemcpy(dst, tmp, (size_t)count * 4, cudaMemcpyDeviceToHost);
  return e;
}

long get_mem(Kernel* k, long llInput, MCA_LONGLONG* pl, MCA_LONG* plOutput, float** ppOutput) {
  long e;  // Device<T>::GetMemory, device.cu:973-1026
  if ((e = verify_in(llInput, pl, 1, 2))) return e;
  if ((e = verify_out(plOutput, ppOutput))) return e;
  MemItem* m = k->get((long)pl[0]);
  if (!m) return ERROR_MEMORY_NOT_FOUND;
  int64_t count = llInput > 1 ? pl[1] : 0;
  if (llInput <= 1 || count < 0) count = m->count;
  else if (count > m->count) return ERROR_PARAM_OUT_OF_RANGE;
  if (count > 0x7fffffffLL) return ERROR_PARAM_OUT_OF_RANGE;
  if (count <= *plOutput) {
    if ((e = copy_to_host(k, m, count, *ppOutput))) return e;
  } else {
    float* buf = nullptr;
    if ((e = alloc_host(k, count, &buf))) return e;
    if ((e = copy_to_host(k, m, count, buf))) return e;
    *ppOutput = buf;
  }
  *plOutput = (MCA_LONG)count;
  return 0;
}

long set_mem(Kernel* k, long lInput, float* pf, long llInput, MCA_LONGLONG* pl) {
  long e;  // Device<T>::SetMemory, device.cu:1029-1100
  if ((e = verify_in(lInput, pf, 2, 0x7fffffff))) return e;
  if ((e = verify_in(llInput, pl, 2, 2))) return e;
  MemItem* m = k->get((long)pl[0]);
  if (!m) return ERROR_MEMORY_NOT_FOUND;
  const int64_t count = pl[1];
  const float* data;
  if (count == lInput - 2) data = pf + 2;
  else if (count == lInput - 3) data = pf + 3;
  else return ERROR_PARAM_OUT_OF_RANGE;
  if (count > m->count) return ERROR_MEMORY_RANGE_EXCEEDED;
  if (!m->bf16) return (long)cudaMemcpy(m->ptr, data, (size_t)count * 4, cudaMemcpyHostToDevice);
  float* tmp = k->staging((size_t)count);
  if (!tmp) return ERROR_MEMORY_OUT;
  cudaError_t ce = cudaMemcpy(tmp, data, (size_t)count * 4, cudaMemcpyHostToDevice);
  if (ce != cudaSuccess) return ce;
  e = mca_convert_f32_to_bf16(tmp, m->ptr, count, 0);
  if (!e) e = (long)cudaStreamSynchronize(0);
  return e;
}

long convert_mem(Kernel* k, long llInput, MCA_LONGLONG* pl) {
  long e;
  if ((e = verify_in(llInput, pl, 3, 3))) return e;
  MemItem *s = k->get((long)pl[0]), *d = k->get((long)pl[1]);
  if (!s || !d) return ERROR_MEMORY_NOT_FOUND;
  const int64_t n = pl[2];
  if (n <= 0 || n > s->count || n > d->count) return ERROR_PARAM_OUT_OF_RANGE;
  if (s->bf16 == d->bf16) return (long)cudaMemcpyAsync(d->ptr, s->ptr, (size_t)n * (s->bf16 ? 2 : 4), cudaMemcpyDeviceToDevice, 0);
  if (d->bf16) return mca_convert_f32_to_bf16((const float*)s->ptr, d->ptr, n, 0);
  return mca_convert_bf16_to_f32(s->ptr, (float*)d->ptr, n, 0);
}

// ---- attention ids ------------------------------------------------------------------------

long attn_set(Kernel* k, long lInput, float* pf, long llInput, MCA_LONGLONG* pl) {
  long e;  // Device<T>::SetAttn, device.h:2463-2486 (exactly 9 longs there; 10th/11th are extensions)
  if ((e = verify_in(llInput, pl, 9, 11))) return e;
  if ((e = verify_in(lInput, pf, 1, 1))) return e;
  auto it = k->attn.find((long)pl[1]);
  if (it == k->attn.end()) return ERROR_ATTN_NOT_INITIALIZED;
  AttnHandle& a = it->second;
  a.release();  // attnHandle<T>::Set starts with CleanUp(), attn.cu:412
  a.training = pl[3] != 0;
  a.B = (int)pl[4]; a.block = (int)pl[5]; a.H = (int)pl[6]; a.D = (int)pl[7];
  a.dropout = pf[0];
  a.dtype = llInput > 9 ? (int)pl[9] : MCA_DTYPE_F32;
  a.flags = llInput > 10 ? (int)pl[10] : 0;
  if (a.B <= 0 || a.block <= 0 || a.H <= 0 || a.D <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (a.dtype < MCA_DTYPE_F32 || a.dtype > MCA_DTYPE_BF16) return ERROR_PARAM_OUT_OF_RANGE;
  if (a.D > 128) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  if (a.dtype == MCA_DTYPE_BF16 && a.D != 64 && a.D != 128) return ERROR_ATTN_UNSUPPORTED_SHAPE;   // no bf16 kernel for other head sizes
  const size_t rows = (size_t)a.B * a.H * a.block;
  cudaError_t ce;
  if ((ce = cudaMalloc(&a.causal_flag, 8 * sizeof(int))) != cudaSuccess) { a.release(); return ERROR_MEMORY_OUT; }
  cudaMemsetAsync(a.causal_flag, 0, 8 * sizeof(int), 0);
  if ((ce = cudaMalloc(&a.lse, rows * 4)) != cudaSuccess) { a.release(); return ERROR_MEMORY_OUT; }
  if (a.training) {
    // What Backward needs from Forward: the softmax row statistics and the output.  The
    // reference keeps (B,H,T,T) probabilities instead (attn.cu:436-452).
    if (cudaMalloc(&a.row_max, rows * 4) != cudaSuccess || cudaMalloc(&a.row_sum, rows * 4) != cudaSuccess ||
        cudaMalloc(&a.delta, rows * 4) != cudaSuccess || cudaMalloc(&a.y_copy, rows * a.D * 4) != cudaSuccess) {
      cudaGetLastError();
      a.release();
      return ERROR_MEMORY_OUT;
    }
  }
  if ((a.dtype == MCA_DTYPE_F32 || a.dtype == MCA_DTYPE_TF32) && !(a.flags & MCA_FLAG_EXACT_FP32) && mca_sdpa_forward_f32_tc_supported(a.D) &&
      (int64_t)a.B * a.H <= 65535) {
    // fp32 callers get the tensor-core forward: room for the fp16 halves of q, k, v.  If it cannot be had the handle
    // simply keeps to the CUDA-core kernels.
    a.split_ws_bytes = mca_sdpa_forward_f32_tc_workspace_bytes_d(a.B, a.H, a.block, a.D);
    if (cudaMalloc(&a.split_ws, (size_t)a.split_ws_bytes) != cudaSuccess) { cudaGetLastError(); a.split_ws = nullptr; a.split_ws_bytes = 0; }
  }
  a.configured = true;
  return 0;
}

// Decide how the mask of this call is applied.  A (T,T) mask is classified on every call (one pass over
// T*T floats, small next to the attention itself): the caller may have rewritten the handle with SETMEM, or
// freed it and been given the same address again, so nothing about it is remembered between calls.
constexpr long kMaskClassMiss = -7001;   // internal: the class assumed for this call's kernels was wrong

long resolve_mask(Kernel* k, AttnHandle& a, long hMask, bool batch_mask, int T, const float** mask, int* mode,
                  bool need_host_answer, bool may_speculate = false) {
  *mask = nullptr;
  if (a.flags & MCA_FLAG_CAUSAL_IMPLICIT) { *mode = MCA_MASK_CAUSAL; return 0; }
  if (hMask == 0) { *mode = MCA_MASK_NONE; return 0; }
  float* m = nullptr;
  long e = check_f32(k, hMask, batch_mask ? (int64_t)a.B * T : (int64_t)T * T, &m);
  if (e) return e;
  *mask = m;
  if (batch_mask) { *mode = MCA_MASK_BATCH; return 0; }
  *mode = MCA_MASK_TT;
  if ((e = mca_classify_causal_mask_ws(m, T, a.causal_flag, a.causal_flag + 6, 0))) return e;
  if (need_host_answer && may_speculate && !k->async && a.spec_allowed && a.spec_class >= 0) {
    a.spec_pending = true;
    a.spec_assumed = a.spec_class;
    if (a.spec_class == 1) *mode = MCA_MASK_CAUSAL;
    return 0;
  }
  if (need_host_answer) {
    // into pinned memory on the stream, then one stream synchronisation: a third of the latency of a blocking copy
    // into pageable memory
    if (k->answer_words() == nullptr) return ERROR_MEMORY_OUT;
    cudaError_t ce = cudaMemcpyAsync(k->h_answer, a.causal_flag, sizeof(int), cudaMemcpyDeviceToHost, 0);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(0);
    if (ce != cudaSuccess) return ce;
    if (*k->h_answer == 1) *mode = MCA_MASK_CAUSAL;
    a.spec_class = *k->h_answer == 1 ? 1 : 0;
  }
  return 0;
}

// Keep-bits of this call's (T,T) or batch mask, packed into buffers the handle owns (room for the configured block
// size, allocated on first use).  The backward of the same handle reads what the forward packed.
long pack_mask_bits(AttnHandle& a, const float* mask, int mode, int T) {
  const size_t rows = (size_t)std::max(a.block, a.B);
  const size_t need = rows * (size_t)mca_mask_bits_row_words(a.block);
  if (a.mask_bits == nullptr || a.mask_bits_words < need) {
    cudaFree(a.mask_bits); cudaFree(a.mask_bits_t);
    a.mask_bits = a.mask_bits_t = nullptr; a.mask_bits_words = 0;
    if (cudaMalloc(&a.mask_bits, need * 4) != cudaSuccess || cudaMalloc(&a.mask_bits_t, need * 4) != cudaSuccess) {
      cudaGetLastError(); cudaFree(a.mask_bits); a.mask_bits = nullptr;
      return ERROR_MEMORY_OUT;
    }
    a.mask_bits_words = need;
  }
  return mca_mask_pack(mask, mode, a.B, T, a.mask_bits, a.mask_bits_t, 0);
}

// fp32 room for a bf16 handle whose mask the tensor-core kernels do not apply: q, k, v, y (and, for training handles,
// the three gradients and dY), at the configured block size.
long ensure_mask_ws(AttnHandle& a) {
  const size_t n = (size_t)a.B * a.H * a.block * a.D;
  const size_t need = (a.training ? 8 : 4) * n;
  if (a.mask_ws != nullptr && a.mask_ws_floats >= need) return 0;
  cudaFree(a.mask_ws);
  a.mask_ws = nullptr; a.mask_ws_floats = 0;
  if (cudaMalloc(&a.mask_ws, need * sizeof(float)) != cudaSuccess) { cudaGetLastError(); a.mask_ws = nullptr; return ERROR_MEMORY_OUT; }
  a.mask_ws_floats = need;
  return 0;
}

// Read the status words a tensor-core kernel writes when one of its bounded waits gives up.  Blocking: in
// synchronous mode it follows every tensor-core launch; in asynchronous mode the words are read for every
// attention handle at the next call that synchronises (CUDA_FN_SYNCHRONIZEDEVICE).
long read_status(Kernel* k, AttnHandle& a) {
  if (!a.causal_flag) return 0;
  // into pinned words on the stream, then one stream synchronisation (a blocking copy into pageable memory takes
  // several microseconds longer, on every call of the synchronous mode)
  if (k->answer_words() == nullptr) return ERROR_MEMORY_OUT;
  int* w = k->h_answer + 2;
  cudaError_t ce = cudaMemcpyAsync(w, a.causal_flag, 5 * sizeof(int), cudaMemcpyDeviceToHost, 0);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(0);
  if (ce != cudaSuccess) return ce;
  const int* st = w + 1;
  if (a.spec_pending) {   // the class this call's kernels were chosen on, against what its classification found
    a.spec_pending = false;
    const int actual = w[0] == 1 ? 1 : 0;
    const bool matters = a.spec_assumed == 1 && actual == 0;   // the other way round the result is right, only slower
    a.spec_class = actual;
    if (matters && st[0] == 0) return kMaskClassMiss;
  }
  if (st[0] != 0) {
    char buf[96];
    snprintf(buf, sizeof(buf), "status %d at stage %d block %d iter %d", st[0], st[1], st[2], st[3]);
    k->last_detail = buf;
    cudaMemset(a.causal_flag + 1, 0, 4 * sizeof(int));   // the next launch starts clean
    a.have_fwd = false;                                   // whatever that launch left behind is not a result
    return ERROR_ATTN_KERNEL_TIMEOUT;
  }
  return 0;
}
long tc_status(Kernel* k, AttnHandle& a) {
  if (k->async) { a.status_pending = true; return 0; }
  return read_status(k, a);
}
long sync_and_collect_status(Kernel* k) {
  cudaError_t ce = cudaStreamSynchronize(0);
  if (ce != cudaSuccess) return ce;
  long first = 0;
  for (auto& kv : k->attn) {
    if (!kv.second.status_pending) continue;
    kv.second.status_pending = false;
    const long e = read_status(k, kv.second);
    if (e && !first) first = e;
  }
  return first;
}

void remember_forward(AttnHandle& a, int T, int mode, int layout, long hMask, bool batch_mask) {
  a.have_fwd = true; a.fwd_T = T; a.fwd_mask_mode = mode; a.fwd_layout = layout;
  a.fwd_split = false;
  const bool reads_mask = mode == MCA_MASK_TT || mode == MCA_MASK_BATCH;
  a.fwd_mask_handle = reads_mask ? hMask : 0;
  a.fwd_batch_mask = batch_mask;
}

// layout MCA_LAYOUT_PACKED: pl[3..5] all name the (B,T,3C) projection output and pl[7] a (B,T,C) tensor
long attn_fwd_once(Kernel* k, long llInput, MCA_LONGLONG* pl, int layout);

long attn_fwd(Kernel* k, long llInput, MCA_LONGLONG* pl, int layout) {
  long e = attn_fwd_once(k, llInput, pl, layout);
  if (e != kMaskClassMiss) return e;
  AttnHandle& a = k->attn.find((long)pl[1])->second;   // the handle exists: the first pass ran its kernels
  a.spec_allowed = false;                              // this time the class is read before the kernels are chosen
  e = attn_fwd_once(k, llInput, pl, layout);
  a.spec_allowed = true;
  return e;
}

long attn_fwd_once(Kernel* k, long llInput, MCA_LONGLONG* pl, int layout) {
  long e;  // Device<T>::AttnForward, device.h:2488-2506; attnHandle<T>::Forward, attn.cu:518-602
  if ((e = verify_in(llInput, pl, 9, 9))) return e;
  auto it = k->attn.find((long)pl[1]);
  if (it == k->attn.end() || !it->second.configured) return ERROR_ATTN_NOT_INITIALIZED;
  AttnHandle& a = it->second;
  a.spec_pending = false;
  const int T = (int)pl[2];
  if (T > a.block) return ERROR_ATTN_INVALID_BLOCK_SIZE;  // attn.cu:530-531
  if (T <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (a.training && a.dropout > 0.f) return ERROR_ATTN + 3;  // the reference's guard always fails here (attn.cu:265)
  const int64_t n = (int64_t)a.B * a.H * T * a.D;
  const bool packed = layout == MCA_LAYOUT_PACKED;
  const int64_t n_in = packed ? 3 * n : n;               // elements the q / k / v handles must hold
  const int64_t C = (int64_t)a.H * a.D;                  // k and v start C and 2C elements into a packed row
  const bool batch_mask = pl[8] != 0;
  const float* mask = nullptr;
  int mode = 0;
  a.have_fwd = false;
  // A tf32 handle asks for single-pass tf32 products, which exist for inference at head size 64 with a causal mask or
  // none.  Everything else it is given -- training, other head sizes, other masks -- goes the way of an fp32 handle:
  // the split-operand tensor-core kernels where they apply (more accurate than tf32, forward and backward), else the
  // exact fp32 kernels.
  bool fp32_path = a.dtype == MCA_DTYPE_F32 || (a.dtype == MCA_DTYPE_TF32 && (a.training || a.D != 64));
  if (a.dtype == MCA_DTYPE_TF32 && !fp32_path) {
    if ((e = resolve_mask(k, a, (long)pl[6], batch_mask, T, &mask, &mode, true))) return e;
    fp32_path = mode == MCA_MASK_TT || mode == MCA_MASK_BATCH;
  }
  if (fp32_path) {
    float *q, *kk, *v, *y;
    if ((e = check_f32(k, (long)pl[3], n_in, &q)) || (e = check_f32(k, (long)pl[4], n_in, &kk)) ||
        (e = check_f32(k, (long)pl[5], n_in, &v)) || (e = check_f32(k, (long)pl[7], n, &y)))
      return e;
    if (packed) { kk += C; v += 2 * C; }
    const bool split_path = a.split_ws != nullptr && (mca_sdpa_backward_f32_tc_supported(a.D) != 0 || !a.training);
    if ((e = resolve_mask(k, a, (long)pl[6], batch_mask, T, &mask, &mode, a.split_ws != nullptr, split_path))) return e;
    const bool save = a.training && T == a.block;
    const bool bits = mode == MCA_MASK_TT || mode == MCA_MASK_BATCH;   // packed for the kernel; causal / none need nothing
    // Head sizes with a tensor-core forward but no tensor-core backward (128): the forward leaves the row statistics
    // the exact fp32 backward recomputes the probabilities from; a saved forward under a general or batch mask keeps
    // to the exact kernels, whose masked-row convention that backward shares.
    const bool tc_bwd = mca_sdpa_backward_f32_tc_supported(a.D) != 0;
    if (a.split_ws != nullptr && (tc_bwd || !save || !bits)) {
      if (bits && (e = pack_mask_bits(a, mask, mode, T))) return e;
      const bool stats = save && !tc_bwd;
      e = mca_sdpa_forward_f32_tc_masked(q, kk, v, mode == MCA_MASK_CAUSAL, a.B, a.H, T, a.D, y, stats ? a.row_max : nullptr,
                                         stats ? a.row_sum : nullptr, save ? a.y_copy : nullptr, save && tc_bwd ? a.lse : nullptr,
                                         a.split_ws, a.split_ws_bytes, a.causal_flag + 1, layout, bits ? a.mask_bits : nullptr,
                                         bits ? mode : MCA_MASK_NONE, 0);
      if (e) return e;
      if (save) { remember_forward(a, T, mode, layout, 0, false); a.fwd_split = tc_bwd; }
      return tc_status(k, a);
    }
    e = mca_sdpa_forward_f32_layout(q, kk, v, mask, mode, a.causal_flag, a.B, a.H, T, a.D, y, save ? a.row_max : nullptr,
                                    save ? a.row_sum : nullptr, save ? a.y_copy : nullptr, layout, 0);
    if (!e && save) remember_forward(a, T, mode, layout, (long)pl[6], batch_mask);
    return e;
  }
  // bf16, or single-pass tf32 (inference, head size 64, causal mask or none)
  const bool bf16 = a.dtype == MCA_DTYPE_BF16;
  if (a.dtype == MCA_DTYPE_TF32) {
    // classified above, and the class is known on the host
  } else if ((e = resolve_mask(k, a, (long)pl[6], batch_mask, T, &mask, &mode, true, bf16 && !(a.flags & MCA_FLAG_EXACT_FP32)))) {
    return e;
  }
  void *q, *kk, *v, *y;
  if ((e = check_any(k, (long)pl[3], n_in, bf16, &q)) || (e = check_any(k, (long)pl[4], n_in, bf16, &kk)) ||
      (e = check_any(k, (long)pl[5], n_in, bf16, &v)) || (e = check_any(k, (long)pl[7], n, bf16, &y)))
    return e;
  if (packed) {
    const size_t esz = bf16 ? 2 : 4;
    kk = static_cast<char*>(kk) + C * esz;
    v = static_cast<char*>(v) + 2 * C * esz;
  }
  if (bf16 && (mode == MCA_MASK_TT || mode == MCA_MASK_BATCH) && !(a.flags & MCA_FLAG_EXACT_FP32)) {
    // a general or batch mask: packed into keep-bits, applied by the same tensor-core kernel
    if ((e = pack_mask_bits(a, mask, mode, T))) return e;
    const bool keep = a.training && T == a.block;   // Backward needs O: the kernel writes the handle's copy itself
    e = mca_sdpa_forward_tc_keep(q, kk, v, MCA_DTYPE_BF16, 0, a.B, a.H, T, a.D, y, keep ? a.y_copy : nullptr, a.lse,
                                 a.causal_flag + 1, layout, a.mask_bits, mode, 0);
    if (e) return e;
    if (keep) remember_forward(a, T, mode, layout, 0, false);
    return tc_status(k, a);
  }
  if (bf16 && (mode == MCA_MASK_TT || mode == MCA_MASK_BATCH)) {
    // MCA_FLAG_EXACT_FP32 on a bf16 handle with such a mask: the exact fp32 kernels on fp32 copies of its tensors
    // (same mask semantics: -1e29 logits, a uniform fully-masked row).
    if ((e = ensure_mask_ws(a))) return e;
    float* w = a.mask_ws;
    float *qf = w, *kf = packed ? w + C : w + n, *vf = packed ? w + 2 * C : w + 2 * n, *yf = w + 3 * n;
    if (packed) e = mca_convert_bf16_to_f32(q, w, 3 * n, 0);   // pl[3..5] name one (B,T,3C) tensor
    else if (!(e = mca_convert_bf16_to_f32(q, qf, n, 0)) && !(e = mca_convert_bf16_to_f32(kk, kf, n, 0)))
      e = mca_convert_bf16_to_f32(v, vf, n, 0);
    if (e) return e;
    const bool save = a.training && T == a.block;
    e = mca_sdpa_forward_f32_layout(qf, kf, vf, mask, mode, a.causal_flag, a.B, a.H, T, a.D, yf, save ? a.row_max : nullptr,
                                    save ? a.row_sum : nullptr, save ? a.y_copy : nullptr, layout, 0);
    if (e) return e;
    if ((e = mca_convert_f32_to_bf16(yf, y, n, 0))) return e;
    if (save) remember_forward(a, T, mode, layout, (long)pl[6], batch_mask);
    return 0;
  }
  // Backward needs O and the log-sum-exp of this Forward; it cannot trust the data of hY.  The handle's copy keeps the
  // layout y was written in and is one more destination of the kernel's epilogue.
  const bool keep = a.training && T == a.block && bf16;
  e = mca_sdpa_forward_tc_keep(q, kk, v, a.dtype, mode == MCA_MASK_CAUSAL, a.B, a.H, T, a.D, y, keep ? a.y_copy : nullptr, a.lse,
                               a.causal_flag + 1, layout, nullptr, MCA_MASK_NONE, 0);
  if (e) return e;
  if (keep) remember_forward(a, T, mode, layout, 0, false);
  return tc_status(k, a);
}

// layout MCA_LAYOUT_PACKED: pl[2,4,6] name the (B,T,3C) projection output, pl[3,5,7] its gradient, pl[10] a (B,T,C) gradient
long attn_bwd(Kernel* k, long llInput, MCA_LONGLONG* pl, int layout) {
  long e;  // Device<T>::AttnBackward, device.h:2508-2529; attnHandle<T>::Backward, attn.cu:608-661
  if ((e = verify_in(llInput, pl, 11, 11))) return e;
  auto it = k->attn.find((long)pl[1]);
  if (it == k->attn.end() || !it->second.configured) return ERROR_ATTN_NOT_INITIALIZED;
  AttnHandle& a = it->second;
  // The reference's Backward always works at the configured block size on the tensors its
  // Forward left in the handle (attn.cu:622-634); it reads neither hMask nor the data of hY.
  if (!a.have_fwd || a.fwd_T != a.block || a.fwd_layout != layout) return ERROR_ATTN_BACKWARD_WITHOUT_FORWARD;
  // The kernels that write dQ and those that write dK, dV run side by side, each reading q, k, v and dY: a gradient
  // handle that names an input's memory (a blob's diff and data never do) is refused instead of corrupting them.
  for (int g : {3, 5, 7})
    for (int i : {2, 4, 6, 10})
      if (pl[g] != 0 && pl[g] == pl[i]) return ERROR_PARAM_OUT_OF_RANGE;
  const int T = a.block;
  const int64_t n = (int64_t)a.B * a.H * T * a.D;
  const bool packed = layout == MCA_LAYOUT_PACKED;
  const int64_t n_in = packed ? 3 * n : n;
  const int64_t C = (int64_t)a.H * a.D;
  if (a.dtype == MCA_DTYPE_BF16) {
    void *q, *dq, *kk, *dk, *v, *dv, *dy;
    if ((e = check_any(k, (long)pl[2], n_in, true, &q)) || (e = check_any(k, (long)pl[3], n_in, true, &dq)) ||
        (e = check_any(k, (long)pl[4], n_in, true, &kk)) || (e = check_any(k, (long)pl[5], n_in, true, &dk)) ||
        (e = check_any(k, (long)pl[6], n_in, true, &v)) || (e = check_any(k, (long)pl[7], n_in, true, &dv)) ||
        (e = check_any(k, (long)pl[10], n, true, &dy)))
      return e;
    if (packed) {
      kk = static_cast<char*>(kk) + C * 2; dk = static_cast<char*>(dk) + C * 2;
      v = static_cast<char*>(v) + 2 * C * 2; dv = static_cast<char*>(dv) + 2 * C * 2;
    }
    const bool fwd_masked = a.fwd_mask_mode == MCA_MASK_TT || a.fwd_mask_mode == MCA_MASK_BATCH;
    if (fwd_masked && a.fwd_mask_handle == 0) {
      // the forward applied the mask on the tensor cores from the keep-bits it packed into the handle: so does this
      e = mca_sdpa_backward_tc_masked(q, kk, v, a.y_copy, dy, a.lse, a.delta, MCA_DTYPE_BF16, 0, a.B, a.H, T, a.D, dq, dk, dv,
                                      a.causal_flag + 1, layout, a.mask_bits, a.mask_bits_t, a.fwd_mask_mode, 0);
      if (e) return e;
      return tc_status(k, a);
    }
    if (fwd_masked) {
      // the forward ran the exact fp32 kernels on fp32 copies (MCA_FLAG_EXACT_FP32): so does this; the mask is looked
      // up again by the handle the forward was given
      const float* mask = nullptr;
      int mode = a.fwd_mask_mode;
      if ((e = resolve_mask(k, a, a.fwd_mask_handle, a.fwd_batch_mask, T, &mask, &mode, false))) return e;
      if ((e = ensure_mask_ws(a))) return e;
      float* w = a.mask_ws;
      float *qf = w, *kf = packed ? w + C : w + n, *vf = packed ? w + 2 * C : w + 2 * n;
      float *gq = w + 4 * n, *gk = packed ? gq + C : gq + n, *gv = packed ? gq + 2 * C : gq + 2 * n, *dyf = w + 7 * n;
      if (packed) e = mca_convert_bf16_to_f32(q, w, 3 * n, 0);
      else if (!(e = mca_convert_bf16_to_f32(q, qf, n, 0)) && !(e = mca_convert_bf16_to_f32(kk, kf, n, 0)))
        e = mca_convert_bf16_to_f32(v, vf, n, 0);
      if (e || (e = mca_convert_bf16_to_f32(dy, dyf, n, 0))) return e;
      e = mca_sdpa_backward_f32_layout(qf, kf, vf, dyf, a.y_copy, mask, a.fwd_mask_mode, a.causal_flag, a.row_max, a.row_sum,
                                       a.delta, a.B, a.H, T, a.D, gq, gk, gv, layout, 0);
      if (e) return e;
      if (packed) return mca_convert_f32_to_bf16(gq, dq, 3 * n, 0);
      if ((e = mca_convert_f32_to_bf16(gq, dq, n, 0)) || (e = mca_convert_f32_to_bf16(gk, dk, n, 0))) return e;
      return mca_convert_f32_to_bf16(gv, dv, n, 0);
    }
    e = mca_sdpa_backward_tc_layout(q, kk, v, a.y_copy, dy, a.lse, a.delta, MCA_DTYPE_BF16,
                                    a.fwd_mask_mode == MCA_MASK_CAUSAL, a.B, a.H, T, a.D, dq, dk, dv, a.causal_flag + 1,
                                    layout, 0);
    if (e) return e;
    return tc_status(k, a);
  }
  float *q, *dq, *kk, *dk, *v, *dv, *dy;
  if ((e = check_f32(k, (long)pl[2], n_in, &q)) || (e = check_f32(k, (long)pl[3], n_in, &dq)) ||
      (e = check_f32(k, (long)pl[4], n_in, &kk)) || (e = check_f32(k, (long)pl[5], n_in, &dk)) ||
      (e = check_f32(k, (long)pl[6], n_in, &v)) || (e = check_f32(k, (long)pl[7], n_in, &dv)) ||
      (e = check_f32(k, (long)pl[10], n, &dy)))
    return e;
  if (packed) { kk += C; dk += C; v += 2 * C; dv += 2 * C; }
  if (a.fwd_split) {
    // the forward ran on the tensor cores with split operands; so does the backward, from the halves of q, k, v that
    // forward left in the handle's workspace (the reference's Backward likewise works on what its Forward saved)
    const bool bits = a.fwd_mask_mode == MCA_MASK_TT || a.fwd_mask_mode == MCA_MASK_BATCH;   // packed by the forward
    e = mca_sdpa_backward_f32_tc_masked(dy, a.y_copy, a.lse, a.delta, a.fwd_mask_mode == MCA_MASK_CAUSAL, a.B, a.H, T, a.D, dq, dk,
                                        dv, a.split_ws, a.split_ws_bytes, a.causal_flag + 1, layout, bits ? a.mask_bits : nullptr,
                                        bits ? a.mask_bits_t : nullptr, bits ? a.fwd_mask_mode : MCA_MASK_NONE, 0);
    if (e) return e;
    return tc_status(k, a);
  }
  // The probabilities are recomputed, so the forward's mask is applied again: it is looked up by the handle
  // the forward was given (a freed handle is an error, not a dangling pointer) and classified afresh.
  const float* mask = nullptr;
  int mode = a.fwd_mask_mode;
  if (a.fwd_mask_handle != 0) {
    if ((e = resolve_mask(k, a, a.fwd_mask_handle, a.fwd_batch_mask, T, &mask, &mode, false))) return e;
  }
  return mca_sdpa_backward_f32_layout(q, kk, v, dy, a.y_copy, mask, mode, a.causal_flag, a.row_max, a.row_sum, a.delta,
                                      a.B, a.H, T, a.D, dq, dk, dv, layout, 0);
}

// ---- rope ids ------------------------------------------------------------------------------

long rope_create(Kernel* k, long lInput, float* pf, long llInput, MCA_LONGLONG* pl, MCA_LONG* plOutput,
                 float** ppOutput) {
  long e;  // Device<T>::CreateRope, device.h:4200-4228
  if ((e = verify_in(lInput, pf, 1, 1))) return e;
  if ((e = verify_in(llInput, pl, 7, 7))) return e;
  if ((e = verify_out(plOutput, ppOutput))) return e;
  const int shared = (int)pl[0];
  if (shared > 0) {  // Memory<T>::CreateRope with a shared index returns the existing handle, memory.h:2182-2226
    for (auto& kv : k->rope)
      if (kv.second.shared_index == shared) { kv.second.refs++; return set_out((float)kv.first, plOutput, ppOutput); }
  }
  RopeHandle r;
  r.shared_index = shared;
  r.B = (int)pl[3]; r.T = (int)pl[4]; r.H = (int)pl[5]; r.D = (int)pl[6];
  if (r.T <= 0 || r.H <= 0 || r.D <= 0 || (r.D & 1)) return ERROR_PARAM_OUT_OF_RANGE;
  const size_t n = (size_t)r.T * (r.D / 2);
  std::vector<float> c(n), s(n);
  mca_rope_tables_host(r.T, r.D, pf[0], c.data(), s.data());
  if (cudaMalloc(&r.cos_t, n * 4) != cudaSuccess || cudaMalloc(&r.sin_t, n * 4) != cudaSuccess) {
    cudaGetLastError(); cudaFree(r.cos_t); return ERROR_MEMORY_OUT;
  }
  cudaMemcpy(r.cos_t, c.data(), n * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(r.sin_t, s.data(), n * 4, cudaMemcpyHostToDevice);
  const long h = k->next_handle++;
  k->rope[h] = r;
  return set_out((float)h, plOutput, ppOutput);
}

long rope_free(Kernel* k, long lInput, float* pf) {
  long e;
  if ((e = verify_in(lInput, pf, 1, 1))) return e;
  auto it = k->rope.find((long)pf[0]);
  if (it == k->rope.end()) return ERROR_ROPE_NOT_INITIALIZED;
  if (--it->second.refs > 0) return 0;
  cudaFree(it->second.cos_t); cudaFree(it->second.sin_t);
  k->rope.erase(it);
  return 0;
}

long rope_run(Kernel* k, long llInput, MCA_LONGLONG* pl, bool backward) {
  long e;  // Device<T>::RopeForward / RopeBackward, device.h:4243-4283
  if (!backward) { if ((e = verify_in(llInput, pl, 4, 5))) return e; }
  else { if ((e = verify_in(llInput, pl, 5, 5))) return e; }
  auto it = k->rope.find((long)pl[0]);
  if (it == k->rope.end()) return ERROR_ROPE_NOT_INITIALIZED;
  RopeHandle& r = it->second;
  const int64_t n = pl[1];
  float *x, *y;
  int off = -1;
  if (!backward) {
    if ((e = check_f32(k, (long)pl[2], n, &x)) || (e = check_f32(k, (long)pl[3], n, &y))) return e;
    if (llInput > 4) off = (int)pl[4];
  } else {  // longs {hRope,n,hX,hYdiff,hXdiff}: rotate hYdiff by -angle into hXdiff (rope.cu:828-864)
    if ((e = check_f32(k, (long)pl[3], n, &x)) || (e = check_f32(k, (long)pl[4], n, &y))) return e;
  }
  // positions beyond the table would read out of bounds in the reference; refuse instead
  const int64_t half = r.D / 2, full = half * r.H;
  const int64_t last_pos = std::min<int64_t>(n / 2 - 1, (int64_t)r.T * full - 1) / full;
  if ((off > 0 ? off : 0) + (last_pos + 1) * half > (int64_t)r.T * half) return ERROR_PARAM_OUT_OF_RANGE;
  return mca_rope_f32(x, y, n, r.T, r.H, r.D, r.cos_t, r.sin_t, off, backward ? 1 : 0, 0);
}

// ---- decode ids ----------------------------------------------------------------------------

long decode_create(Kernel* k, long lInput, float* pf, long llInput, MCA_LONGLONG* pl, MCA_LONG* plOutput,
                   float** ppOutput) {
  long e;
  if ((e = verify_in(lInput, pf, 1, 1))) return e;
  if ((e = verify_in(llInput, pl, 6, 6))) return e;
  if ((e = verify_out(plOutput, ppOutput))) return e;
  DecodeHandle d;
  d.B = (int)pl[0]; d.n_heads = (int)pl[1]; d.n_kv_heads = (int)pl[2]; d.hs = (int)pl[3]; d.seq_len = (int)pl[4];
  d.bf16 = pl[5] != 0;
  if (d.B <= 0 || d.n_heads <= 0 || d.n_kv_heads <= 0 || d.seq_len <= 0 || d.n_heads % d.n_kv_heads) return ERROR_PARAM_OUT_OF_RANGE;
  if (!mca_decode_head_size_supported(d.hs)) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  int sl, ns;
  if ((e = mca_decode_plan(d.B, d.n_heads, d.n_kv_heads, d.hs, d.seq_len, &sl, &ns, &d.scratch_floats))) return e;
  // the plan's split length grows with the work, so the longest plan bounds every shorter one
  int64_t worst = d.scratch_floats;
  for (int len = 128; len < d.seq_len; len *= 2) {
    int64_t need;
    mca_decode_plan(d.B, d.n_heads, d.n_kv_heads, d.hs, len, &sl, &ns, &need);
    worst = std::max(worst, need);
  }
  worst = std::max<int64_t>(worst, (int64_t)d.B * d.n_heads * ((d.seq_len + 127) / 128) * (d.hs + 2));
  d.scratch_floats = worst;
  const size_t n = (size_t)d.seq_len * (d.hs / 2);
  std::vector<float> c(n), s(n);
  if (pf[0] > 0.f) {
    mca_rope_tables_host(d.seq_len, d.hs, pf[0], c.data(), s.data());  // same table as precompute_freqs_cis
  } else {
    // theta <= 0: no rotation (cos 1, sin 0 reproduces q and k bit for bit).  This is the KV-cache step of
    // MultiheadAttentionLayer (MultiheadAttentionLayer.cs:713-777: append k, v at nPos, scores over 0..nPos,
    // softmax, times V) whose caches (nPos+1, heads, size) have the layout of one sequence here.
    std::fill(c.begin(), c.end(), 1.0f);
    std::fill(s.begin(), s.end(), 0.0f);
  }
  if (cudaMalloc(&d.fr, n * 4) != cudaSuccess || cudaMalloc(&d.fi, n * 4) != cudaSuccess ||
      cudaMalloc(&d.scratch, (size_t)d.scratch_floats * 4) != cudaSuccess) {
    cudaGetLastError(); cudaFree(d.fr); cudaFree(d.fi); return ERROR_MEMORY_OUT;
  }
  cudaMemcpy(d.fr, c.data(), n * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(d.fi, s.data(), n * 4, cudaMemcpyHostToDevice);
  const long h = k->next_handle++;
  k->decode[h] = d;
  return set_out((float)h, plOutput, ppOutput);
}

long decode_free(Kernel* k, long lInput, float* pf) {
  long e;
  if ((e = verify_in(lInput, pf, 1, 1))) return e;
  auto it = k->decode.find((long)pf[0]);
  if (it == k->decode.end()) return ERROR_PARAM_OUT_OF_RANGE;
  cudaFree(it->second.fr); cudaFree(it->second.fi); cudaFree(it->second.scratch);
  k->decode.erase(it);
  return 0;
}

long decode_step(Kernel* k, long llInput, MCA_LONGLONG* pl) {
  long e;
  if ((e = verify_in(llInput, pl, 9, 9))) return e;
  auto it = k->decode.find((long)pl[0]);
  if (it == k->decode.end()) return ERROR_PARAM_OUT_OF_RANGE;
  DecodeHandle& d = it->second;
  const int dim = d.n_heads * d.hs, kv_dim = d.n_kv_heads * d.hs;
  float *q, *kn = nullptr, *vn = nullptr, *out, *posf;
  void *kc, *vc;
  if ((e = check_f32(k, (long)pl[1], (int64_t)d.B * dim, &q))) return e;
  if (pl[2] != 0 || pl[3] != 0) {
    if ((e = check_f32(k, (long)pl[2], (int64_t)d.B * kv_dim, &kn)) || (e = check_f32(k, (long)pl[3], (int64_t)d.B * kv_dim, &vn))) return e;
  }
  const int64_t cache_n = (int64_t)d.B * d.seq_len * kv_dim;
  if ((e = check_any(k, (long)pl[4], cache_n, d.bf16, &kc)) || (e = check_any(k, (long)pl[5], cache_n, d.bf16, &vc))) return e;
  // positions travel in a memory handle holding int32 values (allocated as `count` 4-byte elements)
  if ((e = check_f32(k, (long)pl[6], d.B, &posf))) return e;
  if ((e = check_f32(k, (long)pl[8], (int64_t)d.B * dim, &out))) return e;
  const int max_len = (int)pl[7];
  if (max_len <= 0 || max_len > d.seq_len) return ERROR_PARAM_OUT_OF_RANGE;
  e = mca_decode_attention(q, kn, vn, kc, vc, d.bf16 ? 1 : 0, (int64_t)d.seq_len * kv_dim, (const int*)posf, d.B,
                           d.n_heads, d.n_kv_heads, d.hs, d.seq_len, max_len, d.fr, d.fi, d.scratch, d.scratch_floats, out, 0);
  if (e || k->async) return e;
  // synchronous mode: a position outside [0, maxLen) was refused on the device (that sequence's output is zero,
  // its cache untouched); report it instead of returning success
  cudaError_t ce = cudaStreamSynchronize(0);
  if (ce != cudaSuccess) return ce;
  int st[3] = {0, 0, 0};
  if ((e = mca_decode_status(st))) return e;
  if (st[0] != 0) {
    char buf[96];
    snprintf(buf, sizeof(buf), "%d sequence(s) with a position outside [0, %d): first is sequence %d at position %d", st[0],
             max_len, st[1], st[2]);
    k->last_detail = buf;
    return ERROR_PARAM_OUT_OF_RANGE;
  }
  return 0;
}

// Batches above eight sequences run the projections on the tensor cores; in synchronous mode a bounded wait that gave
// up inside that kernel is reported here instead of returning success.
long proj_result(Kernel* k, long e, long B) {
  if (e || k->async || B <= 8) return e;
  cudaError_t ce = cudaStreamSynchronize(0);
  if (ce != cudaSuccess) return ce;
  int st[4] = {0, 0, 0, 0};
  if ((e = mca_proj_tc_status(st))) return e;
  if (st[0] != 0) {
    char buf[96];
    snprintf(buf, sizeof(buf), "projection kernel: status %d at stage %d block %d iter %d", st[0], st[1], st[2], st[3]);
    k->last_detail = buf;
    return ERROR_ATTN_KERNEL_TIMEOUT;
  }
  return 0;
}

long decode_qkv(Kernel* k, long lInput, float* pf, long llInput, MCA_LONGLONG* pl) {
  long e;
  if ((e = verify_in(lInput, pf, 1, 1))) return e;
  if ((e = verify_in(llInput, pl, 11, 11))) return e;
  const int B = (int)pl[5], dim = (int)pl[6], kv_dim = (int)pl[7];
  if (B <= 0 || dim <= 0 || kv_dim <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  float *x, *rw, *q, *kk, *v;
  if ((e = check_f32(k, (long)pl[0], (int64_t)B * dim, &x)) || (e = check_f32(k, (long)pl[1], dim, &rw)) ||
      (e = check_f32(k, (long)pl[8], (int64_t)B * dim, &q)) || (e = check_f32(k, (long)pl[9], (int64_t)B * kv_dim, &kk)) ||
      (e = check_f32(k, (long)pl[10], (int64_t)B * kv_dim, &v)))
    return e;
  MemItem *wq = k->get((long)pl[2]), *wk = k->get((long)pl[3]), *wv = k->get((long)pl[4]);
  if (!wq || !wk || !wv) return ERROR_MEMORY_NOT_FOUND;
  if (wq->bf16 != wk->bf16 || wq->bf16 != wv->bf16) return ERROR_MEMORY_MIXED_HALF_TYPES;
  if (wq->count < (int64_t)dim * dim || wk->count < (int64_t)kv_dim * dim || wv->count < (int64_t)kv_dim * dim) return ERROR_MEMORY_TOO_SMALL;
  return proj_result(k, mca_decode_qkv_rmsnorm(x, rw, pf[0], wq->ptr, wk->ptr, wv->ptr, wq->bf16 ? 1 : 0, B, dim, kv_dim, q, kk, v, 0), B);
}

long decode_out(Kernel* k, long llInput, MCA_LONGLONG* pl) {
  long e;
  if ((e = verify_in(llInput, pl, 5, 5))) return e;
  const int B = (int)pl[2], dim = (int)pl[3];
  if (B <= 0 || dim <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  float *attn, *x;
  if ((e = check_f32(k, (long)pl[0], (int64_t)B * dim, &attn)) || (e = check_f32(k, (long)pl[4], (int64_t)B * dim, &x))) return e;
  MemItem* wo = k->get((long)pl[1]);
  if (!wo) return ERROR_MEMORY_NOT_FOUND;
  if (wo->count < (int64_t)dim * dim) return ERROR_MEMORY_TOO_SMALL;
  return proj_result(k, mca_decode_out_proj(attn, wo->ptr, wo->bf16 ? 1 : 0, B, dim, x, 0), B);
}

long decode_ffn(Kernel* k, long lInput, float* pf, long llInput, MCA_LONGLONG* pl) {
  long e;
  if ((e = verify_in(lInput, pf, 1, 1)) || (e = verify_in(llInput, pl, 9, 9))) return e;
  const int64_t B = pl[5], dim = pl[6], hidden = pl[7];
  if (B <= 0 || dim <= 0 || hidden <= 0 || B > INT32_MAX || dim > INT32_MAX || hidden > INT32_MAX) return ERROR_PARAM_OUT_OF_RANGE;
  float *x, *g, *h;
  if ((e = check_f32(k, (long)pl[0], B * dim, &x)) || (e = check_f32(k, (long)pl[1], dim, &g)) ||
      (e = check_f32(k, (long)pl[8], B * hidden, &h)))
    return e;
  MemItem *w1 = k->get((long)pl[2]), *w2 = k->get((long)pl[3]), *w3 = k->get((long)pl[4]);
  if (!w1 || !w2 || !w3) return ERROR_MEMORY_NOT_FOUND;
  if (w1->count < hidden * dim || w2->count < hidden * dim || w3->count < hidden * dim) return ERROR_MEMORY_TOO_SMALL;
  if (w1->bf16 != w2->bf16 || w1->bf16 != w3->bf16) return ERROR_MEMORY_MIXED_HALF_TYPES;
  return proj_result(k, mca_decode_ffn(g, pf[0], w1->ptr, w2->ptr, w3->ptr, w1->bf16 ? 1 : 0, (int)B, (int)dim, (int)hidden, h, x, 0), (long)B);
}

long decode_logits(Kernel* k, long lInput, float* pf, long llInput, MCA_LONGLONG* pl) {
  long e;
  if ((e = verify_in(lInput, pf, 1, 1)) || (e = verify_in(llInput, pl, 7, 7))) return e;
  const int64_t B = pl[3], dim = pl[4], vocab = pl[5];
  if (B <= 0 || dim <= 0 || vocab <= 0 || B > INT32_MAX || dim > INT32_MAX || vocab > INT32_MAX) return ERROR_PARAM_OUT_OF_RANGE;
  float *x, *g, *out;
  if ((e = check_f32(k, (long)pl[0], B * dim, &x)) || (e = check_f32(k, (long)pl[1], dim, &g)) ||
      (e = check_f32(k, (long)pl[6], B * vocab, &out)))
    return e;
  MemItem* wc = k->get((long)pl[2]);
  if (!wc) return ERROR_MEMORY_NOT_FOUND;
  if (wc->count < vocab * dim) return ERROR_MEMORY_TOO_SMALL;
  return proj_result(k, mca_decode_logits(x, g, pf[0], wc->ptr, wc->bf16 ? 1 : 0, (int)B, (int)dim, (int)vocab, out, 0), (long)B);
}

// Device<T>::CreateLayerNorm / FreeLayerNorm / LayerNormForward / LayerNormBackward, device.h:4123-4195
long layernorm_create(Kernel* k, long lInput, float* pf, long llInput, MCA_LONGLONG* pl, MCA_LONG* plOutput, float** ppOutput) {
  long e;
  if ((e = verify_in(lInput, pf, 1, 1)) || (e = verify_in(llInput, pl, 5, 5)) || (e = verify_out(plOutput, ppOutput))) return e;
  const int64_t count = pl[1], outer = pl[2], channels = pl[3], inner = pl[4];
  if (count <= 0 || outer <= 0 || channels <= 0 || inner <= 0 || inner > INT32_MAX) return ERROR_PARAM_OUT_OF_RANGE;
  if (count != outer * channels * inner) return ERROR_PARAM_OUT_OF_RANGE;   // LayerNormMemory<T>::Initialize, layernorm.cu:154-155
  LayerNormHandle h;
  h.rows = outer * channels; h.inner = (int)inner; h.eps = pf[0];
  if (cudaMalloc(&h.stdev, (size_t)h.rows * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return ERROR_MEMORY_OUT; }
  const long id = k->next_handle++;
  k->layernorm[id] = h;
  return set_out((float)id, plOutput, ppOutput);
}

long layernorm_free(Kernel* k, long lInput, float* pf) {
  long e;
  if ((e = verify_in(lInput, pf, 1, 1))) return e;
  auto it = k->layernorm.find((long)pf[0]);
  if (it == k->layernorm.end()) return ERROR_LAYERNORM_NOT_INITIALIZED;
  cudaFree(it->second.stdev);
  k->layernorm.erase(it);
  return 0;
}

long layernorm_run(Kernel* k, long llInput, MCA_LONGLONG* pl, bool backward) {
  long e;
  if ((e = verify_in(llInput, pl, backward ? 4 : 3, backward ? 4 : 3))) return e;
  auto it = k->layernorm.find((long)pl[0]);
  if (it == k->layernorm.end()) return ERROR_LAYERNORM_NOT_INITIALIZED;
  LayerNormHandle& h = it->second;
  const int64_t n = h.rows * h.inner;
  if (!backward) {
    float *x, *y;
    if ((e = check_f32(k, (long)pl[1], n, &x)) || (e = check_f32(k, (long)pl[2], n, &y))) return e;
    h.have_fwd = true;
    return mca_layernorm_forward_f32(x, y, h.stdev, h.rows, h.inner, h.eps, 0);
  }
  if (!h.have_fwd) return ERROR_LAYERNORM_NOT_INITIALIZED;   // the divisor is the forward's stdev
  float *y, *dy, *dx;
  if ((e = check_f32(k, (long)pl[1], n, &y)) || (e = check_f32(k, (long)pl[2], n, &dy)) || (e = check_f32(k, (long)pl[3], n, &dx))) return e;
  return mca_layernorm_backward_f32(y, dy, h.stdev, dx, h.rows, h.inner, h.eps, 0);
}

long rmsnorm_run(Kernel* k, long lInput, float* pf, long llInput, MCA_LONGLONG* pl, bool backward) {
  long e;
  if ((e = verify_in(llInput, pl, backward ? 8 : 6, backward ? 8 : 6))) return e;
  const int64_t rows = pl[backward ? 6 : 4], inner = pl[backward ? 7 : 5];
  if (rows <= 0 || inner <= 0 || inner > INT32_MAX) return ERROR_PARAM_OUT_OF_RANGE;
  const int64_t n = rows * inner;
  float *x, *w = nullptr;
  if ((e = check_f32(k, (long)pl[0], n, &x))) return e;
  if (pl[1] != 0 && (e = check_f32(k, (long)pl[1], inner, &w))) return e;
  if (!backward) {
    if ((e = verify_in(lInput, pf, 1, 1))) return e;
    float *y, *inv = nullptr;
    if ((e = check_f32(k, (long)pl[2], n, &y))) return e;
    if (pl[3] != 0 && (e = check_f32(k, (long)pl[3], rows, &inv))) return e;
    return mca_rmsnorm_forward_f32(x, w, y, inv, rows, (int)inner, pf[0], 0);
  }
  float *dy, *inv, *dx, *dw = nullptr;
  if ((e = check_f32(k, (long)pl[2], n, &dy)) || (e = check_f32(k, (long)pl[3], rows, &inv)) || (e = check_f32(k, (long)pl[4], n, &dx))) return e;
  if (pl[5] != 0) {
    if (!w) return ERROR_PARAM_NULL;
    if ((e = check_f32(k, (long)pl[5], inner, &dw))) return e;
    const int64_t need = mca_rmsnorm_backward_scratch_floats((int)inner);
    if (need > k->norm_scratch_floats) {
      cudaFree(k->norm_scratch);
      k->norm_scratch = nullptr; k->norm_scratch_floats = 0;
      if (cudaMalloc(&k->norm_scratch, (size_t)need * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return ERROR_MEMORY_OUT; }
      k->norm_scratch_floats = need;
    }
  }
  return mca_rmsnorm_backward_f32(x, w, dy, inv, dx, dw, k->norm_scratch, k->norm_scratch_floats, rows, (int)inner, 0);
}

long tft_fwd(Kernel* k, long llInput, MCA_LONGLONG* pl) {
  long e;
  if ((e = verify_in(llInput, pl, 11, 11))) return e;
  const int B = (int)pl[4], H = (int)pl[5], Nq = (int)pl[6], Nk = (int)pl[7], d = (int)pl[8];
  if (B <= 0 || H <= 0 || Nq <= 0 || Nk <= 0 || d <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  float *q, *kk, *v, *mask = nullptr, *out, *attn;
  if ((e = check_f32(k, (long)pl[0], (int64_t)B * H * Nq * d, &q)) || (e = check_f32(k, (long)pl[1], (int64_t)B * H * Nk * d, &kk)) ||
      (e = check_f32(k, (long)pl[2], (int64_t)B * Nk * d, &v)) || (e = check_f32(k, (long)pl[9], (int64_t)B * Nq * d, &out)) ||
      (e = check_f32(k, (long)pl[10], (int64_t)B * Nq * Nk, &attn)))
    return e;
  if (pl[3] != 0 && (e = check_f32(k, (long)pl[3], (int64_t)Nq * Nk, &mask))) return e;
  return mca_tft_attention_forward_f32(q, kk, v, mask, B, H, Nq, Nk, d, out, attn, 0);
}

long tft_bwd(Kernel* k, long llInput, MCA_LONGLONG* pl) {
  long e;
  if ((e = verify_in(llInput, pl, 14, 14))) return e;
  const int B = (int)pl[6], H = (int)pl[7], Nq = (int)pl[8], Nk = (int)pl[9], d = (int)pl[10];
  if (B <= 0 || H <= 0 || Nq <= 0 || Nk <= 0 || d <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  float *q, *kk, *v, *mask = nullptr, *go, *ga = nullptr, *dq, *dk, *dv;
  if ((e = check_f32(k, (long)pl[0], (int64_t)B * H * Nq * d, &q)) || (e = check_f32(k, (long)pl[1], (int64_t)B * H * Nk * d, &kk)) ||
      (e = check_f32(k, (long)pl[2], (int64_t)B * Nk * d, &v)) || (e = check_f32(k, (long)pl[4], (int64_t)B * Nq * d, &go)) ||
      (e = check_f32(k, (long)pl[11], (int64_t)B * H * Nq * d, &dq)) || (e = check_f32(k, (long)pl[12], (int64_t)B * H * Nk * d, &dk)) ||
      (e = check_f32(k, (long)pl[13], (int64_t)B * Nk * d, &dv)))
    return e;
  if (pl[3] != 0 && (e = check_f32(k, (long)pl[3], (int64_t)Nq * Nk, &mask))) return e;
  if (pl[5] != 0 && (e = check_f32(k, (long)pl[5], (int64_t)B * Nq * Nk, &ga))) return e;
  return mca_tft_attention_backward_f32(q, kk, v, mask, go, ga, B, H, Nq, Nk, d, dq, dk, dv, 0);
}

// ---- extensions (parent side) --------------------------------------------------------------

// This library's own dlopen handle: what an extension is given as hParent (g_hModule in the reference).
void* self_module() {
  static void* self = nullptr;
  if (!self) {
    Dl_info info;
    if (dladdr(reinterpret_cast<void*>(&DLL_InvokeFloat), &info) && info.dli_fname)
      self = dlopen(info.dli_fname, RTLD_NOW | RTLD_NOLOAD);
  }
  return self;
}

// extensionHandle<float>::InitializeFloat, Cuda Files/extension.cu:33-83.  An empty path selects the llama2
// extension built into this library.
long extension_create(Kernel* k, MCA_LONG kernel_idx, const char* path, MCA_LONG* plOutput, float** ppOutput) {
  long e;
  if ((e = verify_out(plOutput, ppOutput))) return e;
  ExtensionHandle x;
  ExtInitFn init = nullptr;
  if (!path || !path[0]) {
    init = &DLL_InitFloatCustomExtension;
    x.run = &DLL_InvokeFloatCustomExtension;
    x.run_ex = &DLL_InvokeFloatCustomExtensionEx;
  } else {
    x.lib = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!x.lib) { k->last_detail = dlerror(); return 126; }  // ERROR_MOD_NOT_FOUND, what GetLastError gives after LoadLibrary
    init = (ExtInitFn)dlsym(x.lib, "DLL_InitFloatCustomExtension");
    x.run = (ExtInvokeFn)dlsym(x.lib, "DLL_InvokeFloatCustomExtension");
    x.run_ex = (ExtInvokeExFn)dlsym(x.lib, "DLL_InvokeFloatCustomExtensionEx");   // optional
    if (!init || !x.run) { dlclose(x.lib); return 50; }  // ERROR_NOT_SUPPORTED
  }
  void* self = self_module();
  if (!self) { if (x.lib) dlclose(x.lib); return ERROR_DLL_NOT_INIT; }
  if ((e = init(self, kernel_idx))) { if (x.lib) dlclose(x.lib); return e; }
  const long h = k->next_handle++;
  k->extensions[h] = x;
  return set_out((float)h, plOutput, ppOutput);
}

long extension_free(Kernel* k, long lInput, float* pf) {
  long e;
  if ((e = verify_in(lInput, pf, 1, 1))) return e;
  auto it = k->extensions.find((long)pf[0]);
  if (it == k->extensions.end()) return ERROR_PARAM_OUT_OF_RANGE;
  if (it->second.lib) dlclose(it->second.lib);
  k->extensions.erase(it);
  return 0;
}

// Device<T>::ExtensionRun, device.h:4570-4588 (floats {hExtension, fn, args...}); with a string the call goes to
// the extension's ...Ex entry (Kernel<T>::RunExtensionFloat, CudaDnnDLL.cpp:1053-1064).  The extension writes
// its own message into szErr.
long extension_run(Kernel* k, long lInput, float* pf, const char* text, float** ppOutput, MCA_LONG* plOutput,
                   MCA_LPTSTR szErr, MCA_LONG lszErrMax) {
  long e;
  if ((e = verify_in(lInput, pf, 2, 0x7fffffff))) return e;
  auto it = k->extensions.find((long)pf[0]);
  if (it == k->extensions.end()) return ERROR_PARAM_OUT_OF_RANGE;
  const MCA_LONG fn = (MCA_LONG)pf[1];
  float* args = lInput > 2 ? pf + 2 : nullptr;
  if (szErr && lszErrMax > 0) szErr[0] = 0;
  if (text) {
    if (!it->second.run_ex) return ERROR_NOT_IMPLEMENTED;
    return it->second.run_ex(fn, args, (MCA_LONG)(lInput - 2), nullptr, nullptr, const_cast<char*>(text), nullptr, 0, szErr, lszErrMax);
  }
  return it->second.run(fn, args, (MCA_LONG)(lInput - 2), ppOutput, plOutput, szErr, lszErrMax);
}

// ---- kernel lifecycle ----------------------------------------------------------------------

long kernel_init(float* pInput, long lInput, long* idx_out) {
  long e;  // CUDA_DLL_INITIALIZE: floats {deviceId, flags}, CudaDnnDLL.cpp:154-176
  if ((e = verify_in(lInput, pInput, 1, 3))) return e;
  const int dev = (int)pInput[0];
  int count = 0;
  cudaError_t ce = cudaGetDeviceCount(&count);
  if (ce != cudaSuccess) { cudaGetLastError(); return ce; }
  if (dev < 0 || dev >= count) return ERROR_PARAM_OUT_OF_RANGE;
  cudaDeviceProp prop;
  if ((ce = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess) return ce;
  if (prop.major != 10) return ERROR_ATTN_NOT_B200;  // sm_100a code only: fail loudly elsewhere
  if ((ce = cudaSetDevice(dev)) != cudaSuccess) return ce;
  std::lock_guard<std::mutex> lock(g_table_lock);
  for (int i = 1; i < kMaxKernels; ++i) {
    if (!g_kernels[i]) {
      g_kernels[i] = new Kernel();
      g_kernels[i]->device = dev;
      *idx_out = i;
      return 0;
    }
  }
  return ERROR_MEMORY_OUT;
}

void kernel_cleanup(long idx) {
  std::lock_guard<std::mutex> lock(g_table_lock);
  Kernel* k = g_kernels[idx];
  if (!k) return;
  cudaSetDevice(k->device);
  cudaDeviceSynchronize();
  for (auto& kv : k->mem) cudaFree(kv.second.ptr);
  for (auto& kv : k->attn) kv.second.release();
  for (auto& kv : k->rope) { cudaFree(kv.second.cos_t); cudaFree(kv.second.sin_t); }
  for (auto& kv : k->layernorm) cudaFree(kv.second.stdev);
  cudaFree(k->norm_scratch);
  for (auto& kv : k->decode) { cudaFree(kv.second.fr); cudaFree(kv.second.fi); cudaFree(kv.second.scratch); }
  for (void* p : k->host_bufs) cudaFreeHost(p);
  if (k->h_answer) cudaFreeHost(k->h_answer);
  for (auto& kv : k->extensions) if (kv.second.lib) dlclose(kv.second.lib);
  if (k->ev0) cudaEventDestroy(k->ev0);
  if (k->ev1) cudaEventDestroy(k->ev1);
  cudaFree(k->stage);
  delete k;
  g_kernels[idx] = nullptr;
}

long run(Kernel* k, long fn, float* pf, long lInput, MCA_LONGLONG* pl, long llInput, float** ppOutput,
         MCA_LONG* plOutput) {
  cudaError_t ce = cudaSetDevice(k->device);
  if (ce != cudaSuccess) return ce;
  k->last_detail.clear();
  long e;
  switch (fn) {
    case CUDA_FN_SETDEVICE: return 0;
    case CUDA_FN_SYNCHRONIZEDEVICE: return sync_and_collect_status(k);
    case CUDA_FN_ALLOCMEM: return alloc_mem(k, lInput, pf, llInput, pl, plOutput, ppOutput, false);
    case MCA_FN_ALLOCMEM_BF16: return alloc_mem(k, lInput, pf, llInput, pl, plOutput, ppOutput, true);
    case CUDA_FN_FREEMEM: return free_mem(k, llInput, pl);
    case CUDA_FN_GETMEM: return get_mem(k, llInput, pl, plOutput, ppOutput);
    case CUDA_FN_SETMEM: return set_mem(k, lInput, pf, llInput, pl);
    case MCA_FN_CONVERT: return finish(k, convert_mem(k, llInput, pl));
    case CUDNN_FN_CREATE_CUDNN: {
      if ((e = verify_out(plOutput, ppOutput))) return e;
      const long h = k->next_handle++;
      k->cudnn[h] = 1;
      return set_out((float)h, plOutput, ppOutput);
    }
    case CUDNN_FN_FREE_CUDNN:
      if ((e = verify_in(lInput, pf, 1, 1))) return e;
      k->cudnn.erase((long)pf[0]);
      return 0;
    case CUDNN_FN_ATTN_CREATE: {
      if ((e = verify_out(plOutput, ppOutput))) return e;
      const long h = k->next_handle++;
      k->attn[h] = AttnHandle();
      return set_out((float)h, plOutput, ppOutput);
    }
    case CUDNN_FN_ATTN_FREE: {
      if ((e = verify_in(lInput, pf, 1, 1))) return e;
      auto it = k->attn.find((long)pf[0]);
      if (it == k->attn.end()) return ERROR_PARAM_OUT_OF_RANGE;
      cudaStreamSynchronize(0);
      it->second.release();
      k->attn.erase(it);
      return 0;
    }
    case CUDNN_FN_ATTN_SET: return finish(k, attn_set(k, lInput, pf, llInput, pl));
    case CUDNN_FN_ATTN_FWD: return finish(k, attn_fwd(k, llInput, pl, MCA_LAYOUT_BHTD));
    case CUDNN_FN_ATTN_BWD: return finish(k, attn_bwd(k, llInput, pl, MCA_LAYOUT_BHTD));
    case MCA_FN_ATTN_FWD_PACKED: {
      if ((e = verify_in(llInput, pl, 7, 7))) return e;
      MCA_LONGLONG a9[9] = {pl[0], pl[1], pl[2], pl[3], pl[3], pl[3], pl[4], pl[5], pl[6]};
      return finish(k, attn_fwd(k, 9, a9, MCA_LAYOUT_PACKED));
    }
    case MCA_FN_ATTN_BWD_PACKED: {
      if ((e = verify_in(llInput, pl, 7, 7))) return e;
      MCA_LONGLONG a11[11] = {pl[0], pl[1], pl[2], pl[3], pl[2], pl[3], pl[2], pl[3], pl[4], pl[5], pl[6]};
      return finish(k, attn_bwd(k, 11, a11, MCA_LAYOUT_PACKED));
    }
    case CUDA_FN_CREATE_LAYERNORM: return layernorm_create(k, lInput, pf, llInput, pl, plOutput, ppOutput);
    case CUDA_FN_FREE_LAYERNORM: return layernorm_free(k, lInput, pf);
    case CUDA_FN_LAYERNORM_FWD: return finish(k, layernorm_run(k, llInput, pl, false));
    case CUDA_FN_LAYERNORM_BWD: return finish(k, layernorm_run(k, llInput, pl, true));
    case MCA_FN_RMSNORM_FWD: return finish(k, rmsnorm_run(k, lInput, pf, llInput, pl, false));
    case MCA_FN_RMSNORM_BWD: return finish(k, rmsnorm_run(k, lInput, pf, llInput, pl, true));
    case CUDA_FN_CREATE_ROPE: return rope_create(k, lInput, pf, llInput, pl, plOutput, ppOutput);
    case CUDA_FN_FREE_ROPE: return rope_free(k, lInput, pf);
    case CUDA_FN_ROPE_FWD: return finish(k, rope_run(k, llInput, pl, false));
    case CUDA_FN_ROPE_BWD: return finish(k, rope_run(k, llInput, pl, true));
    case MCA_FN_DECODE_CREATE: return decode_create(k, lInput, pf, llInput, pl, plOutput, ppOutput);
    case MCA_FN_DECODE_FREE: return decode_free(k, lInput, pf);
    case MCA_FN_DECODE_STEP: return finish(k, decode_step(k, llInput, pl));
    case MCA_FN_DECODE_QKV: return finish(k, decode_qkv(k, lInput, pf, llInput, pl));
    case MCA_FN_DECODE_OUT: return finish(k, decode_out(k, llInput, pl));
    case MCA_FN_DECODE_FFN: return finish(k, decode_ffn(k, lInput, pf, llInput, pl));
    case MCA_FN_DECODE_LOGITS: return finish(k, decode_logits(k, lInput, pf, llInput, pl));
    case MCA_FN_TFT_ATTN_FWD: return finish(k, tft_fwd(k, llInput, pl));
    case MCA_FN_TFT_ATTN_BWD: return finish(k, tft_bwd(k, llInput, pl));
    case MCA_FN_ATTN_FWD_HOST:
      if ((e = verify_in(llInput, pl, 10, 11))) return e;
      return mca_sdpa_forward_host(reinterpret_cast<const void*>(pl[0]), reinterpret_cast<const void*>(pl[1]),
                                   reinterpret_cast<const void*>(pl[2]), reinterpret_cast<void*>(pl[3]), (int)pl[4],
                                   (int)pl[5], (int)pl[6], (int)pl[7], (int)pl[8], (int)pl[9],
                                   llInput > 10 ? (int)pl[10] : 0);
    case MCA_FN_SET_ASYNC:
      if ((e = verify_in(llInput, pl, 1, 1))) return e;
      if (k->async && pl[0] == 0 && (e = sync_and_collect_status(k))) return e;
      k->async = pl[0] != 0;
      return 0;
    case MCA_FN_SET_TIMING:
      if ((e = verify_in(llInput, pl, 1, 1))) return e;
      k->timing = pl[0] != 0;
      if (k->timing && !k->ev0) {
        cudaError_t c1 = cudaEventCreate(&k->ev0), c2 = cudaEventCreate(&k->ev1);
        if (c1 != cudaSuccess || c2 != cudaSuccess) { k->timing = false; return c1 != cudaSuccess ? c1 : c2; }
      }
      return 0;
    case CUDA_FN_FREE_EXTENSION: return extension_free(k, lInput, pf);
    case MCA_FN_WAIT_PROBE: {
      if ((e = verify_in(llInput, pl, 2, 2))) return e;
      auto it = k->attn.find((long)pl[0]);
      if (it == k->attn.end() || !it->second.configured) return ERROR_ATTN_NOT_INITIALIZED;
      if ((e = mca_wait_probe(it->second.causal_flag + 1, (int)pl[1], 0))) return e;
      return finish(k, tc_status(k, it->second));
    }
  }
  return ERROR_NOT_IMPLEMENTED;
}

// Every dispatched call is counted per function id; with MCA_FN_SET_TIMING on it is also bracketed by two events on
// the stream the work is issued on (the per-call figure the reference only has as a host Stopwatch around a layer,
// MyCaffe/layers/Layer.cs:695-722).  Read back as text through DLL_QueryString(MCA_FN_QUERY_COUNTERS).
long run_counted(Kernel* k, long fn, float* pf, long lInput, MCA_LONGLONG* pl, long llInput, float** ppOutput,
                 MCA_LONG* plOutput) {
  const bool timed = k->timing && fn != MCA_FN_SET_TIMING && fn != MCA_FN_ATTN_FWD_HOST;
  if (timed) { cudaSetDevice(k->device); cudaEventRecord(k->ev0, 0); }
  const long e = run(k, fn, pf, lInput, pl, llInput, ppOutput, plOutput);
  CallCounter& c = k->counters[fn];
  c.calls++;
  if (e) c.errors++;
  if (timed) {
    cudaEventRecord(k->ev1, 0);
    if (cudaEventSynchronize(k->ev1) == cudaSuccess) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, k->ev0, k->ev1) == cudaSuccess) { c.gpu_ms_last = ms; c.gpu_ms_total += ms; }
    }
    cudaGetLastError();
  }
  return e;
}

long invoke(MCA_LONG lKernelIdx, MCA_LONG fn, float* pInput, MCA_LONG lInput, MCA_LONGLONG* plInput,
            MCA_LONG llInput, float** ppOutput, MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG lszErrMax) {
  if (lKernelIdx < 0 || lKernelIdx >= kMaxKernels) return ERROR_PARAM_OUT_OF_RANGE;  // CudaDnnDLL.cpp:144-145
  long e = 0;
  if (fn == CUDA_DLL_INITIALIZE) {
    if ((e = verify_out(plOutput, ppOutput))) { get_error(e, szErr, lszErrMax); return e; }
    long idx = 0;
    if ((e = kernel_init(pInput, lInput, &idx))) { get_error(e, szErr, lszErrMax); return e; }
    return set_out((float)idx, plOutput, ppOutput);
  }
  if (fn == CUDA_DLL_CLEANUP) { kernel_cleanup(lKernelIdx); return 0; }
  Kernel* k = g_kernels[lKernelIdx];
  if (!k) { e = ERROR_PARAM_NULL; get_error(e, szErr, lszErrMax); return e; }
  if (fn == CUDA_DLL_FREEMEM) {  // Kernel<T>::FreeHost, CudaDnnDLL.cpp:188-201
    for (size_t i = 0; i < k->host_bufs.size(); ++i)
      if (k->host_bufs[i] == (void*)pInput) {
        cudaFreeHost(pInput);
        k->host_bufs.erase(k->host_bufs.begin() + i);
        return 0;
      }
    e = ERROR_MEMORY_NOT_FOUND;
    get_error(e, szErr, lszErrMax);
    return e;
  }
  if (fn == CUDA_FN_EXTENSION_RUN) {  // Kernel<T>::Run(lfnIdx, ..., szErr), Cuda Files/main.cu:1262-1275
    cudaSetDevice(k->device);
    k->last_detail.clear();
    e = extension_run(k, lInput, pInput, nullptr, ppOutput, plOutput, szErr, lszErrMax);
    if (e && szErr && lszErrMax > 0 && szErr[0] == 0) get_error(e, szErr, lszErrMax, k);
    return e;
  }
  e = run_counted(k, fn, pInput, lInput, plInput, llInput, ppOutput, plOutput);
  if (e) get_error(e, szErr, lszErrMax, k);
  return e;
}

// DLL_InvokeFloatEx: only the two ids that take a string exist there (CudaDnnDLL.cpp:1036-1084); everything else is
// ERROR_NOT_SUPPORTED in the reference.  Other ids are passed to the ordinary dispatch here so that a binding that
// routes everything through this entry keeps working.
long invoke_ex(MCA_LONG lKernelIdx, MCA_LONG fn, float* pInput, MCA_LONG lInput, const char* text, float** ppOutput,
               MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG lszErrMax) {
  if (fn != CUDA_FN_CREATE_EXTENSION && fn != CUDA_FN_EXTENSION_RUN)
    return invoke(lKernelIdx, fn, pInput, lInput, nullptr, 0, ppOutput, plOutput, szErr, lszErrMax);
  if (lKernelIdx < 0 || lKernelIdx >= kMaxKernels) return ERROR_PARAM_OUT_OF_RANGE;
  Kernel* k = g_kernels[lKernelIdx];
  long e = 0;
  if (!k) { e = ERROR_PARAM_NULL; get_error(e, szErr, lszErrMax); return e; }
  cudaSetDevice(k->device);
  k->last_detail.clear();
  if (fn == CUDA_FN_CREATE_EXTENSION) {
    e = extension_create(k, lKernelIdx, text, plOutput, ppOutput);
    if (e) get_error(e, szErr, lszErrMax, k);
    return e;
  }
  e = extension_run(k, lInput, pInput, text ? text : "", ppOutput, plOutput, szErr, lszErrMax);
  if (e && szErr && lszErrMax > 0 && szErr[0] == 0) get_error(e, szErr, lszErrMax, k);
  return e;
}

// Device<T>::GetDeviceName, Cuda Files/device.cu:528-554.
long device_name(long lInput, const MCA_LONG* pInput, char** out) {
  if (!pInput) return ERROR_PARAM_NULL;
  if (lInput < 1) return ERROR_PARAM_OUT_OF_RANGE;
  cudaDeviceProp prop;
  cudaError_t ce = cudaGetDeviceProperties(&prop, (int)pInput[0]);
  if (ce != cudaSuccess) { cudaGetLastError(); return ce; }
  char* dst = (char*)malloc(512);
  if (!dst) return ERROR_MEMORY_OUT;
  const double gb = (double)prop.totalGlobalMem / 1000000000.00;
  const bool p2p = sizeof(void*) == 8 && prop.tccDriver == 1 && prop.major >= 2;
  snprintf(dst, 512, "%s (%d.%02d GB - %s; compute %d.%d)", prop.name, (int)gb, (int)(gb * 100) % 100, p2p ? "P2P on" : "P2P off",
           prop.major, prop.minor);
  *out = dst;
  return 0;
}

long counters_text(const Kernel* k, char** out) {
  std::string t;
  char line[160];
  for (const auto& kv : k->counters) {
    snprintf(line, sizeof(line), "%ld calls=%ld errors=%ld gpu_ms_last=%.4f gpu_ms_total=%.4f\n", kv.first, kv.second.calls,
             kv.second.errors, kv.second.gpu_ms_last, kv.second.gpu_ms_total);
    t += line;
  }
  char* dst = (char*)malloc(t.size() + 1);
  if (!dst) return ERROR_MEMORY_OUT;
  memcpy(dst, t.c_str(), t.size() + 1);
  *out = dst;
  return 0;
}

}  // namespace

extern "C" {

MCA_LONG DLL_InvokeFloat(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, float* pInput, MCA_LONG lInput, float** ppOutput,
                         MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG lszErrMax) {
  return (MCA_LONG)invoke(lKernelIdx, lFunctionIdx, pInput, lInput, nullptr, 0, ppOutput, plOutput, szErr, lszErrMax);
}

MCA_LONG DLL_InvokeFloatEx2(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, float* pInput, MCA_LONG lInput,
                            MCA_LONGLONG* plInput, MCA_LONG llInput, float** ppOutput, MCA_LONG* plOutput,
                            MCA_LPTSTR szErr, MCA_LONG lszErrMax) {
  return (MCA_LONG)invoke(lKernelIdx, lFunctionIdx, pInput, lInput, plInput, llInput, ppOutput, plOutput, szErr, lszErrMax);
}

MCA_LONG DLL_InvokeFloatEx(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, float* pInput, MCA_LONG lInput, MCA_LPTSTR pszInput,
                           float** ppOutput, MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG lszErrMax) {
  return (MCA_LONG)invoke_ex(lKernelIdx, lFunctionIdx, pInput, lInput, pszInput, ppOutput, plOutput, szErr, lszErrMax);
}

MCA_LONG DLL_InvokeDouble(MCA_LONG, MCA_LONG, double*, MCA_LONG, double**, MCA_LONG*, MCA_LPTSTR szErr, MCA_LONG lszErrMax) {
  get_error(ERROR_NOT_IMPLEMENTED, szErr, lszErrMax);
  return ERROR_NOT_IMPLEMENTED;
}

MCA_LONG DLL_InvokeDoubleEx2(MCA_LONG, MCA_LONG, double*, MCA_LONG, MCA_LONGLONG*, MCA_LONG, double**, MCA_LONG*,
                             MCA_LPTSTR szErr, MCA_LONG lszErrMax) {
  get_error(ERROR_NOT_IMPLEMENTED, szErr, lszErrMax);
  return ERROR_NOT_IMPLEMENTED;
}

MCA_LONG DLL_InvokeDoubleEx(MCA_LONG, MCA_LONG, double*, MCA_LONG, MCA_LPTSTR, double**, MCA_LONG*, MCA_LPTSTR szErr,
                            MCA_LONG lszErrMax) {
  get_error(ERROR_NOT_IMPLEMENTED, szErr, lszErrMax);
  return ERROR_NOT_IMPLEMENTED;
}

MCA_LONG DLL_QueryString(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, MCA_LONG* pInput, MCA_LONG lInput, MCA_LPTSTR* ppOutput,
                         MCA_LPTSTR szErr, MCA_LONG lszErrMax) {
  if (lKernelIdx < 0 || lKernelIdx >= kMaxKernels) return ERROR_PARAM_OUT_OF_RANGE;
  Kernel* k = g_kernels[lKernelIdx];
  long e = 0;
  if (!k) { e = ERROR_PARAM_OUT_OF_RANGE; get_error(e, szErr, lszErrMax); return (MCA_LONG)e; }  // CudaDnnDLL.cpp:928-931
  if (lFunctionIdx == CUDA_DLL_FREEMEM) {  // the string came from malloc, CudaDnnDLL.cpp:876-882
    if (ppOutput && *ppOutput) { free(*ppOutput); *ppOutput = nullptr; }
    return 0;
  }
  if (!ppOutput) return ERROR_PARAM_NULL;
  *ppOutput = nullptr;
  if (szErr && lszErrMax > 0) szErr[0] = 0;
  switch (lFunctionIdx) {
    case CUDA_FN_GET_DEVICE_NAME: e = device_name(lInput, pInput, ppOutput); break;
    case MCA_FN_QUERY_VERSION: {
      const char* v = mca_version();
      *ppOutput = (char*)malloc(strlen(v) + 1);
      if (*ppOutput) strcpy(*ppOutput, v); else e = ERROR_MEMORY_OUT;
      break;
    }
    case MCA_FN_QUERY_COUNTERS: e = counters_text(k, ppOutput); break;
    default: e = ERROR_PARAM_OUT_OF_RANGE;  // Kernel<T>::Query, Cuda Files/main.cu:2475-2476
  }
  if (e) get_error(e, szErr, lszErrMax);
  return (MCA_LONG)e;
}

MCA_LONG DLL_QueryStringFloatEx(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, MCA_LONG* pInput, MCA_LONG lInput,
                                MCA_LPTSTR pszOutput, MCA_LONG lOutputMax, MCA_LPTSTR szErr, MCA_LONG lszErrMax) {
  if (lKernelIdx < 0 || lKernelIdx >= kMaxKernels) return ERROR_PARAM_OUT_OF_RANGE;
  Kernel* k = g_kernels[lKernelIdx];
  long e = 0;
  if (!k) { e = ERROR_PARAM_OUT_OF_RANGE; get_error(e, szErr, lszErrMax); return (MCA_LONG)e; }
  if (szErr && lszErrMax > 0) szErr[0] = 0;
  if (lFunctionIdx != CUDA_FN_GET_EXTENSION_STRING) e = ERROR_PARAM_OUT_OF_RANGE;  // Kernel<T>::QueryEx, main.cu:2492-2499
  else if (lInput < 2) e = ERROR_PARAM_OUT_OF_RANGE;                               // Device<T>::QueryExtensionResult, device.h:4591-4603
  else if (!pInput) e = ERROR_PARAM_NULL;
  else {
    // extensionHandle<float>::Query, Cuda Files/extension.cu:153-180: at most five arguments, passed as floats
    auto it = k->extensions.find((long)pInput[0]);
    const long n = lInput - 2;
    if (it == k->extensions.end() || n > 5) e = ERROR_PARAM_OUT_OF_RANGE;
    else if (!it->second.run_ex) e = ERROR_NOT_IMPLEMENTED;
    else {
      float args[5];
      for (long i = 0; i < n; ++i) args[i] = (float)pInput[2 + i];
      float* out = nullptr;
      MCA_LONG n_out = 0;
      cudaSetDevice(k->device);
      e = it->second.run_ex(pInput[1], args, (MCA_LONG)n, &out, &n_out, nullptr, pszOutput, lOutputMax, szErr, lszErrMax);
      if (!e && out != nullptr && pszOutput && lOutputMax > 0) strncat(pszOutput, "\n[END]", (size_t)lOutputMax - strlen(pszOutput) - 1);
    }
  }
  if (e && szErr && lszErrMax > 0 && szErr[0] == 0) get_error(e, szErr, lszErrMax);
  return (MCA_LONG)e;
}

MCA_LONG DLL_QueryStringDoubleEx(MCA_LONG lKernelIdx, MCA_LONG, MCA_LONG*, MCA_LONG, MCA_LPTSTR, MCA_LONG, MCA_LPTSTR szErr,
                                 MCA_LONG lszErrMax) {
  if (lKernelIdx < 0 || lKernelIdx >= kMaxKernels) return ERROR_PARAM_OUT_OF_RANGE;
  get_error(ERROR_NOT_IMPLEMENTED, szErr, lszErrMax);
  return ERROR_NOT_IMPLEMENTED;
}

MCA_LONG Internal_GetPointerDouble(MCA_LONG, MCA_LONG lKernelIdx, MCA_LONG, void**) {
  if (lKernelIdx < 0 || lKernelIdx >= kMaxKernels) return ERROR_PARAM_OUT_OF_RANGE;
  return ERROR_PARAM_NULL;  // no double kernel exists in any slot
}

MCA_LONG Internal_AllocHostDouble(MCA_LONG lKernelIdx, MCA_LONG, double**, double*, bool) {
  if (lKernelIdx < 0 || lKernelIdx >= kMaxKernels) return ERROR_PARAM_OUT_OF_RANGE;
  return ERROR_PARAM_NULL;
}

MCA_LONG Internal_GetPointerFloat(MCA_LONG ht, MCA_LONG lKernelIdx, MCA_LONG hHandle, void** ppPtr) {
  if (lKernelIdx < 0 || lKernelIdx >= kMaxKernels) return ERROR_PARAM_OUT_OF_RANGE;
  Kernel* k = g_kernels[lKernelIdx];
  if (!k || !ppPtr) return ERROR_PARAM_NULL;
  if (ht != MCA_HT_MEMORY) return ERROR_NOT_IMPLEMENTED;
  MemItem* m = k->get(hHandle);
  if (!m) return ERROR_MEMORY_NOT_FOUND;
  *ppPtr = m->ptr;
  return 0;
}

MCA_LONG Internal_AllocHostFloat(MCA_LONG lKernelIdx, MCA_LONG lCount, float** ppDst, float* pSrc, bool bSrcOnDevice) {
  if (lKernelIdx < 0 || lKernelIdx >= kMaxKernels) return ERROR_PARAM_OUT_OF_RANGE;
  Kernel* k = g_kernels[lKernelIdx];
  if (!k || !ppDst) return ERROR_PARAM_NULL;
  if (lCount <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  long e = alloc_host(k, lCount, ppDst);
  if (e) return (MCA_LONG)e;
  if (pSrc)
    return (MCA_LONG)cudaMemcpy(*ppDst, pSrc, (size_t)lCount * 4, bSrcOnDevice ? cudaMemcpyDeviceToHost : cudaMemcpyHostToHost);
  return 0;
}

int mca_rope_tables_host(int T, int D, float theta, float* cos_table, float* sin_table) {
  if (!cos_table || !sin_table) return ERROR_PARAM_NULL;
  if (T <= 0 || D <= 0 || (D & 1)) return ERROR_PARAM_OUT_OF_RANGE;
  const int half = D / 2;
  std::vector<float> freq(half);
  for (int i = 0, idx = 0; i < D; i += 2, ++idx) freq[idx] = 1.0f / powf(theta, (float)(i / (float)D));
  for (int pos = 0; pos < T; ++pos)
    for (int i = 0; i < half; ++i) {
      const float f = freq[i] * pos;
      cos_table[(size_t)pos * half + i] = cosf(f);
      sin_table[(size_t)pos * half + i] = sinf(f);
    }
  return 0;
}

const char* mca_version(void) { return "mycaffe_attn_b200 0.2 sm_100a"; }

}  // extern "C"

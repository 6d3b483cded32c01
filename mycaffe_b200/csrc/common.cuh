// Shared declarations for the attention library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cstdlib>
#include <cuda_bf16.h>
#include <stdint.h>

// Error codes of the reference's native layer that this path can return
// (CudaDnnDLL/Cuda Files/util.h:128-146,198-211).  CUDA runtime codes pass through unchanged.
constexpr int ERROR_BASE = 90000;
constexpr int ERROR_DLL_NOT_INIT = ERROR_BASE - 1;
constexpr int ERROR_PARAM = ERROR_BASE;
constexpr int ERROR_PARAM_OUT_OF_RANGE = ERROR_PARAM + 1;
constexpr int ERROR_PARAM_NULL = ERROR_PARAM + 2;
constexpr int ERROR_MEMORY_OUT = ERROR_PARAM + 7;
constexpr int ERROR_MEMORY_NULL = ERROR_PARAM + 8;
constexpr int ERROR_NOT_IMPLEMENTED = ERROR_PARAM + 9;
constexpr int ERROR_MEMORY_RANGE_EXCEEDED = ERROR_PARAM + 10;
constexpr int ERROR_MEMORY_MIXED_HALF_TYPES = ERROR_PARAM + 11;
constexpr int ERROR_MEMORY_NOT_FOUND = ERROR_PARAM + 14;
constexpr int ERROR_MEMORY_TOO_SMALL = ERROR_PARAM + 16;
// ERROR_MATRIX = +20, VECTOR = +40, NN = +60, CUDA = +80, TSNE = NN+40 = +100, SSD = +120,
// LAYERNORM = +160, ROPE = +200, RNN8 = +240, ATTN = +280 (util.h:150-211).
constexpr int ERROR_ROPE = ERROR_PARAM + 200;
constexpr int ERROR_ROPE_NOT_INITIALIZED = ERROR_ROPE + 1;
constexpr int ERROR_LAYERNORM = ERROR_ROPE - 40;                  // util.h:195-198
constexpr int ERROR_LAYERNORM_NOT_INITIALIZED = ERROR_LAYERNORM + 1;
constexpr int ERROR_ATTN = ERROR_PARAM + 280;
constexpr int ERROR_ATTN_NOT_INITIALIZED = ERROR_ATTN + 1;
constexpr int ERROR_ATTN_INCOMPATIBLE_BLOB_SIZE = ERROR_ATTN + 4;
constexpr int ERROR_ATTN_INVALID_BLOCK_SIZE = ERROR_ATTN + 5;
// Codes added by this library (outside every range the reference defines).
constexpr int ERROR_ATTN_B200 = ERROR_PARAM + 900;
constexpr int ERROR_ATTN_UNSUPPORTED_SHAPE = ERROR_ATTN_B200 + 1;   // head size / dtype combination has no kernel
constexpr int ERROR_ATTN_KERNEL_TIMEOUT = ERROR_ATTN_B200 + 2;      // a bounded device-side wait gave up
constexpr int ERROR_ATTN_BACKWARD_WITHOUT_FORWARD = ERROR_ATTN_B200 + 3;
constexpr int ERROR_ATTN_NOT_B200 = ERROR_ATTN_B200 + 4;            // device is not compute capability 10.x
constexpr int ERROR_ATTN_SCRATCH_TOO_SMALL = ERROR_ATTN_B200 + 5;
constexpr int ERROR_ATTN_STATIC_SCRATCH_EXCEEDED = ERROR_ATTN_B200 + 6;  // problem too large for the built-in scratch

// Value the reference writes over masked logits (finite): attn.cu:302-329.
#define MCA_MASKED_LOGIT (-1e29f)

// Mask modes shared by host and device code.
enum McaMaskMode : int {
  MCA_MASK_NONE = 0,    // hMask == 0 (attn.cu:544,571)
  MCA_MASK_TT = 1,      // (1,1,T,T), masked where mask == 0 (apply_mask)
  MCA_MASK_BATCH = 2,   // (B,T,1,1) key mask, masked where mask == 0 (apply_mask_batch)
  MCA_MASK_CAUSAL = 3,  // analytic lower triangle: same result as a tril(ones) MCA_MASK_TT mask
};

// Keep-bits of a caller's mask as the tensor-core kernels read them (mca_mask_pack): the words of query row r of batch
// item b for key tile j start at bits + b * batch_stride + r * row_stride + 4 j; bits_t is the transpose of a (T,T) mask.
struct McaMaskBits {
  const uint32_t* bits;
  const uint32_t* bits_t;
  int64_t batch_stride, row_stride;
};

// Element strides of a (B, H, T, D) view whose head dimension is contiguous.
struct McaStrides {
  int64_t b, h, t;
};
// layout 0: separate contiguous (B,H,T,D) tensors.  layout 1: q | k | v are the three feature thirds of a
// (B, T, 3*H*D) projection output (the c_attn blob of CausalSelfAttentionLayer.cs:537-557 before its split and
// head transposes) and the attention output is (B, T, H*D) (what c_proj consumes, :604).
static inline McaStrides mca_in_strides(int layout, int H, int T, int D) {
  if (layout == 1) return McaStrides{(int64_t)T * 3 * H * D, (int64_t)D, (int64_t)3 * H * D};
  return McaStrides{(int64_t)H * T * D, (int64_t)T * D, (int64_t)D};
}
static inline McaStrides mca_out_strides(int layout, int H, int T, int D) {
  if (layout == 1) return McaStrides{(int64_t)T * H * D, (int64_t)D, (int64_t)H * D};
  return McaStrides{(int64_t)H * T * D, (int64_t)T * D, (int64_t)D};
}

#define MCA_CUDA_TRY(expr)                      \
  do {                                          \
    cudaError_t _e = (expr);                    \
    if (_e != cudaSuccess) return (int)_e;      \
  } while (0)

static inline int mca_launch_status() {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
  return 0;
}

__host__ __device__ static inline int mca_ceil_div(int a, int b) { return (a + b - 1) / b; }

// Programmatic dependent launch.  A kernel launched with mca_launch_pdl may start while the
// previous kernel of the stream is still running (once every CTA of that kernel has executed
// mca_pdl_launch_dependents or exited); what it does before mca_pdl_wait() must depend on nothing
// the previous kernels write and must write nothing they read.  mca_pdl_wait() returns when all
// earlier kernels of the stream have completed and their writes are visible; in a kernel that was
// launched the ordinary way both calls do nothing.
#ifdef __CUDACC__
// 16-byte asynchronous copy global -> shared, bypassing L1; groups complete in order.
__device__ __forceinline__ void mca_cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void mca_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void mca_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mca_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void mca_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline int mca_launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  static const bool plain = getenv("MCA_NO_PDL") != nullptr;   // every launch the ordinary way (for comparisons)
  cfg.attrs = attr; cfg.numAttrs = plain ? 0 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
  if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
  return mca_launch_status();
}
#endif

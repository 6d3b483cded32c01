// Attention forward for tensors that live in HOST memory: the (batch, head) pairs are independent,
// so the problem is cut into chunks of consecutive pairs and three streams overlap, chunk by chunk,
//   host -> device copies of Q, K, V   |   the tcgen05 forward kernel   |   device -> host copy of Y.
// The reference moves whole tensors with blocking copies before and after the kernel
// (blocking cudaMemcpy, CudaDnnDLL/Cuda Files/memory.cu:451,539; the attention call
// itself synchronises the stream, attn.cu:601), so its host-to-host time is the SUM of the copy and
// kernel times; here it is close to the largest of them (the PCIe copy of the inputs).
//
// Host tensors may be fp32 (what the reference ABI carries; converted to bf16 on the device as part
// of the input stream) or bf16 (half the PCIe bytes).  Pinned host memory (Internal_AllocHostFloat
// or cudaHostAlloc) is needed for the copies to overlap; pageable memory works but serialises.
// Device staging is grow-only and owned by the library (per device), released by
// mca_host_pipeline_release().
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int SLOTS = 2;

struct Pipeline {
  int device = -1;
  cudaStream_t s_in = nullptr, s_comp = nullptr, s_out = nullptr;
  cudaEvent_t in_done[SLOTS] = {}, comp_done[SLOTS] = {}, out_done[SLOTS] = {};
  void* bf[SLOTS][4] = {};   // q, k, v, y chunks in bf16
  float* f32[SLOTS][4] = {}; // fp32 staging (fp32 host tensors only)
  size_t bf_bytes = 0, f32_bytes = 0;
  int* status = nullptr;
};

std::mutex g_mu;
Pipeline g_pipe[16];

void free_buffers(Pipeline& p) {
  for (int s = 0; s < SLOTS; ++s)
    for (int i = 0; i < 4; ++i) {
      if (p.bf[s][i]) cudaFree(p.bf[s][i]);
      if (p.f32[s][i]) cudaFree(p.f32[s][i]);
      p.bf[s][i] = nullptr;
      p.f32[s][i] = nullptr;
    }
  p.bf_bytes = p.f32_bytes = 0;
}

int ensure(Pipeline& p, int dev, size_t bf_bytes, size_t f32_bytes) {
  if (p.device != dev) {
    p.device = dev;
    MCA_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking));
    MCA_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_comp, cudaStreamNonBlocking));
    MCA_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking));
    for (int s = 0; s < SLOTS; ++s) {
      MCA_CUDA_TRY(cudaEventCreateWithFlags(&p.in_done[s], cudaEventDisableTiming));
      MCA_CUDA_TRY(cudaEventCreateWithFlags(&p.comp_done[s], cudaEventDisableTiming));
      MCA_CUDA_TRY(cudaEventCreateWithFlags(&p.out_done[s], cudaEventDisableTiming));
    }
    MCA_CUDA_TRY(cudaMalloc(&p.status, 8 * sizeof(int)));
  }
  if (bf_bytes > p.bf_bytes || f32_bytes > p.f32_bytes) {
    MCA_CUDA_TRY(cudaDeviceSynchronize());
    const size_t nb = bf_bytes > p.bf_bytes ? bf_bytes : p.bf_bytes;
    const size_t nf = f32_bytes > p.f32_bytes ? f32_bytes : p.f32_bytes;
    free_buffers(p);
    for (int s = 0; s < SLOTS; ++s)
      for (int i = 0; i < 4; ++i) {
        cudaError_t e = cudaMalloc(&p.bf[s][i], nb);
        if (e == cudaSuccess && nf) e = cudaMalloc(reinterpret_cast<void**>(&p.f32[s][i]), nf);
        if (e != cudaSuccess) {
          cudaGetLastError();
          free_buffers(p);
          return e == cudaErrorMemoryAllocation ? ERROR_MEMORY_OUT : (int)e;
        }
      }
    p.bf_bytes = nb;
    p.f32_bytes = nf;
  }
  return 0;
}

}  // namespace

int mca_host_pipeline_chunk(int B, int H, int T, int heads_per_chunk) {
  const int64_t BH = (int64_t)B * H;
  if (heads_per_chunk > 0) return (int)(heads_per_chunk < BH ? heads_per_chunk : BH);
  // enough CTAs (one per 256 query rows) to fill the 148 SMs about four times, but at least
  // four chunks -- eight where a chunk of BH/8 pairs still has a CTA for most SMs -- so that the copies
  // and the kernel have something to overlap with (the first copy and the last read-back are exposed:
  // 1/chunks of each direction's time)
  const int64_t tiles = (T + 255) / 256;
  int64_t c = (4 * 148 + tiles - 1) / tiles;
  if (c > BH / 4) c = BH / 4;
  if (BH >= 8 && c > BH / 8 && (BH / 8) * tiles >= 128) c = BH / 8;
  if (c < 1) c = 1;
  return (int)c;
}

int mca_sdpa_forward_host(const void* q, const void* k, const void* v, void* y, int host_dtype, int causal, int B,
                          int H, int T, int D, int heads_per_chunk) {
  if (!q || !k || !v || !y) return ERROR_PARAM_NULL;
  if (B <= 0 || H <= 0 || T <= 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (host_dtype != MCA_DTYPE_F32 && host_dtype != MCA_DTYPE_BF16) return ERROR_PARAM_OUT_OF_RANGE;
  if (D != 64 && D != 128) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  int dev = 0;
  MCA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 16) return ERROR_PARAM_OUT_OF_RANGE;
  const bool f32 = host_dtype == MCA_DTYPE_F32;
  const int64_t BH = (int64_t)B * H;
  const int chunk = mca_host_pipeline_chunk(B, H, T, heads_per_chunk);
  const int64_t head_elems = (int64_t)T * D;
  const size_t esz = f32 ? 4 : 2;

  std::lock_guard<std::mutex> lock(g_mu);
  Pipeline& p = g_pipe[dev];
  int e = ensure(p, dev, (size_t)chunk * head_elems * 2, f32 ? (size_t)chunk * head_elems * 4 : 0);
  if (e) return e;
  MCA_CUDA_TRY(cudaMemsetAsync(p.status, 0, 8 * sizeof(int), p.s_comp));

  const char* hq = static_cast<const char*>(q);
  const char* hk = static_cast<const char*>(k);
  const char* hv = static_cast<const char*>(v);
  char* hy = static_cast<char*>(y);
  // one chunk through the three streams; returns the first error (the caller still waits for what was issued)
  auto run_chunk = [&](int n, int64_t h0) -> int {
    const int s = n % SLOTS;
    const int c = (int)(BH - h0 < chunk ? BH - h0 : chunk);
    const int64_t elems = (int64_t)c * head_elems;
    const size_t off = (size_t)h0 * head_elems * esz;
    // ---- inputs: the slot's Q/K/V are free once the kernel of chunk n-SLOTS has run
    if (n >= SLOTS) MCA_CUDA_TRY(cudaStreamWaitEvent(p.s_in, p.comp_done[s], 0));
    const char* src[3] = {hq + off, hk + off, hv + off};
    for (int i = 0; i < 3; ++i) {
      if (f32) {
        MCA_CUDA_TRY(cudaMemcpyAsync(p.f32[s][i], src[i], elems * 4, cudaMemcpyHostToDevice, p.s_in));
        const int ce = mca_convert_f32_to_bf16(p.f32[s][i], p.bf[s][i], elems, p.s_in);
        if (ce) return ce;
      } else {
        MCA_CUDA_TRY(cudaMemcpyAsync(p.bf[s][i], src[i], elems * 2, cudaMemcpyHostToDevice, p.s_in));
      }
    }
    MCA_CUDA_TRY(cudaEventRecord(p.in_done[s], p.s_in));
    // ---- kernel: needs the inputs, and the slot's Y must have left for the host (chunk n-SLOTS)
    MCA_CUDA_TRY(cudaStreamWaitEvent(p.s_comp, p.in_done[s], 0));
    if (n >= SLOTS) MCA_CUDA_TRY(cudaStreamWaitEvent(p.s_comp, p.out_done[s], 0));
    const int ke = mca_sdpa_forward_tc(p.bf[s][0], p.bf[s][1], p.bf[s][2], MCA_DTYPE_BF16, causal, 1, c, T, D, p.bf[s][3],
                                       nullptr, p.status, p.s_comp);
    if (ke) return ke;
    MCA_CUDA_TRY(cudaEventRecord(p.comp_done[s], p.s_comp));
    // ---- output
    MCA_CUDA_TRY(cudaStreamWaitEvent(p.s_out, p.comp_done[s], 0));
    if (f32) {
      const int ce = mca_convert_bf16_to_f32(p.bf[s][3], p.f32[s][3], elems, p.s_out);
      if (ce) return ce;
      MCA_CUDA_TRY(cudaMemcpyAsync(hy + off, p.f32[s][3], elems * 4, cudaMemcpyDeviceToHost, p.s_out));
    } else {
      MCA_CUDA_TRY(cudaMemcpyAsync(hy + off, p.bf[s][3], elems * 2, cudaMemcpyDeviceToHost, p.s_out));
    }
    MCA_CUDA_TRY(cudaEventRecord(p.out_done[s], p.s_out));
    return 0;
  };
  int n = 0;
  for (int64_t h0 = 0; h0 < BH && !e; h0 += chunk, ++n) e = run_chunk(n, h0);
  // the call is synchronous: everything issued has finished (also after an error part-way)
  cudaError_t ce = cudaStreamSynchronize(p.s_in);
  cudaError_t c2 = cudaStreamSynchronize(p.s_comp);
  cudaError_t c3 = cudaStreamSynchronize(p.s_out);
  if (e) return e;
  if (ce != cudaSuccess) return (int)ce;
  if (c2 != cudaSuccess) return (int)c2;
  if (c3 != cudaSuccess) return (int)c3;
  int st[8];
  MCA_CUDA_TRY(cudaMemcpy(st, p.status, sizeof(st), cudaMemcpyDeviceToHost));
  return st[0] != 0 ? ERROR_ATTN_KERNEL_TIMEOUT : 0;
}

int mca_host_pipeline_release(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  int dev = 0;
  MCA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 16) return ERROR_PARAM_OUT_OF_RANGE;
  Pipeline& p = g_pipe[dev];
  if (p.device != dev) return 0;
  MCA_CUDA_TRY(cudaDeviceSynchronize());
  free_buffers(p);
  return 0;
}

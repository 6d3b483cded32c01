/* libmycaffe_attn -- C ABI of the B200 (sm_100a) attention library.
 *
 * Two layers, both plain C:
 *
 *  1. The reference's own dispatch ABI.  MyCaffe's C# CudaDnn<T> reaches native code through
 *     DLL_Invoke* with a kernel index, a function id and packed float / long arrays
 *     (CudaDnnDLL/CudaDnnDLL.cpp:134,314,495).  This library exports the same entry points with
 *     the same argument packing, error codes and handle semantics for the function ids on the
 *     attention path (and the few memory ids needed to own the handles), so a host binding for
 *     CudaDnnDLL binds this library unchanged.
 *
 *  2. Raw entry points (mca_*) that take device pointers, sizes and a CUDA stream.  The
 *     dispatch layer calls these; a host that owns its device memory may call them directly.
 *
 * Every function returns 0 on success, a CUDA runtime error code, or one of the ERROR_*
 * codes of the reference (CudaDnnDLL/Cuda Files/util.h:128-211; 90000-based).  There is no CPU
 * fallback anywhere: without a compute-capability-10.x device the calls fail.
 *
 * Paths in comments are relative to the reference project root.
 */
#ifndef MYCAFFE_ATTN_H_
#define MYCAFFE_ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define MCA_API __declspec(dllexport)
#else
#define MCA_API __attribute__((visibility("default")))
#endif

/* Windows types of the reference ABI.  LONG is 32-bit on Windows; LPTSTR is a char string
 * here (the ANSI build of the reference). */
typedef int32_t MCA_LONG;
typedef int64_t MCA_LONGLONG;
typedef char* MCA_LPTSTR;

/* ---- function ids honoured by DLL_Invoke* --------------------------------------------- */
/* Cuda Files/main.h:23-32 */
#define CUDA_DLL_FREEMEM (-1)      /* free a pinned result buffer returned through ppOutput */
#define CUDA_DLL_INITIALIZE (-2)   /* floats {deviceId, flags} -> out[0] = kernel index */
#define CUDA_DLL_CLEANUP (-3)
/* inc/FunctionIDs.h:71-95,126-127,222-226,532-535 */
#define CUDA_FN_SETDEVICE 1
#define CUDA_FN_SYNCHRONIZEDEVICE 5
#define CUDA_FN_ALLOCMEM 20        /* longs {count[,hStream]}; optional floats {count[,pad], data...} to initialise -> out[0] = handle (device.cu:854-899) */
#define CUDA_FN_FREEMEM 21         /* longs {h} */
#define CUDA_FN_GETMEM 22          /* longs {h[,count]} -> floats (device.cu:973-1026) */
#define CUDA_FN_SETMEM 23          /* longs {h,count}, floats {h,count,data...} (device.cu:1029) */
#define CUDNN_FN_CREATE_CUDNN 47   /* -> out[0] = hCuDnn (passed through by ATTN_*) */
#define CUDNN_FN_FREE_CUDNN 48
#define CUDA_FN_CREATE_EXTENSION 67 /* DLL_InvokeFloatEx, string = path of the extension library ("" = this library's own
                                       llama2 extension) -> out[0] = hExtension          (device.h:4498-4524) */
#define CUDA_FN_FREE_EXTENSION 68   /* floats {hExtension}                               (device.h:4556-4566) */
#define CUDA_FN_EXTENSION_RUN 69    /* floats {hExtension, extensionFn, args...}; through DLL_InvokeFloatEx the string
                                       goes to the extension's ...Ex entry             (device.h:4570-4588, CudaDnnDLL.cpp:1053-1064) */
#define CUDNN_FN_ATTN_CREATE 160   /* -> out[0] = hAttn                      (device.h:2435-2448) */
#define CUDNN_FN_ATTN_FREE 161     /* floats {hAttn}                          (device.h:2450-2461) */
#define CUDNN_FN_ATTN_SET 162      /* floats {dropout}; longs {hCuDnn,hAttn,gpuId,bTraining,B,blockSize,H,D,seed}
                                      (device.h:2463-2486) + optional 10th long: MCA_DTYPE_*, 11th: MCA_FLAG_* */
#define CUDNN_FN_ATTN_FWD 163      /* longs {hCuDnn,hAttn,T,hQ,hK,hV,hMask,hY,bBatchMask}   (device.h:2488-2506) */
#define CUDNN_FN_ATTN_BWD 164      /* longs {hCuDnn,hAttn,hQ,hdQ,hK,hdK,hV,hdV,hMask,hY,hdY} (device.h:2508-2529) */
#define CUDA_FN_CREATE_LAYERNORM 970 /* floats {eps}; longs {gpuId,count,outerNum,channels,innerNum} -> hLayerNorm (device.h:4123-4147) */
#define CUDA_FN_FREE_LAYERNORM 971   /* floats {hLayerNorm}                                  (device.h:4150-4160) */
#define CUDA_FN_LAYERNORM_FWD 975    /* longs {hLayerNorm,hXdata,hYdata}                     (device.h:4163-4178) */
#define CUDA_FN_LAYERNORM_BWD 976    /* longs {hLayerNorm,hYdata,hYdiff,hXdiff}              (CudaDnn.cs:6354-6360) */
#define CUDA_FN_CREATE_ROPE 980    /* floats {theta}; longs {sharedIdx,gpuId,count,B,T,H,D} -> hRope (device.h:4200-4228) */
#define CUDA_FN_FREE_ROPE 981      /* floats {hRope} */
#define CUDA_FN_ROPE_FWD 982       /* longs {hRope,n,hX,hY[,freqOffset]}      (device.h:4243-4265) */
#define CUDA_FN_ROPE_BWD 983       /* longs {hRope,n,hX,hYdiff,hXdiff}        (device.h:4267-4283) */
/* ids of DLL_QueryString / DLL_QueryStringFloatEx (Cuda Files/main.h:37-40) */
#define CUDA_FN_GET_DEVICE_NAME 1000      /* longs {deviceId} -> "<name> (<GB> GB - P2P on|off; compute M.m)" (device.cu:528-554) */
#define CUDA_FN_GET_EXTENSION_STRING 1003 /* DLL_QueryStringFloatEx: longs {hExtension, extensionFn, args...} -> extension's string */
/* Ids added by this library (no counterpart in the reference; above its highest id). */
#define MCA_FN_ALLOCMEM_BF16 2001  /* longs {count} -> handle to bf16 storage; SETMEM/GETMEM convert from/to float */
#define MCA_FN_CONVERT 2002        /* longs {hSrc,hDst,count}: copy with float<->bf16 conversion as the handles require */
#define MCA_FN_ATTN_FWD_HOST 2003  /* longs {pQ,pK,pV,pY (host addresses),hostDtype,causal,B,H,T,D[,headsPerChunk]}: mca_sdpa_forward_host */
#define MCA_FN_ATTN_FWD_PACKED 2004  /* longs {hCuDnn,hAttn,T,hQKV,hMask,hY,bBatchMask}: ATTN_FWD reading q,k,v from the (B,T,3C) c_attn output, y as (B,T,C) */
#define MCA_FN_ATTN_BWD_PACKED 2005  /* longs {hCuDnn,hAttn,hQKV,hdQKV,hMask,hY,hdY}: its backward; dQKV (B,T,3C) from dY (B,T,C) */
#define MCA_FN_DECODE_CREATE 2010  /* floats {theta}; longs {B,nHeads,nKvHeads,headSize,seqLen,cacheBf16} -> hDecode.
                                      theta <= 0: no RoPE -- the KV-cache step of MultiheadAttentionLayer.cs:713-777 for B sequences */
#define MCA_FN_DECODE_FREE 2011    /* floats {hDecode} */
#define MCA_FN_DECODE_STEP 2012    /* longs {hDecode,hQ,hKnew,hVnew,hKcache,hVcache,hPos,maxLen,hOut}: one token for B sequences */
#define MCA_FN_DECODE_QKV 2013     /* floats {eps}; longs {hX,hRmsW,hWq,hWk,hWv,B,dim,kvDim,hQ,hK,hV}: RMSNorm + q,k,v projections */
#define MCA_FN_DECODE_OUT 2014     /* longs {hAttn,hWo,B,dim,hX}: x += Wo . attn */
#define MCA_FN_DECODE_FFN 2015     /* floats {eps}; longs {hX,hRmsW,hW1,hW2,hW3,B,dim,hiddenDim,hHidden}: x += W2 (silu(W1 xn) o W3 xn) */
#define MCA_FN_DECODE_LOGITS 2016  /* floats {eps}; longs {hX,hRmsW,hWcls,B,dim,vocab,hLogits}: final RMSNorm + classifier */
#define MCA_FN_TFT_ATTN_FWD 2020   /* longs {hQ,hK,hV,hMask,B,H,Nq,Nk,d,hOut,hAttn} */
#define MCA_FN_TFT_ATTN_BWD 2021   /* longs {hQ,hK,hV,hMask,hdOut,hdAttn,B,H,Nq,Nk,d,hdQ,hdK,hdV} (hMask, hdAttn may be 0) */
#define MCA_FN_RMSNORM_FWD 2040    /* floats {eps}; longs {hX,hW (0: none),hY,hInvRms,rows,inner}: RMSNormLayer forward in one pass */
#define MCA_FN_RMSNORM_BWD 2041    /* longs {hX,hW,hdY,hInvRms,hdX,hdW (0: frozen),rows,inner}: its backward */
#define MCA_FN_SET_ASYNC 2030      /* longs {0|1}: 1 = do not synchronise the stream after each call (default 0, as the reference) */
#define MCA_FN_SET_TIMING 2031     /* longs {0|1}: 1 = bracket every dispatched call with CUDA events (read with MCA_FN_QUERY_COUNTERS) */
#define MCA_FN_WAIT_PROBE 2032     /* longs {hAttn, limitMicroseconds}: runs mca_wait_probe on the handle's status words, then reports
                                      them as a tensor-core launch would (ERROR_ATTN_KERNEL_TIMEOUT); a self-check, no tensor work */
#define MCA_FN_QUERY_VERSION 2050  /* DLL_QueryString: the text of mca_version() */
#define MCA_FN_QUERY_COUNTERS 2051 /* DLL_QueryString: one line per function id used on this kernel index:
                                      "<id> calls=<n> errors=<n> gpu_ms_last=<t> gpu_ms_total=<t>" (times only while timing is on) */

/* Function ids of the llama2 extension (CudaExtension.llm32.llama2/CudaExtension.llm32.cpp:20-26). */
#define LLM_CUDA_EXTENSION_CREATE 1        /* floats {temperature, top-p, seed} (all optional) -> out[0] = hLlm */
#define LLM_CUDA_EXTENSION_DESTROY 2       /* floats {hLlm} */
#define LLM_CUDA_EXTENSION_LOAD 3          /* Ex: floats {hLlm}, string "model.bin;tokenizer.bin" (the tokenizer part is not read) */
#define LLM_CUDA_EXTENSION_QUERYSTATUS 4   /* floats {hLlm} -> {fraction loaded, status (1 = loaded)} */
#define LLM_CUDA_EXTENSION_GENERATE 5      /* not provided: tokenizer and sampler are outside this library */
#define LLM_CUDA_EXTENSION_QUERYRESPONSE 6 /* not provided */
#define LLM_CUDA_EXTENSION_ABORT 7         /* floats {hLlm}: sets the cancel flag */
#define MCA_LLM_EXTENSION_FORWARD 100      /* added: floats {hLlm, token, pos} -> logits (vocab_size floats): one
                                              TransformerGpu::forward(token, pos), llama2_gpu.cpp:32-111 */

/* 10th long of ATTN_SET */
#define MCA_DTYPE_F32 0   /* fp32 tensors at fp32 accuracy (default; what the reference computes): the forward runs on the tensor
                             cores with every operand carried as two fp16 halves (head sizes 16, 32, 64; causal or no mask),
                             otherwise, and always for the backward, exact fp32 arithmetic on CUDA cores */
#define MCA_DTYPE_TF32 1  /* fp32 tensors, tcgen05 kind::tf32 products with fp32 accumulation */
#define MCA_DTYPE_BF16 2  /* bf16 tensors (handles from MCA_FN_ALLOCMEM_BF16), tcgen05 kind::f16 */
/* 11th long of ATTN_SET */
#define MCA_FLAG_CAUSAL_IMPLICIT 1  /* hMask is ignored and the mask is the analytic lower triangle */
#define MCA_FLAG_EXACT_FP32 2       /* MCA_DTYPE_F32 handles: never use the split-operand tensor-core forward */

/* mask_mode of the raw entry points */
#define MCA_MASK_MODE_NONE 0
#define MCA_MASK_MODE_TT 1      /* (T,T) floats, masked where 0 */
#define MCA_MASK_MODE_BATCH 2   /* (B,T) floats key mask, masked where 0 */
#define MCA_MASK_MODE_CAUSAL 3  /* analytic lower triangle, mask pointer unused */

/* tensor layout of the *_layout entry points */
#define MCA_LAYOUT_BHTD 0    /* q, k, v, y: separate contiguous (B,H,T,D) tensors (what attn.cu:535-556 expects) */
#define MCA_LAYOUT_PACKED 1  /* q, k, v: the three feature thirds of one (B,T,3*H*D) tensor (pass base, base + H*D,
                                base + 2*H*D); y, dy: (B,T,H*D).  The form the c_attn output has before
                                CausalSelfAttentionLayer splits and transposes it (CausalSelfAttentionLayer.cs:537-557)
                                and the form c_proj consumes (:604): no channel_copy, no head transposes */

/* handle types of Internal_GetPointer* (Cuda Files/memory.h HANDLE_TYPE) */
#define MCA_HT_MEMORY 1

/* ---- 1. reference dispatch ABI ---------------------------------------------------------- */

/* Replaces DLL_InvokeFloat, CudaDnnDLL/CudaDnnDLL.cpp:134-312. */
MCA_API MCA_LONG DLL_InvokeFloat(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, float* pInput, MCA_LONG lInput,
                                 float** ppOutput, MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG lszErrMax);
/* Replaces DLL_InvokeFloatEx2, CudaDnnDLL.cpp:314-493 (float + 64-bit integer inputs). */
MCA_API MCA_LONG DLL_InvokeFloatEx2(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, float* pInput, MCA_LONG lInput,
                                    MCA_LONGLONG* plInput, MCA_LONG llInput, float** ppOutput, MCA_LONG* plOutput,
                                    MCA_LPTSTR szErr, MCA_LONG lszErrMax);
/* Replaces DLL_InvokeFloatEx, CudaDnnDLL.cpp:495-672 (string input; no id on this path takes one). */
MCA_API MCA_LONG DLL_InvokeFloatEx(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, float* pInput, MCA_LONG lInput,
                                   MCA_LPTSTR pszInput, float** ppOutput, MCA_LONG* plOutput, MCA_LPTSTR szErr,
                                   MCA_LONG lszErrMax);
/* The double twins (CudaDnnDLL.cpp:674-853 and following).  The attention path of this
 * library computes in fp32/tf32/bf16 only: every id returns ERROR_NOT_IMPLEMENTED (90009). */
MCA_API MCA_LONG DLL_InvokeDouble(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, double* pInput, MCA_LONG lInput,
                                  double** ppOutput, MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG lszErrMax);
MCA_API MCA_LONG DLL_InvokeDoubleEx2(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, double* pInput, MCA_LONG lInput,
                                     MCA_LONGLONG* plInput, MCA_LONG llInput, double** ppOutput,
                                     MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG lszErrMax);
/* Replaces DLL_InvokeDoubleEx, CudaDnnDLL.cpp:1090-1160 (ordinal 5): ERROR_NOT_IMPLEMENTED as the other double entries. */
MCA_API MCA_LONG DLL_InvokeDoubleEx(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, double* pInput, MCA_LONG lInput,
                                    MCA_LPTSTR pszInput, double** ppOutput, MCA_LONG* plOutput, MCA_LPTSTR szErr,
                                    MCA_LONG lszErrMax);
/* Replaces DLL_QueryString, CudaDnnDLL.cpp:855-933 (ordinal 3).  pInput are 32-bit LONGs.  The answer is a
 * malloc'ed string returned through *ppOutput; the caller hands it back with lFunctionIdx = CUDA_DLL_FREEMEM.
 * Ids: CUDA_FN_GET_DEVICE_NAME, MCA_FN_QUERY_VERSION, MCA_FN_QUERY_COUNTERS; others ERROR_PARAM_OUT_OF_RANGE
 * (what Kernel<T>::Query answers for an id it does not know, Cuda Files/main.cu:2457-2478). */
MCA_API MCA_LONG DLL_QueryString(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, MCA_LONG* pInput, MCA_LONG lInput,
                                 MCA_LPTSTR* ppOutput, MCA_LPTSTR szErr, MCA_LONG lszErrMax);
/* Replace DLL_QueryStringFloatEx / DLL_QueryStringDoubleEx, CudaDnnDLL.cpp:935-1015: the answer is written into the
 * caller's buffer.  Id CUDA_FN_GET_EXTENSION_STRING forwards to the extension's ...Ex entry and appends "\n[END]"
 * when the extension reports the end of its text (extension.cu:153-180).  The double form returns ERROR_NOT_IMPLEMENTED. */
MCA_API MCA_LONG DLL_QueryStringFloatEx(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, MCA_LONG* pInput, MCA_LONG lInput,
                                        MCA_LPTSTR pszOutput, MCA_LONG lOutputMax, MCA_LPTSTR szErr, MCA_LONG lszErrMax);
MCA_API MCA_LONG DLL_QueryStringDoubleEx(MCA_LONG lKernelIdx, MCA_LONG lFunctionIdx, MCA_LONG* pInput, MCA_LONG lInput,
                                         MCA_LPTSTR pszOutput, MCA_LONG lOutputMax, MCA_LPTSTR szErr, MCA_LONG lszErrMax);
/* Replaces Internal_GetPointerFloat, CudaDnnDLL.cpp:57-73: raw device pointer behind a memory handle. */
MCA_API MCA_LONG Internal_GetPointerFloat(MCA_LONG ht, MCA_LONG lKernelIdx, MCA_LONG hHandle, void** ppPtr);
/* Replaces Internal_AllocHostFloat, CudaDnnDLL.cpp:93-109: pinned host buffer, optionally filled from pSrc. */
MCA_API MCA_LONG Internal_AllocHostFloat(MCA_LONG lKernelIdx, MCA_LONG lCount, float** ppDst, float* pSrc,
                                         bool bSrcOnDevice);
/* Replace Internal_GetPointerDouble / Internal_AllocHostDouble, CudaDnnDLL.cpp:75-91,111-127 (ordinals 101, 103).  No
 * double kernel can exist here (INITIALIZE through DLL_InvokeDouble is refused), so both answer ERROR_PARAM_NULL --
 * the reference's answer for a slot of its double table that holds no kernel. */
MCA_API MCA_LONG Internal_GetPointerDouble(MCA_LONG ht, MCA_LONG lKernelIdx, MCA_LONG hHandle, void** ppPtr);
MCA_API MCA_LONG Internal_AllocHostDouble(MCA_LONG lKernelIdx, MCA_LONG lCount, double** ppDst, double* pSrc,
                                          bool bSrcOnDevice);

/* ---- 1b. extension ABI of the llama2 route ------------------------------------------------ */
/* What a parent CudaDnnDLL resolves in an extension library after LoadLibrary (Cuda Files/extension.cu:18-83,
 * extension.h:20-38).  This library is such an extension: it replaces CudaExtension.llm32.llama2
 * (CudaExtension.llm32.cpp:67-83 init, :91-205 invoke, :213-268 invoke-ex) for loading a llama2 'ak42' checkpoint and
 * running TransformerGpu::forward on it; text generation (tokenizer, sampler) is not part of it.
 * hParent: module handle of the parent (a dlopen handle here; HMODULE on Windows); the extension resolves
 * DLL_InvokeFloat and Internal_AllocHostFloat in it and returns 87 (ERROR_INVALID_PARAMETER) when either is missing.
 * Results are returned in buffers from the parent's Internal_AllocHostFloat, as the reference requires. */
MCA_API MCA_LONG DLL_InitFloatCustomExtension(void* hParent, MCA_LONG lKernelIdx);
MCA_API MCA_LONG DLL_InvokeFloatCustomExtension(MCA_LONG lfnIdx, float* pInput, MCA_LONG lInput, float** ppOutput,
                                                MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG lErrMax);
MCA_API MCA_LONG DLL_InvokeFloatCustomExtensionEx(MCA_LONG lfnIdx, float* pInput, MCA_LONG lInput, float** ppOutput,
                                                  MCA_LONG* plOutput, MCA_LPTSTR szInput, MCA_LPTSTR szOutput,
                                                  MCA_LONG lOutputMax, MCA_LPTSTR szErr, MCA_LONG lErrMax);
/* The double forms (CudaExtension.llm32.cpp:275-490): ERROR_NOT_IMPLEMENTED. */
MCA_API MCA_LONG DLL_InitDoubleCustomExtension(void* hParent, MCA_LONG lKernelIdx);
MCA_API MCA_LONG DLL_InvokeDoubleCustomExtension(MCA_LONG lfnIdx, double* pInput, MCA_LONG lInput, double** ppOutput,
                                                 MCA_LONG* plOutput, MCA_LPTSTR szErr, MCA_LONG lErrMax);
MCA_API MCA_LONG DLL_InvokeDoubleCustomExtensionEx(MCA_LONG lfnIdx, double* pInput, MCA_LONG lInput, double** ppOutput,
                                                   MCA_LONG* plOutput, MCA_LPTSTR szInput, MCA_LPTSTR szOutput,
                                                   MCA_LONG lOutputMax, MCA_LPTSTR szErr, MCA_LONG lErrMax);

/* ---- 2. raw entry points ------------------------------------------------------------------ */
/* All tensors are contiguous row-major device memory; `stream` is a cudaStream_t (0 = default). */

/* fp32 SDPA forward, exact fp32 arithmetic.  Replaces attnHandle<T>::Forward,
 * CudaDnnDLL/Cuda Files/attn.cu:518-602.  q,k,v,y: (B,H,T,D), D <= 128.  causal_flag: optional device
 * int written by mca_classify_causal_mask; when it holds 1 a MASK_MODE_TT mask is treated as causal.
 * row_max,row_sum: optional (B,H,T) softmax statistics kept for the backward; y_copy: optional
 * second copy of y kept for the backward. */
MCA_API int mca_sdpa_forward_f32(const float* q, const float* k, const float* v, const float* mask, int mask_mode,
                                 const int* causal_flag, int B, int H, int T, int D, float* y, float* row_max,
                                 float* row_sum, float* y_copy, void* stream);
/* fp32 SDPA backward.  Replaces attnHandle<T>::Backward, attn.cu:608-661.  Recomputes the
 * probabilities from row_max/row_sum instead of reading a saved (B,H,T,T) tensor.
 * delta_scratch: (B,H,T) floats of scratch. */
MCA_API int mca_sdpa_backward_f32(const float* q, const float* k, const float* v, const float* dy,
                                  const float* y_saved, const float* mask, int mask_mode, const int* causal_flag,
                                  const float* row_max, const float* row_sum, float* delta_scratch, int B, int H,
                                  int T, int D, float* dq, float* dk, float* dv, void* stream);
/* The same two with a tensor layout (MCA_LAYOUT_*): with MCA_LAYOUT_PACKED the kernels read q, k, v
 * straight out of the (B,T,3C) projection output and write y as (B,T,C); in the backward dy is
 * (B,T,C) and dq, dk, dv are the thirds of a (B,T,3C) gradient.  Replaces, besides attn.cu:518-661,
 * the three channel_copy calls and four head transposes either side of it
 * (CausalSelfAttentionLayer.cs:537-557,604,666,719-737).  y_copy, y_saved and the row statistics
 * stay (B,H,T,*) contiguous (they belong to the handle). */
MCA_API int mca_sdpa_forward_f32_layout(const float* q, const float* k, const float* v, const float* mask,
                                        int mask_mode, const int* causal_flag, int B, int H, int T, int D, float* y,
                                        float* row_max, float* row_sum, float* y_copy, int layout, void* stream);
MCA_API int mca_sdpa_backward_f32_layout(const float* q, const float* k, const float* v, const float* dy,
                                         const float* y_saved, const float* mask, int mask_mode,
                                         const int* causal_flag, const float* row_max, const float* row_sum,
                                         float* delta_scratch, int B, int H, int T, int D, float* dq, float* dk,
                                         float* dv, int layout, void* stream);
/* Writes 1 to *flag iff mask (T,T) equals the lower-triangular ones built by fillMask,
 * MyCaffe.layers.gpt/layers.gpt/CausalSelfAttentionLayer.cs:276-291; else 0. */
MCA_API int mca_classify_causal_mask(const float* mask, int T, int* flag, void* stream);

/* The reference's other mask forms on the tensor-core kernels.  A (T,T) mask (apply_mask, attn.cu:302-311 with
 * bBatchMask false: masked where 0) or a (B,T) key mask (bBatchMask true, what MultiheadAttentionLayer.cs:698-702
 * passes) is first packed into keep-bits by mca_mask_pack: `bits` holds rows x mca_mask_bits_row_words(T) words (rows = T
 * or B), `bits_t` (a (T,T) mask only; the backward reads it) the same for the transposed mask; both 16-byte aligned.
 * The *_masked entry points then take (bits, [bits_t,] mask_mode) with mask_mode MCA_MASK_MODE_TT or
 * MCA_MASK_MODE_BATCH and causal = 0; with MCA_MASK_MODE_NONE and null pointers they are the unmasked calls.
 * Semantics as the reference: a masked logit is a finite value far below every real one, so a row whose every key is
 * masked comes out uniform (its lse is written as +inf, which is how the backward recognises it). */
MCA_API int mca_mask_bits_row_words(int T);
MCA_API int mca_mask_pack(const float* mask, int mask_mode, int B, int T, uint32_t* bits, uint32_t* bits_t, void* stream);

/* Tensor-core SDPA forward (tcgen05 + TMEM + TMA).  Same math as attn.cu:518-602 with a causal
 * or absent mask.  dtype: MCA_DTYPE_BF16 (q,k,v,y bf16) or MCA_DTYPE_TF32 (q,k,v,y fp32).
 * D in {64,128}; lse: optional (B,H,T) floats, log2-domain log-sum-exp kept for the backward.
 * status: device int[4] the kernel writes when a bounded wait gives up (0 = ok). */
MCA_API int mca_sdpa_forward_tc(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H,
                                int T, int D, void* y, float* lse, int* status, void* stream);
/* Sequences of up to this many keys (half as many with split fp32 operands) run the forward as CTAs of one 128-row
 * query tile, two to an SM, instead of one CTA of two tiles: the fixed part of a CTA's life then overlaps its neighbour's
 * key loop.  64-wide bf16 heads take that shape at every length unless the value is 0.  len < 0
 * only reads; returns the value before the call (default 8192, or MCA_TC_NARROW_LEN from the environment; 0 = never).
 * A tuning knob of this library with no counterpart in the reference; set it before the first call from other threads. */
MCA_API int mca_tc_narrow_len(int len);

/* fp32 SDPA forward at fp32 accuracy on the tensor cores.  Same math as attn.cu:518-602 with a causal or absent mask.
 * q, k, v, y: fp32, (B,H,T,D) or the packed layout; D in {16, 32, 64, 128} (128: one query tile per CTA and
 * single-stage K and V, since a row's two halves are 512 bytes; forward only, the exact fp32 backward follows it from
 * row_max / row_sum).  A pre-pass scales each tensor by a power of two
 * and writes every element as two fp16 halves hi = fp16(x), lo = fp16(x - hi) into `workspace`
 * (mca_sdpa_forward_f32_tc_workspace_bytes_d(B,H,T,D) bytes, 16-byte aligned); every contraction is then three
 * tcgen05 kind::f16 products hi.hi + hi.lo + lo.hi accumulated in fp32, P split the same way.  Within 1e-5 of the output
 * scale of the fp64 result (measured 1e-7 .. 7e-6).  row_max, row_sum (optional, (B,H,T)) and y_copy (optional, (B,H,T,D) contiguous) are what
 * mca_sdpa_backward_f32 needs; lse (optional, (B,H,T), log2 domain) and y_copy are what mca_sdpa_backward_f32_tc needs.
 * status as mca_sdpa_forward_tc. */
MCA_API int64_t mca_sdpa_forward_f32_tc_workspace_bytes(int B, int H, int T);           /* head sizes up to 64 */
MCA_API int64_t mca_sdpa_forward_f32_tc_workspace_bytes_d(int B, int H, int T, int D);  /* any supported head size */
MCA_API int mca_sdpa_forward_f32_tc_supported(int D);    /* 16, 32, 64, 128 */
MCA_API int mca_sdpa_backward_f32_tc_supported(int D);   /* 16, 32, 64 */
MCA_API int mca_sdpa_forward_f32_tc(const float* q, const float* k, const float* v, int causal, int B, int H, int T, int D,
                                    float* y, float* row_max, float* row_sum, float* y_copy, float* lse, void* workspace,
                                    int64_t workspace_bytes, int* status, int layout, void* stream);
MCA_API int mca_sdpa_forward_f32_tc_masked(const float* q, const float* k, const float* v, int causal, int B, int H, int T,
                                           int D, float* y, float* row_max, float* row_sum, float* y_copy, float* lse,
                                           void* workspace, int64_t workspace_bytes, int* status, int layout,
                                           const uint32_t* mask_bits, int mask_mode, void* stream);
/* Its backward (attnHandle<T>::Backward, attn.cu:608-661) on the tensor cores with the same split operands: `workspace`
 * must still hold what mca_sdpa_forward_f32_tc left in it for the same q, k, v (their fp16 halves and scales); dY is split
 * here.  dy in the output layout, y_copy and lse from the forward; dq, dk, dv fp32 in the input layout;
 * delta_scratch: (B,H,T) floats.  Deterministic (no atomics). */
MCA_API int mca_sdpa_backward_f32_tc(const float* dy, const float* y_copy, const float* lse, float* delta_scratch, int causal,
                                     int B, int H, int T, int D, float* dq, float* dk, float* dv, void* workspace,
                                     int64_t workspace_bytes, int* status, int layout, void* stream);
MCA_API int mca_sdpa_backward_f32_tc_masked(const float* dy, const float* y_copy, const float* lse, float* delta_scratch,
                                            int causal, int B, int H, int T, int D, float* dq, float* dk, float* dv,
                                            void* workspace, int64_t workspace_bytes, int* status, int layout,
                                            const uint32_t* mask_bits, const uint32_t* mask_bits_t, int mask_mode,
                                            void* stream);

/* Self-check of the bounded waits inside the tensor-core kernels: launches one small kernel whose only thread waits
 * on a barrier nothing arrives on, for at most limit_us microseconds (<= 100000), then gives up the way a stalled
 * pipeline stage would: status[0] = 1, status[1] = 99, and the kernel returns.  Nothing hangs, traps or faults.
 * status: device int[4], zeroed by the caller. */
MCA_API int mca_wait_probe(int* status, int limit_us, void* stream);

/* Tensor-core SDPA backward (bf16).  Same math as attnHandle<T>::Backward, attn.cu:608-661, with a
 * causal or absent mask; P is recomputed from `lse` (written by mca_sdpa_forward_tc on the same
 * inputs) instead of read from a saved (B,H,T,T) tensor.  q,k,v,y,dy,dq,dk,dv: (B,H,T,D) bf16,
 * D in {64,128}; delta_scratch: (B,H,T) floats of scratch; status as in the forward.  The gradients must not
 * overlap the inputs (the reference's diff blobs never do): the dQ kernel runs under the tail of the dK/dV kernel. */
MCA_API int mca_sdpa_backward_tc(const void* q, const void* k, const void* v, const void* y, const void* dy,
                                 const float* lse, float* delta_scratch, int dtype, int causal, int B, int H,
                                 int T, int D, void* dq, void* dk, void* dv, int* status, void* stream);

/* Tensor-core SDPA forward for tensors in HOST memory.  Replaces the reference's host round trip
 * SetMemory x3 -> AttnScaledDotProductForward -> GetMemory (CudaDnn.cs:2946,3027,5673-5679; the
 * copies are blocking cudaMemcpy calls, Cuda Files/memory.cu:451,539, and attn.cu:601 synchronises), whose time is the sum of
 * its parts: here chunks of consecutive (batch, head) pairs flow through three streams so that
 * the PCIe copies in both directions overlap the kernel.  q,k,v,y: host (B,H,T,D), fp32
 * (host_dtype MCA_DTYPE_F32; converted to bf16 on the device) or bf16 (MCA_DTYPE_BF16); pinned
 * memory is needed for overlap.  D in {64,128}; causal or no mask; arithmetic as
 * mca_sdpa_forward_tc in bf16.  heads_per_chunk 0 = chosen by mca_host_pipeline_chunk.
 * Returns when y is complete.  Device staging is owned by the library and grows on demand. */
MCA_API int mca_sdpa_forward_host(const void* q, const void* k, const void* v, void* y, int host_dtype, int causal,
                                  int B, int H, int T, int D, int heads_per_chunk);
/* (batch, head) pairs per chunk the pipeline uses (host arithmetic, no device call). */
MCA_API int mca_host_pipeline_chunk(int B, int H, int T, int heads_per_chunk);
/* Free the pipeline's device staging buffers on the current device. */
MCA_API int mca_host_pipeline_release(void);

/* The tensor-core pair with a tensor layout (MCA_LAYOUT_*), as mca_sdpa_forward_f32_layout: the 4-D
 * tensor maps read q, k, v out of the (B,T,3C) projection output; y, dy are (B,T,C); dq, dk, dv are
 * the thirds of a (B,T,3C) gradient.  `y` of the backward has the layout the forward wrote it in. */
MCA_API int mca_sdpa_forward_tc_layout(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H,
                                       int T, int D, void* y, float* lse, int* status, int layout, void* stream);
MCA_API int mca_sdpa_forward_tc_masked(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H,
                                       int T, int D, void* y, float* lse, int* status, int layout,
                                       const uint32_t* mask_bits, int mask_mode, void* stream);
/* As mca_sdpa_forward_tc_masked, and a second copy of the output, same layout, to y_keep (null: none): what a training
 * handle keeps for its Backward (the reference keeps the probabilities, attn.cu:436-452), written by the kernel's own
 * epilogue instead of a device-to-device copy afterwards.  bf16 only. */
MCA_API int mca_sdpa_forward_tc_keep(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H, int T,
                                     int D, void* y, void* y_keep, float* lse, int* status, int layout,
                                     const uint32_t* mask_bits, int mask_mode, void* stream);
MCA_API int mca_sdpa_backward_tc_layout(const void* q, const void* k, const void* v, const void* y, const void* dy,
                                        const float* lse, float* delta_scratch, int dtype, int causal, int B, int H,
                                        int T, int D, void* dq, void* dk, void* dv, int* status, int layout,
                                        void* stream);
MCA_API int mca_sdpa_backward_tc_masked(const void* q, const void* k, const void* v, const void* y, const void* dy,
                                        const float* lse, float* delta_scratch, int dtype, int causal, int B, int H,
                                        int T, int D, void* dq, void* dk, void* dv, int* status, int layout,
                                        const uint32_t* mask_bits, const uint32_t* mask_bits_t, int mask_mode,
                                        void* stream);

/* Head-parallel forward whose epilogue is also the exchange: every finished 16-byte piece of the output
 * tile is stored to each of the n_dst (<= 8) destinations -- this GPU's buffer and the peers' buffers
 * mapped into this process (plain stores over NVLink; no collective follows, only a barrier before
 * the buffers are read).  q,k,v: this rank's heads, (B,H,T,D) bf16 contiguous; y_dst[i]: where this
 * rank's head 0 lies in destination i, with the element strides of the full (B,H_total,T,D) output.
 * No reference counterpart (the reference has no tensor-parallel mode, MyCaffe/common/Parallel.cs:351-508). */
MCA_API int mca_sdpa_forward_tc_scatter(const void* q, const void* k, const void* v, int dtype, int causal, int B, int H,
                                        int T, int D, void* const* y_dst, int n_dst, int64_t y_stride_b,
                                        int64_t y_stride_h, int64_t y_stride_t, float* lse, int* status, void* stream);

/* RoPE on a (B,T,H,D) tensor.  Replaces RopeDataGpu<T>::Forward/Backward, Cuda Files/rope.cu:784-864.
 * Tables are (T,D/2) as built by mca_rope_tables_host. */
MCA_API int mca_rope_f32(const float* x, float* y, int64_t n, int T, int H, int D, const float* cos_table,
                         const float* sin_table, int freq_offset, int backward, void* stream);
/* Host-side table construction, rope.cu:501-553 (powf/cosf/sinf in fp32). */
MCA_API int mca_rope_tables_host(int T, int D, float theta, float* cos_table, float* sin_table);

/* Split-KV decode attention for one new token of B independent sequences.  Replaces
 * Primitives::rope + the cache append + Primitives::attention of TransformerGpu::forward,
 * CudaExtension.llm32.llama2/Files/llama2_gpu.cpp:64-75 (kernels primitives.cu:99-202).
 * q: (B, n_heads*hs) and k_new,v_new: (B, n_kv_heads*hs) are the projections of the new token
 * before RoPE; caches are (B, seq_len, n_kv_heads*hs) fp32 or bf16 with cache_batch_stride
 * elements between sequences; row pos[b] is written, rows 0..pos[b] are attended.  max_len
 * must be >= max_b pos[b]+1.  freq_real/imag: (seq_len, hs/2) or both null (no RoPE, q/k already
 * rotated).  k_new = v_new = null skips the append.  scratch: floats from mca_decode_plan.
 * head_size: 32, 48, 64, 96 or 128 (the reference kernel takes any, primitives.cu:158-202; llama2.c's models use
 * 48, 64 and 128).  Caches must be 16-byte aligned with cache_batch_stride a multiple of 4 (fp32) or 8 (bf16)
 * elements.  A sequence whose pos[b] lies outside [0, max_len) is not followed out of the cache: nothing of it is
 * read or appended, its output row is zero, and mca_decode_status reports it. */
MCA_API int mca_decode_plan(int B, int n_heads, int n_kv_heads, int head_size, int max_len, int* split_len,
                            int* nsplit, int64_t* scratch_floats);
MCA_API int mca_decode_attention(const float* q, const float* k_new, const float* v_new, void* k_cache,
                                 void* v_cache, int cache_is_bf16, int64_t cache_batch_stride, const int* pos,
                                 int B, int n_heads, int n_kv_heads, int head_size, int seq_len, int max_len,
                                 const float* freq_real, const float* freq_imag, float* scratch,
                                 int64_t scratch_floats, float* out, void* stream);
/* 1 if mca_decode_attention has a kernel for this head size. */
MCA_API int mca_decode_head_size_supported(int head_size);
/* Reads and clears the decode kernels' status words on the current device (blocking; call after the stream has been
 * synchronised): status3[0] = number of sequences refused for an out-of-range position since the last call,
 * status3[1] = the first such sequence, status3[2] = its position. */
MCA_API int mca_decode_status(int* status3);

/* Exchange of the decode head outputs between the GPUs that share the heads (one process per GPU), replacing an
 * all-gather per layer-step.  No reference counterpart (the reference decodes on one GPU).  Rank `rank` of n stores its
 * (B, dim_local) slice at column col0 of the (B, dim_total) buffer of every rank (dst[i]: peer memory mapped into this
 * process, this rank's own buffer included; plain stores over NVLink), raises entry `rank` of every rank's flag array
 * (flag_dst[i], int[8]) to `generation`, and waits until every entry of its own array (flag_local) has reached
 * `generation`: when the kernel has finished, this rank's buffer is complete.  Generations grow by one per exchange;
 * alternate between two buffers (a rank may still read exchange g while its peers already store exchange g + 1).
 * counter: a device int, zero before the first call.  The wait is bounded by limit_ms (<= 10000): on expiry the kernel
 * returns with status[0] = 3, status[1] = the rank it waited for, status[2] = that rank's flag. */
MCA_API int mca_decode_exchange(const float* src, float* const* dst, int* const* flag_dst, const int* flag_local,
                                int* counter, int* status, int n, int rank, int B, int dim_local, int dim_total, int col0,
                                int generation, int limit_ms, void* stream);

/* The projections around the decode attention, each fused with its neighbour and bound by the
 * one pass over the weights.  Replace Primitives::rmsnorm + three Primitives::matmul (cublasSgemv)
 * calls, and the Wo matmul + residual add, of TransformerGpu::forward,
 * CudaExtension.llm32.llama2/Files/llama2_gpu.cpp:56-61,78-81 (kernels primitives.cu:281-340).
 * Weights are (out, in) row-major as in the llama2 checkpoint (primitives.cu:322-332), fp32 or bf16;
 * x: (B, dim); dim must be a multiple of 8.
 *   q,k,v = [Wq;Wk;Wv] . (rms_weight o x / sqrt(mean(x^2) + eps));   x_inout += Wo . attn        */
MCA_API int mca_decode_qkv_rmsnorm(const float* x, const float* rms_weight, float eps, const void* wq,
                                   const void* wk, const void* wv, int weights_bf16, int B, int dim, int kv_dim,
                                   float* q_out, float* k_out, float* v_out, void* stream);
MCA_API int mca_decode_out_proj(const float* attn, const void* wo, int weights_bf16, int B, int dim, float* x_inout,
                                void* stream);

/* The feed-forward half of a llama2 layer for one new token of B sequences, in two launches.
 * Replaces rmsnorm, two matmul (cublasSgemv), siglu, matmul and add of TransformerGpu::forward,
 * llama2_gpu.cpp:84-97 (kernels primitives.cu:87-96,281-364); arithmetic as llama2_cpu.cpp:352-376:
 *   xn = rms_weight o x / sqrt(mean(x^2) + eps);  h = silu(W1 xn) o (W3 xn);  x_inout += W2 h.
 * w1, w3: (hidden_dim, dim); w2: (dim, hidden_dim); hidden_scratch: (B, hidden_dim) floats.
 * dim and hidden_dim must be multiples of 8 and at most 45568 (one sequence's activations are staged
 * in shared memory). */
MCA_API int mca_decode_ffn(const float* rms_weight, float eps, const void* w1, const void* w2, const void* w3,
                           int weights_bf16, int B, int dim, int hidden_dim, float* hidden_scratch, float* x_inout,
                           void* stream);
/* Final RMSNorm + classifier: logits (B, vocab_size) = Wcls . (rms_weight o x / sqrt(mean(x^2) + eps)).
 * Replaces llama2_gpu.cpp:101-105.  x is not modified (the reference normalises it in place). */
MCA_API int mca_decode_logits(const float* x, const float* rms_weight, float eps, const void* wcls, int weights_bf16,
                              int B, int dim, int vocab_size, float* logits, void* stream);

/* One decode step of the whole transformer, token -> logits, for B independent sequences.
 * Replaces TransformerGpu::forward(token, pos), llama2_gpu.cpp:32-111 (one sequence, about 16
 * launches per layer with host synchronisations) by 5-6 launches per layer on `stream` with no host
 * round trip; the call only enqueues work and may be captured into a CUDA graph.
 * McaLlamaConfig is the reference's Config (llama2_cpu.h:17-25).  Weights are laid out as the
 * checkpoint is (memory_map_weights, llama2_cpu.cpp:79-103): per-layer matrices stacked as
 * (n_layers, out, in); the matrices and wcls are fp32 or bf16 (weights_bf16), the embedding table
 * and the three norm weights fp32.  Caches are (n_layers, B, seq_len, kv_dim), fp32 or bf16;
 * freq_real/imag (seq_len, head_size/2) as mca_rope_tables_host builds them.  tokens, pos: device
 * int32 (B); row pos[b] of every layer's cache is written; max_len >= max_b pos[b] + 1.
 * workspace: mca_llama_workspace_floats(cfg, B, max_len) floats, 16-byte aligned (returns -1 for a
 * bad configuration).  head_size as mca_decode_attention. */
typedef struct McaLlamaConfig {
  int dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
} McaLlamaConfig;
typedef struct McaLlamaWeights {
  const float* token_embedding_table; /* (vocab_size, dim) */
  const float* rms_att_weight;        /* (n_layers, dim) */
  const float* rms_ffn_weight;        /* (n_layers, dim) */
  const float* rms_final_weight;      /* (dim) */
  const void *wq, *wk, *wv, *wo;      /* (n_layers, dim|kv_dim, dim), wo (n_layers, dim, dim) */
  const void *w1, *w2, *w3;           /* (n_layers, hidden_dim, dim), (n_layers, dim, hidden_dim), as w1 */
  const void* wcls;                   /* (vocab_size, dim) */
  int weights_bf16;
} McaLlamaWeights;
typedef struct McaLlamaState {
  void* key_cache;
  void* value_cache;
  int cache_is_bf16;
  const float* freq_real;
  const float* freq_imag;
  float* workspace;
  int64_t workspace_floats;
} McaLlamaState;
/* Decode projections for 9 to 64 sequences run one pass over the weights on the tensor cores (fp32 weights as fp16
 * hi/lo halves, three MMAs; bf16 weights directly) instead of one streaming pass per eight sequences; same results to
 * fp32 round-off.  No counterpart in the reference (it decodes one sequence with cublasSgemv,
 * CudaExtension.llm32.llama2/Files/primitives.cu:322-340).  The kernel keeps its activation pieces and partial sums
 * in arrays that are part of the library image, so two such products must not overlap on one device.
 * mca_proj_tc_enable(0) switches it off (the streaming kernel then serves every batch); returns the previous setting.
 * mca_proj_tc_status: the kernel's status words ([0] != 0: a bounded wait gave up; reading clears them). */
MCA_API int mca_proj_tc_enable(int on);
MCA_API int mca_proj_tc_status(int* status4);

MCA_API int64_t mca_llama_workspace_floats(const McaLlamaConfig* cfg, int B, int max_len);
MCA_API int mca_llama_forward(const McaLlamaConfig* cfg, const McaLlamaWeights* weights, const McaLlamaState* state,
                              const int* tokens, const int* pos, int B, int max_len, float* logits, void* stream);

/* Decode attention for callers that must not allocate device memory.  No counterpart in the
 * reference.  Some hosts cannot call cudaMalloc at the point where they decode -- a plug-in that is
 * only handed its inputs and outputs, or code running where the allocator must stay untouched -- so
 * this variant keeps the split-KV partials in an 8 MiB array that is part of the library image
 * (mca_decode_static_scratch_floats() floats; every GPU that loads the library holds it until
 * exit).  Same arguments and result as mca_decode_attention without the scratch pair.  It calls no
 * cudaMalloc, cudaFree or any other allocating routine.  The first call on each device looks up
 * the array's device address (cudaGetSymbolAddress, with that device current); make that first
 * call before any stream capture.  A problem whose partials do not fit (B * n_heads * nsplit *
 * (head_size + 2) floats, see mca_decode_plan) is refused with 90906.  All calls share the one
 * array and it keeps the previous call's contents: nothing in it needs clearing, but two calls
 * whose kernels overlap on the GPU (different streams or threads) race on it. */
MCA_API int64_t mca_decode_static_scratch_floats(void);
MCA_API int mca_decode_attention_static(const float* q, const float* k_new, const float* v_new, void* k_cache,
                                        void* v_cache, int cache_is_bf16, int64_t cache_batch_stride,
                                        const int* pos, int B, int n_heads, int n_kv_heads, int head_size,
                                        int seq_len, int max_len, const float* freq_real, const float* freq_imag,
                                        float* out, void* stream);

/* TFT interpretable attention forward.  Replaces the attention block of
 * MultiHeadAttentionInterpLayer<T>.forward, MyCaffe.layers.tft/layers.tft/
 * MultiHeadAttentionInterpLayer.cs:728-759.  q (B,H,Nq,d), k (B,H,Nk,d), v (B,Nk,d) shared by the
 * heads, mask (Nq,Nk) masked where 1 (or null) -> out (B,Nq,d) = mean_h P_h V, attn (B,Nq,Nk) = mean_h P_h. */
MCA_API int mca_tft_attention_forward_f32(const float* q, const float* k, const float* v, const float* mask, int B,
                                          int H, int Nq, int Nk, int d, float* out, float* attn, void* stream);

/* TFT interpretable attention backward.  Replaces the attention part of
 * MultiHeadAttentionInterpLayer<T>.backward, MultiHeadAttentionInterpLayer.cs:780-859.
 * d_out (B,Nq,d) and d_attn (B,Nq,Nk, may be null) are the gradients of the two outputs of the
 * forward; returns dq (B,H,Nq,d), dk (B,H,Nk,d), dv (B,Nk,d). */
MCA_API int mca_tft_attention_backward_f32(const float* q, const float* k, const float* v, const float* mask,
                                           const float* d_out, const float* d_attn, int B, int H, int Nq, int Nk,
                                           int d, float* dq, float* dk, float* dv, void* stream);

/* LayerNorm over rows of `inner` floats, one pass each way.  Replace LayerNormData<T>::Forward /
 * Backward, CudaDnnDLL/Cuda Files/layernorm.cu:291-333, :340-384 (10 and 9 kernels over seven
 * count-sized scratch tensors; no affine part, the C# layer applies it):
 *   y = (x - mean) / stdev,  stdev = sqrt(mean((x - mean)^2) + eps)        (stdev: `rows` floats, kept for backward)
 *   dx = (dy - (y * mean(y dy) + mean(dy))) / stdev
 * As the reference does (add_scalar over outer*channels items of its count-sized stdev tensor,
 * layernorm.cu:377), the divisor of the first `rows` elements of the flat tensor is stdev + eps.
 * inner <= 16384. */
MCA_API int mca_layernorm_forward_f32(const float* x, float* y, float* stdev, int64_t rows, int inner, float eps,
                                      void* stream);
MCA_API int mca_layernorm_backward_f32(const float* y, const float* dy, const float* stdev, float* dx, int64_t rows,
                                       int inner, float eps, void* stream);
/* RMSNorm layer, one pass each way.  Replace the 8 and 14 CudaDnn calls of RMSNormLayer<T>.forward /
 * backward, MyCaffe.layers.gpt/layers.gpt/RMSNormLayer.cs:156-179, :190-231:
 *   inv = 1 / sqrt(mean(x^2) + eps);  y = w o (x inv)                     (w may be null; inv_rms: `rows` floats or null)
 *   g = dy o w;  dx = g inv - x sum(g x) inv^3 / inner;  dw = sum over ALL rows of dy o (x inv)
 * (the reference's channel_sum writes outerNum*inner sums into the inner-sized weight diff,
 * RMSNormLayer.cs:199 with math.cu:6945-6961: identical to this for outerNum == 1, out of bounds beyond).
 * dw null skips the weight gradient; otherwise scratch holds mca_rmsnorm_backward_scratch_floats(inner) floats. */
MCA_API int mca_rmsnorm_forward_f32(const float* x, const float* w, float* y, float* inv_rms, int64_t rows, int inner,
                                    float eps, void* stream);
MCA_API int64_t mca_rmsnorm_backward_scratch_floats(int inner);
MCA_API int mca_rmsnorm_backward_f32(const float* x, const float* w, const float* dy, const float* inv_rms, float* dx,
                                     float* dw, float* scratch, int64_t scratch_floats, int64_t rows, int inner,
                                     void* stream);

/* float <-> bf16 copies used at the handle boundary. */
MCA_API int mca_convert_f32_to_bf16(const float* x, void* y, int64_t n, void* stream);
MCA_API int mca_convert_bf16_to_f32(const void* x, float* y, int64_t n, void* stream);

/* Library identification: "mycaffe_attn_b200 <version> sm_100a". */
MCA_API const char* mca_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MYCAFFE_ATTN_H_ */

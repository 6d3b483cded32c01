// P/Invoke binding of libmycaffe_attn for MyCaffe's C# host (MyCaffe/common/CudaDnn.cs).
//
// CudaDnn<T> reaches its native DLL through the COM object CudaControlLib.ICudaKernel (CudaDnn.cs:1118,1693-1735),
// which forwards RunFloat / RunFloatEx / RunFloatEx2 / QueryString to the exports of CudaDnnDLL
// (CudaDnnDLL/CudaDnnDLL.cpp:134,314,495,855; ordinals in CudaDnnDLL.12.3.def).  This file binds the same exports of
// libmycaffe_attn directly, so the attention ids (160-164), the RoPE ids (980-983), the LayerNorm ids (970-976), the
// memory ids they need and the llama2 extension can be served without the COM layer.  Argument packing is the one
// CudaDnn.cs already builds (attention :5614-5700, memory :2584-2723, extensions :3703-3812).
//
// This file is written against the reference's sources and cannot be compiled where the library is built (no .NET
// there); mycaffe_b200/cudadnn.py is the same binding in Python/ctypes and is what the test-suite drives.
using System;
using System.Runtime.InteropServices;
using System.Text;

namespace MyCaffe.common
{
    /// <summary>Raw exports (names and signatures of CudaDnnDLL.cpp; LONG = 32-bit, LONGLONG = 64-bit).</summary>
    internal static class AttnNative
    {
        const string Dll = "mycaffe_attn";   // libmycaffe_attn.so (Linux) / mycaffe_attn.dll (Windows)
        const CallingConvention CC = CallingConvention.StdCall;   // WINAPI; ignored on x64 and on Linux

        [DllImport(Dll, CallingConvention = CC, CharSet = CharSet.Ansi)]
        internal static extern int DLL_InvokeFloat(int lKernelIdx, int lFunctionIdx, float[] pInput, int lInput,
            ref IntPtr ppOutput, ref int plOutput, StringBuilder szErr, int lszErrMax);

        [DllImport(Dll, CallingConvention = CC, CharSet = CharSet.Ansi)]
        internal static extern int DLL_InvokeFloatEx2(int lKernelIdx, int lFunctionIdx, float[] pInput, int lInput,
            long[] plInput, int llInput, ref IntPtr ppOutput, ref int plOutput, StringBuilder szErr, int lszErrMax);

        [DllImport(Dll, CallingConvention = CC, CharSet = CharSet.Ansi)]
        internal static extern int DLL_InvokeFloatEx(int lKernelIdx, int lFunctionIdx, float[] pInput, int lInput,
            string pszInput, ref IntPtr ppOutput, ref int plOutput, StringBuilder szErr, int lszErrMax);

        // CUDA_DLL_FREEMEM (-1): hands a pinned result buffer back (Kernel<T>::FreeHost, CudaDnnDLL.cpp:188-201)
        [DllImport(Dll, CallingConvention = CC, CharSet = CharSet.Ansi, EntryPoint = "DLL_InvokeFloat")]
        internal static extern int DLL_FreeResult(int lKernelIdx, int lFunctionIdx, IntPtr pBuffer, int lInput,
            IntPtr ppOutput, IntPtr plOutput, StringBuilder szErr, int lszErrMax);

        [DllImport(Dll, CallingConvention = CC, CharSet = CharSet.Ansi)]
        internal static extern int DLL_QueryString(int lKernelIdx, int lFunctionIdx, int[] pInput, int lInput,
            ref IntPtr ppOutput, StringBuilder szErr, int lszErrMax);

        [DllImport(Dll, CallingConvention = CC, CharSet = CharSet.Ansi)]
        internal static extern int DLL_QueryStringFloatEx(int lKernelIdx, int lFunctionIdx, int[] pInput, int lInput,
            StringBuilder pszOutput, int lOutputMax, StringBuilder szErr, int lszErrMax);

        [DllImport(Dll, CallingConvention = CC)]
        internal static extern int Internal_GetPointerFloat(int ht, int lKernelIdx, int hHandle, out IntPtr ppPtr);

        [DllImport(Dll, CallingConvention = CC)]
        internal static extern int Internal_AllocHostFloat(int lKernelIdx, int lCount, out IntPtr ppDst, IntPtr pSrc,
            [MarshalAs(UnmanagedType.I1)] bool bSrcOnDevice);
    }

    /// <summary>Function ids (CudaDnnDLL/inc/FunctionIDs.h, Cuda Files/main.h) and the ids this library adds.</summary>
    internal static class AttnFn
    {
        internal const int FREEMEM_HOST = -1, INITIALIZE = -2, CLEANUP = -3;
        internal const int ALLOCMEM = 20, FREEMEM = 21, GETMEM = 22, SETMEM = 23, CREATE_CUDNN = 47, FREE_CUDNN = 48;
        internal const int CREATE_EXTENSION = 67, FREE_EXTENSION = 68, EXTENSION_RUN = 69;
        internal const int ATTN_CREATE = 160, ATTN_FREE = 161, ATTN_SET = 162, ATTN_FWD = 163, ATTN_BWD = 164;
        internal const int CREATE_LAYERNORM = 970, FREE_LAYERNORM = 971, LAYERNORM_FWD = 975, LAYERNORM_BWD = 976;
        internal const int CREATE_ROPE = 980, FREE_ROPE = 981, ROPE_FWD = 982, ROPE_BWD = 983;
        internal const int GET_DEVICE_NAME = 1000, GET_EXTENSION_STRING = 1003;
        // added by libmycaffe_attn (include/mycaffe_attn.h)
        internal const int ALLOCMEM_BF16 = 2001, CONVERT = 2002, ATTN_FWD_HOST = 2003, ATTN_FWD_PACKED = 2004, ATTN_BWD_PACKED = 2005;
        internal const int DECODE_CREATE = 2010, DECODE_FREE = 2011, DECODE_STEP = 2012, DECODE_QKV = 2013, DECODE_OUT = 2014;
        internal const int DECODE_FFN = 2015, DECODE_LOGITS = 2016, TFT_ATTN_FWD = 2020, TFT_ATTN_BWD = 2021;
        internal const int SET_ASYNC = 2030, SET_TIMING = 2031, RMSNORM_FWD = 2040, RMSNORM_BWD = 2041;
        internal const int QUERY_VERSION = 2050, QUERY_COUNTERS = 2051;
        internal const int DTYPE_F32 = 0, DTYPE_TF32 = 1, DTYPE_BF16 = 2, FLAG_CAUSAL_IMPLICIT = 1;
        // llama2 extension (CudaExtension.llm32.cpp:20-26) and the id added to it
        internal const int LLM_CREATE = 1, LLM_DESTROY = 2, LLM_LOAD = 3, LLM_QUERYSTATUS = 4, LLM_ABORT = 7, LLM_FORWARD = 100;
    }

    /// <summary>One native kernel index, with the calling conventions of ICudaKernel.RunFloat / RunFloatEx2.</summary>
    public sealed class AttnKernel : IDisposable
    {
        const int ErrMax = 1024;
        int m_hKernel;

        public AttnKernel(int nDeviceID)
        {
            float[] rg = RunFloat(AttnFn.INITIALIZE, new float[] { nDeviceID, 0 });
            m_hKernel = (int)rg[0];
        }

        public int KernelHandle { get { return m_hKernel; } }

        /// <summary>Scalar results come back in the caller's buffer; larger ones in a pinned buffer of the library that
        /// is copied out and returned with FREEMEM (-1), as the COM layer does.</summary>
        float[] finish(int rc, StringBuilder sbErr, IntPtr pOut, IntPtr pOwn, int nOut)
        {
            if (rc != 0)
                throw new Exception("[" + rc.ToString() + "] " + sbErr.ToString());
            float[] rgOut = new float[nOut];
            if (nOut > 0)
                Marshal.Copy(pOut, rgOut, 0, nOut);
            if (pOut != pOwn)
                AttnNative.DLL_FreeResult(m_hKernel, AttnFn.FREEMEM_HOST, pOut, 0, IntPtr.Zero, IntPtr.Zero, sbErr, ErrMax);
            return rgOut;
        }

        public float[] RunFloat(int nFn, float[] rgf)
        {
            StringBuilder sbErr = new StringBuilder(ErrMax);
            IntPtr pOwn = Marshal.AllocHGlobal(sizeof(float));
            try
            {
                IntPtr pOut = pOwn;
                int nOut = 1;
                int rc = AttnNative.DLL_InvokeFloat(m_hKernel, nFn, rgf, (rgf == null) ? 0 : rgf.Length, ref pOut, ref nOut, sbErr, ErrMax);
                return finish(rc, sbErr, pOut, pOwn, nOut);
            }
            finally { Marshal.FreeHGlobal(pOwn); }
        }

        public float[] RunFloatEx2(int nFn, float[] rgf, long[] rgl)
        {
            StringBuilder sbErr = new StringBuilder(ErrMax);
            IntPtr pOwn = Marshal.AllocHGlobal(sizeof(float));
            try
            {
                IntPtr pOut = pOwn;
                int nOut = 1;
                int rc = AttnNative.DLL_InvokeFloatEx2(m_hKernel, nFn, rgf, (rgf == null) ? 0 : rgf.Length, rgl, (rgl == null) ? 0 : rgl.Length,
                                                       ref pOut, ref nOut, sbErr, ErrMax);
                return finish(rc, sbErr, pOut, pOwn, nOut);
            }
            finally { Marshal.FreeHGlobal(pOwn); }
        }

        public float[] RunFloatEx(int nFn, float[] rgf, string strInput)
        {
            StringBuilder sbErr = new StringBuilder(ErrMax);
            IntPtr pOwn = Marshal.AllocHGlobal(sizeof(float));
            try
            {
                IntPtr pOut = pOwn;
                int nOut = 1;
                int rc = AttnNative.DLL_InvokeFloatEx(m_hKernel, nFn, rgf, (rgf == null) ? 0 : rgf.Length, strInput, ref pOut, ref nOut, sbErr, ErrMax);
                return finish(rc, sbErr, pOut, pOwn, nOut);
            }
            finally { Marshal.FreeHGlobal(pOwn); }
        }

        public string QueryString(int nFn, int[] rgArg)
        {
            StringBuilder sbErr = new StringBuilder(ErrMax);
            IntPtr pStr = IntPtr.Zero;
            int rc = AttnNative.DLL_QueryString(m_hKernel, nFn, rgArg, (rgArg == null) ? 0 : rgArg.Length, ref pStr, sbErr, ErrMax);
            if (rc != 0)
                throw new Exception("[" + rc.ToString() + "] " + sbErr.ToString());
            string str = Marshal.PtrToStringAnsi(pStr);
            AttnNative.DLL_QueryString(m_hKernel, AttnFn.FREEMEM_HOST, null, 0, ref pStr, sbErr, ErrMax);
            return str;
        }

        // ---- the attention methods of CudaDnn<T> (CudaDnn.cs:5614-5700), same names, same packing ----

        public long CreateCuDNN() { return (long)RunFloat(AttnFn.CREATE_CUDNN, null)[0]; }
        public long CreateAttn() { return (long)RunFloat(AttnFn.ATTN_CREATE, null)[0]; }
        public void FreeAttn(long h) { RunFloat(AttnFn.ATTN_FREE, new float[] { h }); }

        public void SetAttn(long hCuDnn, long hAttn, int nGpuID, bool bTraining, int nBatch, int nBlockSize, int nHeads, int nSize,
                            float fDropout, long lSeed = 0)
        {
            RunFloatEx2(AttnFn.ATTN_SET, new float[] { fDropout },
                        new long[] { hCuDnn, hAttn, nGpuID, bTraining ? 1 : 0, nBatch, nBlockSize, nHeads, nSize, lSeed });
        }

        /// <summary>Addition: the 10th / 11th long select bf16 or tf32 arithmetic and the analytic causal mask.</summary>
        public void SetAttnEx(long hCuDnn, long hAttn, int nGpuID, bool bTraining, int nBatch, int nBlockSize, int nHeads, int nSize,
                              float fDropout, long lSeed, int nDtype, int nFlags)
        {
            RunFloatEx2(AttnFn.ATTN_SET, new float[] { fDropout },
                        new long[] { hCuDnn, hAttn, nGpuID, bTraining ? 1 : 0, nBatch, nBlockSize, nHeads, nSize, lSeed, nDtype, nFlags });
        }

        public void AttnScaledDotProductForward(long hCuDnn, long hAttn, int nBlockSize, long hQ, long hK, long hV, long hMask, long hY,
                                                bool bBatchMask = false)
        {
            RunFloatEx2(AttnFn.ATTN_FWD, null, new long[] { hCuDnn, hAttn, nBlockSize, hQ, hK, hV, hMask, hY, bBatchMask ? 1 : 0 });
        }

        public void AttnScaledDotProductBackward(long hCuDnn, long hAttn, long hQ, long hdQ, long hK, long hdK, long hV, long hdV,
                                                 long hMask, long hY, long hdY)
        {
            RunFloatEx2(AttnFn.ATTN_BWD, null, new long[] { hCuDnn, hAttn, hQ, hdQ, hK, hdK, hV, hdV, hMask, hY, hdY });
        }

        /// <summary>Addition (ids 2004 / 2005): q, k, v read in place from the (B,T,3C) c_attn output, y as (B,T,C); replaces the
        /// channel_copy x3 and transpose_hw x4 of CausalSelfAttentionLayer.cs:537-557,604.</summary>
        public void AttnScaledDotProductForwardPacked(long hCuDnn, long hAttn, int nBlockSize, long hQKV, long hMask, long hY, bool bBatchMask = false)
        {
            RunFloatEx2(AttnFn.ATTN_FWD_PACKED, null, new long[] { hCuDnn, hAttn, nBlockSize, hQKV, hMask, hY, bBatchMask ? 1 : 0 });
        }

        public void AttnScaledDotProductBackwardPacked(long hCuDnn, long hAttn, long hQKV, long hdQKV, long hMask, long hY, long hdY)
        {
            RunFloatEx2(AttnFn.ATTN_BWD_PACKED, null, new long[] { hCuDnn, hAttn, hQKV, hdQKV, hMask, hY, hdY });
        }

        // ---- RoPE (CudaDnn.cs:6375-6431) ----

        public long CreateRope(int nSharedIndex, int nGpuID, int nCount, int nBatch, int nSeqLen, int nHeads, int nDim, float fTheta = 10000.0f)
        {
            return (long)RunFloatEx2(AttnFn.CREATE_ROPE, new float[] { fTheta }, new long[] { nSharedIndex, nGpuID, nCount, nBatch, nSeqLen, nHeads, nDim })[0];
        }
        public void FreeRope(long h) { RunFloat(AttnFn.FREE_ROPE, new float[] { h }); }
        public void RopeForward(long hRope, int n, long hX, long hY, int nFreqOffset = -1)
        {
            RunFloatEx2(AttnFn.ROPE_FWD, null, new long[] { hRope, n, hX, hY, nFreqOffset });
        }
        public void RopeBackward(long hRope, int n, long hX, long hYdiff, long hXdiff)
        {
            RunFloatEx2(AttnFn.ROPE_BWD, null, new long[] { hRope, n, hX, hYdiff, hXdiff });
        }

        // ---- extensions (CudaDnn.cs:3703-3812): the llama2 route ----

        public long CreateExtension(string strExtensionDllPath) { return (long)RunFloatEx(AttnFn.CREATE_EXTENSION, null, strExtensionDllPath)[0]; }
        public void FreeExtension(long hExtension) { RunFloat(AttnFn.FREE_EXTENSION, new float[] { hExtension }); }

        public float[] RunExtension(long hExtension, long lfnIdx, float[] rgParam)
        {
            float[] rg = new float[2 + ((rgParam == null) ? 0 : rgParam.Length)];
            rg[0] = hExtension; rg[1] = lfnIdx;
            if (rgParam != null) Array.Copy(rgParam, 0, rg, 2, rgParam.Length);
            return RunFloat(AttnFn.EXTENSION_RUN, rg);
        }

        public float[] RunExtensionEx(long hExtension, long lfnIdx, float[] rgParam, string strInput)
        {
            float[] rg = new float[2 + ((rgParam == null) ? 0 : rgParam.Length)];
            rg[0] = hExtension; rg[1] = lfnIdx;
            if (rgParam != null) Array.Copy(rgParam, 0, rg, 2, rgParam.Length);
            return RunFloatEx(AttnFn.EXTENSION_RUN, rg, strInput);
        }

        /// <summary>One TransformerGpu::forward(token, pos) of a model loaded through the llama2 extension: the logits.</summary>
        public float[] LlamaForward(long hExtension, long hLlm, int nToken, int nPos)
        {
            return RunExtension(hExtension, AttnFn.LLM_FORWARD, new float[] { hLlm, nToken, nPos });
        }

        public void Dispose()
        {
            if (m_hKernel != 0)
            {
                StringBuilder sbErr = new StringBuilder(ErrMax);
                IntPtr pOut = IntPtr.Zero;
                int nOut = 0;
                AttnNative.DLL_InvokeFloat(m_hKernel, AttnFn.CLEANUP, null, 0, ref pOut, ref nOut, sbErr, ErrMax);
                m_hKernel = 0;
            }
        }
    }
}

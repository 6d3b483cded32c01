"""Host-side mirror of the attention part of MyCaffe's ``CudaDnn<T>`` class
(MyCaffe/common/CudaDnn.cs), over the C ABI of libmycaffe_attn.so.

The reference's host side is C#; no .NET toolchain exists where this package is built, so the
same surface is written in Python with ctypes.  Method names, argument order and meaning and
the error behaviour (a non-zero native code becomes an exception carrying the native message,
as the COM layer does for C#) follow ``CudaDnn.cs``: memory ``:2584-2723``, attention
``:5611-5701``, RoPE ``:6375-6431``.  Every call goes through ``DLL_InvokeFloatEx2`` with the
packed float / long arrays the C# code builds.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from . import function_ids as ids


class CudaDnnError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"[{code}] {message}")
        self.code = int(code)
        self.native_message = message


class CudaDnn:
    """One instance == one native kernel index (CudaDnn.cs:1693-1735)."""

    def __init__(self, device_id: int = 0):
        self._lib = _lib.load()
        self._kernel = 0
        out = self._invoke(ids.CUDA_DLL_INITIALIZE, [float(device_id), 0.0], None)
        self._kernel = int(out[0])
        self.device_id = device_id

    # ------------------------------------------------------------------ plumbing
    def _invoke(self, fn, floats=None, longs=None, out_capacity=1, out_buf=None):
        lib = self._lib
        fa = np.ascontiguousarray(floats, dtype=np.float32) if floats is not None else None
        la = np.ascontiguousarray(longs, dtype=np.int64) if longs is not None else None
        if out_buf is None:
            out_buf = np.zeros(max(1, out_capacity), np.float32)
        pp = C.cast(out_buf.ctypes.data, C.POINTER(C.c_float))
        n_out = _lib.LONG(out_buf.size)
        err = C.create_string_buffer(1024)
        rc = lib.DLL_InvokeFloatEx2(
            self._kernel, fn,
            fa.ctypes.data_as(C.POINTER(C.c_float)) if fa is not None else None, fa.size if fa is not None else 0,
            la.ctypes.data_as(C.POINTER(C.c_int64)) if la is not None else None, la.size if la is not None else 0,
            C.byref(pp), C.byref(n_out), err, 1024)
        if rc != 0:
            raise CudaDnnError(rc, err.value.decode(errors="replace"))
        n = n_out.value
        if C.cast(pp, C.c_void_p).value != out_buf.ctypes.data:
            # the library returned a pinned buffer of its own; copy out and release it (FREEMEM -1)
            res = np.ctypeslib.as_array(pp, shape=(n,)).copy()
            lib.DLL_InvokeFloat(self._kernel, ids.CUDA_DLL_FREEMEM, pp, 0, None, None, err, 1024)
            return res
        return out_buf[:n]

    def _finish(self, rc, err, pp, n_out, out_buf):
        if rc != 0:
            raise CudaDnnError(rc, err.value.decode(errors="replace"))
        n = n_out.value
        if C.cast(pp, C.c_void_p).value != out_buf.ctypes.data:
            res = np.ctypeslib.as_array(pp, shape=(n,)).copy()
            self._lib.DLL_InvokeFloat(self._kernel, ids.CUDA_DLL_FREEMEM, pp, 0, None, None, err, 1024)
            return res
        return out_buf[:n]

    def _invoke_float(self, fn, floats=None, text=None):
        """DLL_InvokeFloat (RunFloat), or DLL_InvokeFloatEx (RunFloatEx) when a string goes with the call."""
        fa = np.ascontiguousarray(floats, dtype=np.float32) if floats is not None else None
        out_buf = np.zeros(1, np.float32)
        pp = C.cast(out_buf.ctypes.data, C.POINTER(C.c_float))
        n_out = _lib.LONG(out_buf.size)
        err = C.create_string_buffer(1024)
        fp = fa.ctypes.data_as(C.POINTER(C.c_float)) if fa is not None else None
        nf = fa.size if fa is not None else 0
        if text is None:
            rc = self._lib.DLL_InvokeFloat(self._kernel, fn, fp, nf, C.byref(pp), C.byref(n_out), err, 1024)
        else:
            rc = self._lib.DLL_InvokeFloatEx(self._kernel, fn, fp, nf, text.encode(), C.byref(pp), C.byref(n_out), err, 1024)
        return self._finish(rc, err, pp, n_out, out_buf)

    def QueryString(self, fn, ints=()):
        """DLL_QueryString: the answer is a string the library allocates and takes back (FREEMEM)."""
        ia = np.ascontiguousarray(list(ints), dtype=np.int32)
        out = C.c_void_p()
        err = C.create_string_buffer(1024)
        rc = self._lib.DLL_QueryString(self._kernel, fn, ia.ctypes.data_as(C.POINTER(_lib.LONG)) if ia.size else None, ia.size,
                                       C.byref(out), err, 1024)
        if rc != 0:
            raise CudaDnnError(rc, err.value.decode(errors="replace"))
        text = C.string_at(out.value).decode() if out.value else ""
        self._lib.DLL_QueryString(self._kernel, ids.CUDA_DLL_FREEMEM, None, 0, C.byref(out), err, 1024)
        return text

    def GetDeviceName(self, nDeviceID):
        return self.QueryString(ids.CUDA_FN_GET_DEVICE_NAME, [int(nDeviceID)])

    # ------------------------------------------------------------------ extensions (CudaDnn.cs:3703-3812)
    def CreateExtension(self, strExtensionDllPath="") -> int:
        """An empty path selects the llama2 extension built into the library."""
        return int(self._invoke_float(ids.CUDA_FN_CREATE_EXTENSION, None, strExtensionDllPath)[0])

    def FreeExtension(self, hExtension):
        self._invoke_float(ids.CUDA_FN_FREE_EXTENSION, [float(hExtension)])

    def RunExtension(self, hExtension, lfnIdx, rgParam=None):
        return np.array(self._invoke_float(ids.CUDA_FN_EXTENSION_RUN, [float(hExtension), float(lfnIdx)] + [float(x) for x in (rgParam or [])]))

    def RunExtensionEx(self, hExtension, lfnIdx, rgParam, strInput):
        return np.array(self._invoke_float(ids.CUDA_FN_EXTENSION_RUN,
                                           [float(hExtension), float(lfnIdx)] + [float(x) for x in (rgParam or [])], strInput))

    def QueryExtensionStrings(self, hExtension, lfnIdx, rgParam=()):
        ia = np.ascontiguousarray([int(hExtension), int(lfnIdx)] + [int(x) for x in rgParam], dtype=np.int32)
        buf = C.create_string_buffer(4096)
        err = C.create_string_buffer(1024)
        rc = self._lib.DLL_QueryStringFloatEx(self._kernel, ids.CUDA_FN_GET_EXTENSION_STRING, ia.ctypes.data_as(C.POINTER(_lib.LONG)),
                                              ia.size, buf, 4096, err, 1024)
        if rc != 0:
            raise CudaDnnError(rc, err.value.decode(errors="replace"))
        return buf.value.decode()

    def SetTiming(self, enabled: bool):
        """Addition: bracket every dispatched call with CUDA events; read with QueryCounters()."""
        self._invoke(ids.MCA_FN_SET_TIMING, None, [1 if enabled else 0])

    def QueryCounters(self):
        """{function id: {calls, errors, gpu_ms_last, gpu_ms_total}} of this kernel index."""
        res = {}
        for line in self.QueryString(ids.MCA_FN_QUERY_COUNTERS).splitlines():
            f = line.split()
            res[int(f[0])] = {kv.split("=")[0]: float(kv.split("=")[1]) for kv in f[1:]}
        return res

    def Dispose(self):
        if self._kernel:
            self._lib.DLL_InvokeFloat(self._kernel, ids.CUDA_DLL_CLEANUP, None, 0, None, None, None, 0)
            self._kernel = 0

    def __del__(self):
        try:
            self.Dispose()
        except Exception:
            pass

    @property
    def KernelHandle(self):
        return self._kernel

    # ------------------------------------------------------------------ memory (CudaDnn.cs:2584-2723)
    def AllocMemory(self, data_or_count) -> int:
        if np.isscalar(data_or_count):
            return int(self._invoke(ids.CUDA_FN_ALLOCMEM, None, [int(data_or_count)])[0])
        data = np.ascontiguousarray(data_or_count, np.float32).ravel()
        packed = np.empty(data.size + 1, np.float32)
        packed[0] = data.size
        packed[1:] = data
        return int(self._invoke(ids.CUDA_FN_ALLOCMEM, packed, [data.size])[0])

    def AllocMemoryBf16(self, data_or_count) -> int:
        """Extension: bf16 storage behind a handle; host data stays float and is converted on the device."""
        if np.isscalar(data_or_count):
            return int(self._invoke(ids.MCA_FN_ALLOCMEM_BF16, None, [int(data_or_count)])[0])
        data = np.ascontiguousarray(data_or_count, np.float32).ravel()
        packed = np.empty(data.size + 1, np.float32)
        packed[0] = data.size
        packed[1:] = data
        return int(self._invoke(ids.MCA_FN_ALLOCMEM_BF16, packed, [data.size])[0])

    def FreeMemory(self, h):
        self._invoke(ids.CUDA_FN_FREEMEM, None, [int(h)])

    def GetMemory(self, h, count=-1) -> np.ndarray:
        cap = int(count) if count and count > 0 else 1
        return np.array(self._invoke(ids.CUDA_FN_GETMEM, None, [int(h), int(count)], out_capacity=cap))

    def GetMemoryInto(self, h, out: np.ndarray):
        """GETMEM into a caller-owned float32 buffer (no intermediate copy)."""
        assert out.dtype == np.float32 and out.flags.c_contiguous
        self._invoke(ids.CUDA_FN_GETMEM, None, [int(h), out.size], out_buf=out.reshape(-1))

    def _invoke_raw(self, fn, packed_floats: np.ndarray, longs):
        """Invoke with an already packed float32 array (used to send large host buffers without a copy)."""
        assert packed_floats.dtype == np.float32 and packed_floats.flags.c_contiguous
        return self._invoke(fn, packed_floats, longs)

    def SetMemory(self, h, data):
        data = np.ascontiguousarray(data, np.float32).ravel()
        packed = np.empty(data.size + 2, np.float32)
        packed[0] = h
        packed[1] = data.size
        packed[2:] = data
        self._invoke(ids.CUDA_FN_SETMEM, packed, [int(h), data.size])

    def SetMemoryInt32(self, h, data):
        """int32 values through a 4-byte-element handle (bit pattern preserved)."""
        self.SetMemory(h, np.ascontiguousarray(data, np.int32).view(np.float32))

    def ConvertMemory(self, hSrc, hDst, count):
        self._invoke(ids.MCA_FN_CONVERT, None, [int(hSrc), int(hDst), int(count)])

    def GetPointer(self, h) -> int:
        p = C.c_void_p()
        rc = self._lib.Internal_GetPointerFloat(1, self._kernel, int(h), C.byref(p))
        if rc:
            raise CudaDnnError(rc, "Internal_GetPointerFloat")
        return int(p.value)

    def SynchronizeDevice(self):
        self._invoke(ids.CUDA_FN_SYNCHRONIZEDEVICE)

    def SetAsync(self, enabled: bool):
        """Extension: skip the per-call stream synchronise that the reference performs."""
        self._invoke(ids.MCA_FN_SET_ASYNC, None, [1 if enabled else 0])

    # ------------------------------------------------------------------ cuDNN handle (passed through only)
    def CreateCuDNN(self) -> int:
        return int(self._invoke(ids.CUDNN_FN_CREATE_CUDNN)[0])

    def FreeCuDNN(self, h):
        self._invoke(ids.CUDNN_FN_FREE_CUDNN, [float(h)])

    # ------------------------------------------------------------------ attention (CudaDnn.cs:5611-5701)
    def CreateAttn(self) -> int:
        return int(self._invoke(ids.CUDNN_FN_ATTN_CREATE)[0])

    def FreeAttn(self, h):
        self._invoke(ids.CUDNN_FN_ATTN_FREE, [float(h)])

    def SetAttn(self, hCuDnn, hAttn, nGpuID, bTraining, nBatch, nBlockSize, nHeads, nSize, fDropout, lSeed=0,
                dtype=None, flags=None):
        longs = [hCuDnn, hAttn, nGpuID, 1 if bTraining else 0, nBatch, nBlockSize, nHeads, nSize, lSeed]
        if dtype is not None or flags is not None:
            longs.append(dtype or 0)
        if flags is not None:
            longs.append(flags)
        self._invoke(ids.CUDNN_FN_ATTN_SET, [float(fDropout)], longs)

    def AttnScaledDotProductForward(self, hCuDnn, hAttn, nBlockSize, hQ, hK, hV, hMask, hY, bBatchMask=False):
        self._invoke(ids.CUDNN_FN_ATTN_FWD, None,
                     [hCuDnn, hAttn, nBlockSize, hQ, hK, hV, hMask, hY, 1 if bBatchMask else 0])

    def AttnScaledDotProductBackward(self, hCuDnn, hAttn, hQ, hdQ, hK, hdK, hV, hdV, hMask, hY, hdY):
        self._invoke(ids.CUDNN_FN_ATTN_BWD, None, [hCuDnn, hAttn, hQ, hdQ, hK, hdK, hV, hdV, hMask, hY, hdY])

    # ------------------------------------------------------------------ LayerNorm (CudaDnn.cs:6307-6360)
    def CreateLayerNorm(self, nGpuID, nCount, nOuterNum, nChannels, nInnerNum, fEps=1e-10) -> int:
        return int(self._invoke(ids.CUDA_FN_CREATE_LAYERNORM, [float(fEps)],
                                [nGpuID, nCount, nOuterNum, nChannels, nInnerNum])[0])

    def FreeLayerNorm(self, h):
        self._invoke(ids.CUDA_FN_FREE_LAYERNORM, [float(h)])

    def LayerNormForward(self, hLayerNorm, hXdata, hYdata):
        self._invoke(ids.CUDA_FN_LAYERNORM_FWD, None, [hLayerNorm, hXdata, hYdata])

    def LayerNormBackward(self, hLayerNorm, hYdata, hYdiff, hXdiff):
        self._invoke(ids.CUDA_FN_LAYERNORM_BWD, None, [hLayerNorm, hYdata, hYdiff, hXdiff])

    # ------------------------------------------------------------------ RMSNorm layer (RMSNormLayer.cs:156-231)
    def RmsNormForward(self, hX, hW, hY, hInvRms, nRows, nInner, fEps=1e-5):
        """y = w * x / sqrt(mean(x^2) + eps) in one pass; hW = 0 for a layer without weights."""
        self._invoke(ids.MCA_FN_RMSNORM_FWD, [float(fEps)], [hX, hW, hY, hInvRms, nRows, nInner])

    def RmsNormBackward(self, hX, hW, hdY, hInvRms, hdX, hdW, nRows, nInner):
        """dx (and dw unless hdW = 0) from dy and the 1/rms the forward saved."""
        self._invoke(ids.MCA_FN_RMSNORM_BWD, None, [hX, hW, hdY, hInvRms, hdX, hdW, nRows, nInner])

    # ------------------------------------------------------------------ RoPE (CudaDnn.cs:6375-6431)
    def CreateRope(self, nSharedIndex, nGpuID, nCount, nBatch, nSeqLen, nHeads, nDim, fTheta=10000.0) -> int:
        return int(self._invoke(ids.CUDA_FN_CREATE_ROPE, [float(fTheta)],
                                [nSharedIndex, nGpuID, nCount, nBatch, nSeqLen, nHeads, nDim])[0])

    def FreeRope(self, h):
        self._invoke(ids.CUDA_FN_FREE_ROPE, [float(h)])

    def RopeForward(self, hRope, n, hX, hY, nFreqOffset=-1):
        self._invoke(ids.CUDA_FN_ROPE_FWD, None, [hRope, n, hX, hY, nFreqOffset])

    def RopeBackward(self, hRope, n, hX, hYdiff, hXdiff):
        self._invoke(ids.CUDA_FN_ROPE_BWD, None, [hRope, n, hX, hYdiff, hXdiff])

    # ------------------------------------------------------------------ extensions: decode, TFT
    def CreateDecode(self, nBatch, nHeads, nKvHeads, nHeadSize, nSeqLen, bCacheBf16=False, fTheta=10000.0) -> int:
        return int(self._invoke(ids.MCA_FN_DECODE_CREATE, [float(fTheta)],
                                [nBatch, nHeads, nKvHeads, nHeadSize, nSeqLen, 1 if bCacheBf16 else 0])[0])

    def FreeDecode(self, h):
        self._invoke(ids.MCA_FN_DECODE_FREE, [float(h)])

    def DecodeStep(self, hDecode, hQ, hKnew, hVnew, hKcache, hVcache, hPos, nMaxLen, hOut):
        self._invoke(ids.MCA_FN_DECODE_STEP, None, [hDecode, hQ, hKnew, hVnew, hKcache, hVcache, hPos, nMaxLen, hOut])

    def DecodeQkv(self, hX, hRmsW, hWq, hWk, hWv, nBatch, nDim, nKvDim, hQ, hK, hV, fEps=1e-5):
        """RMSNorm + q,k,v projections of the new token (llama2_gpu.cpp:56-61)."""
        self._invoke(ids.MCA_FN_DECODE_QKV, [float(fEps)], [hX, hRmsW, hWq, hWk, hWv, nBatch, nDim, nKvDim, hQ, hK, hV])

    def DecodeOut(self, hAttn, hWo, nBatch, nDim, hX):
        """x += Wo . attn (llama2_gpu.cpp:78-81)."""
        self._invoke(ids.MCA_FN_DECODE_OUT, None, [hAttn, hWo, nBatch, nDim, hX])

    def DecodeFfn(self, hX, hRmsW, hW1, hW2, hW3, nBatch, nDim, nHiddenDim, hHidden, fEps=1e-5):
        """x += W2 . (silu(W1 xn) * (W3 xn)), xn = rmsnorm(x) (llama2_gpu.cpp:84-97)."""
        self._invoke(ids.MCA_FN_DECODE_FFN, [float(fEps)], [hX, hRmsW, hW1, hW2, hW3, nBatch, nDim, nHiddenDim, hHidden])

    def DecodeLogits(self, hX, hRmsW, hWcls, nBatch, nDim, nVocab, hLogits, fEps=1e-5):
        """logits = Wcls . rmsnorm(x) (llama2_gpu.cpp:101-105)."""
        self._invoke(ids.MCA_FN_DECODE_LOGITS, [float(fEps)], [hX, hRmsW, hWcls, nBatch, nDim, nVocab, hLogits])

    def AttnScaledDotProductForwardPacked(self, hCuDnn, hAttn, nBlockSize, hQKV, hMask, hY, bBatchMask=False):
        """ATTN_FWD on the (B,T,3C) c_attn output: q, k, v are read in place, y is written as (B,T,C)."""
        self._invoke(ids.MCA_FN_ATTN_FWD_PACKED, None,
                     [hCuDnn, hAttn, nBlockSize, hQKV, hMask, hY, 1 if bBatchMask else 0])

    def AttnScaledDotProductBackwardPacked(self, hCuDnn, hAttn, hQKV, hdQKV, hMask, hY, hdY):
        self._invoke(ids.MCA_FN_ATTN_BWD_PACKED, None, [hCuDnn, hAttn, hQKV, hdQKV, hMask, hY, hdY])

    def AttnForwardHost(self, q, k, v, y, bCausal, nHeadsPerChunk=0):
        """Forward for (B,H,T,D) numpy tensors in host memory (float32, or bf16 bit patterns as uint16),
        copies overlapped with the kernel; `y` is filled in place."""
        B, H, T, D = q.shape
        dt = ids.MCA_DTYPE_F32 if q.dtype == np.float32 else ids.MCA_DTYPE_BF16
        for a in (q, k, v, y):
            assert a.flags.c_contiguous and a.dtype == q.dtype and a.shape == q.shape
        assert q.dtype in (np.float32, np.uint16)
        self._invoke(ids.MCA_FN_ATTN_FWD_HOST, None,
                     [q.ctypes.data, k.ctypes.data, v.ctypes.data, y.ctypes.data, dt, 1 if bCausal else 0, B, H, T, D,
                      int(nHeadsPerChunk)])

    def TftAttnBackward(self, hQ, hK, hV, hMask, hdOut, hdAttn, nBatch, nHeads, nQ, nK, nDim, hdQ, hdK, hdV):
        self._invoke(ids.MCA_FN_TFT_ATTN_BWD, None,
                     [hQ, hK, hV, hMask, hdOut, hdAttn, nBatch, nHeads, nQ, nK, nDim, hdQ, hdK, hdV])

    def TftAttnForward(self, hQ, hK, hV, hMask, nBatch, nHeads, nQ, nK, nDim, hOut, hAttn):
        self._invoke(ids.MCA_FN_TFT_ATTN_FWD, None, [hQ, hK, hV, hMask, nBatch, nHeads, nQ, nK, nDim, hOut, hAttn])

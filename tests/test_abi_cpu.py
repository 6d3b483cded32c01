"""CPU-only checks of the drop-in boundary: the shared library loads, exports every symbol the
public header declares, agrees with the header on function ids, and fails loudly without a GPU."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "mycaffe_attn.h").read_text()


@pytest.fixture(scope="module")
def lib():
    from mycaffe_b200 import build, _lib
    build.build()
    return _lib.load()


def declared_functions():
    return sorted(set(re.findall(r"MCA_API\s+[\w\s\*]+?\s+\*?(\w+)\s*\(", HEADER)))


def test_header_declares_the_reference_exports():
    names = declared_functions()
    for required in ["DLL_InvokeFloat", "DLL_InvokeFloatEx", "DLL_InvokeFloatEx2", "DLL_InvokeDouble",
                     "DLL_InvokeDoubleEx2", "Internal_GetPointerFloat", "Internal_AllocHostFloat"]:
        assert required in names


# EXPORTS of CudaDnnDLL/CudaDnnDLL.12.3.def (ordinals 1-7, 100-103), the two query-string entries CudaDnnDLL.cpp:935,976
# adds beside them, and EXPORTS of CudaExtension.llm32.llama2/CudaExtension.llm32.11.8.def (ordinals 1-6).
REFERENCE_DEF_EXPORTS = ["DLL_InvokeFloat", "DLL_InvokeDouble", "DLL_QueryString", "DLL_InvokeFloatEx", "DLL_InvokeDoubleEx",
                         "DLL_InvokeFloatEx2", "DLL_InvokeDoubleEx2", "Internal_GetPointerFloat", "Internal_GetPointerDouble",
                         "Internal_AllocHostFloat", "Internal_AllocHostDouble", "DLL_QueryStringFloatEx", "DLL_QueryStringDoubleEx"]
EXTENSION_DEF_EXPORTS = ["DLL_InitFloatCustomExtension", "DLL_InvokeFloatCustomExtension", "DLL_InitDoubleCustomExtension",
                         "DLL_InvokeDoubleCustomExtension", "DLL_InvokeFloatCustomExtensionEx", "DLL_InvokeDoubleCustomExtensionEx"]


def test_every_export_of_the_reference_def_files_resolves(lib):
    """A loader that GetProcAddress'es the reference's whole export table must find every name."""
    raw = C.CDLL(str(lib._name))
    names = declared_functions()
    for n in REFERENCE_DEF_EXPORTS + EXTENSION_DEF_EXPORTS:
        assert n in names, f"{n} not declared in the header"
        assert getattr(raw, n) is not None


def test_double_and_uninitialised_entries_answer_without_a_gpu(lib):
    from mycaffe_b200 import function_ids as ids
    err = C.create_string_buffer(256)
    out = C.c_void_p()
    # double twins: not implemented, with a message
    assert lib.DLL_InvokeDoubleEx(0, ids.CUDNN_FN_ATTN_CREATE, None, 0, None, None, None, err, 256) == ids.ERROR_NOT_IMPLEMENTED
    assert b"not implemented" in err.value
    assert lib.DLL_QueryStringDoubleEx(0, 1003, None, 0, None, 0, err, 256) == ids.ERROR_NOT_IMPLEMENTED
    assert lib.Internal_GetPointerDouble(1, 3, 1, C.byref(out)) == ids.ERROR_PARAM_NULL      # empty double table, CudaDnnDLL.cpp:84-88
    assert lib.Internal_AllocHostDouble(3, 1, None, None, False) == ids.ERROR_PARAM_NULL
    assert lib.Internal_GetPointerDouble(1, 5000, 1, C.byref(out)) == ids.ERROR_PARAM_OUT_OF_RANGE
    assert lib.DLL_InitDoubleCustomExtension(None, 0) == ids.ERROR_NOT_IMPLEMENTED
    # query string on a slot that holds no kernel: ERROR_PARAM_OUT_OF_RANGE (CudaDnnDLL.cpp:928-931)
    assert lib.DLL_QueryString(9, ids.CUDA_FN_GET_DEVICE_NAME, None, 0, C.byref(out), err, 256) == ids.ERROR_PARAM_OUT_OF_RANGE
    assert lib.DLL_QueryStringFloatEx(9, ids.CUDA_FN_GET_EXTENSION_STRING, None, 0, None, 0, err, 256) == ids.ERROR_PARAM_OUT_OF_RANGE
    # the extension before DLL_InitFloatCustomExtension: PEER_E_NOT_INITIALIZED (CudaExtension.llm32.cpp:95-96)
    n = C.c_int32(0)
    pp = C.POINTER(C.c_float)()
    rc = lib.DLL_InvokeFloatCustomExtension(ids.LLM_CUDA_EXTENSION_CREATE, None, 0, C.byref(pp), C.byref(n), err, 256)
    assert rc & 0xFFFFFFFF == 0x80630001
    assert lib.DLL_InitFloatCustomExtension(None, 1) == 87                                   # ERROR_INVALID_PARAMETER
    # initialised against this library as the parent (it exports DLL_InvokeFloat and Internal_AllocHostFloat)
    assert lib.DLL_InitFloatCustomExtension(C.c_void_p(lib._handle), 1) == 0
    rc = lib.DLL_InvokeFloatCustomExtension(999, None, 0, C.byref(pp), C.byref(n), err, 256)
    assert rc == 50 and b"not supported" in err.value                                        # ERROR_NOT_SUPPORTED + the reference's text
    rc = lib.DLL_InvokeFloatCustomExtensionEx(ids.LLM_CUDA_EXTENSION_GENERATE, None, 0, None, None, b"x", None, 0, err, 256)
    assert rc == 50 and b"not provided" in err.value


def test_decode_head_sizes(lib):
    assert [h for h in range(1, 257) if lib.mca_decode_head_size_supported(h)] == [32, 48, 64, 96, 128]


def test_library_exports_every_declared_symbol(lib):
    from mycaffe_b200 import _lib
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mycaffe_attn.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert lib.mca_version().decode().endswith("sm_100a")


def test_function_ids_match_header():
    from mycaffe_b200 import function_ids as ids
    for name, val in re.findall(r"#define\s+((?:CUDA|CUDNN|MCA)_(?:FN|DLL|DTYPE|FLAG)\w+)\s+\(?(-?\d+)\)?", HEADER):
        assert getattr(ids, name) == int(val), name
    # the reference's values (inc/FunctionIDs.h:222-226,532-535; Cuda Files/main.h:30-32)
    assert (ids.CUDNN_FN_ATTN_CREATE, ids.CUDNN_FN_ATTN_FREE, ids.CUDNN_FN_ATTN_SET, ids.CUDNN_FN_ATTN_FWD,
            ids.CUDNN_FN_ATTN_BWD) == (160, 161, 162, 163, 164)
    assert (ids.CUDA_FN_CREATE_ROPE, ids.CUDA_FN_FREE_ROPE, ids.CUDA_FN_ROPE_FWD, ids.CUDA_FN_ROPE_BWD) == (980, 981, 982, 983)
    assert (ids.CUDA_DLL_FREEMEM, ids.CUDA_DLL_INITIALIZE, ids.CUDA_DLL_CLEANUP) == (-1, -2, -3)
    assert ids.ERROR_ATTN_INVALID_BLOCK_SIZE == 90285 and ids.ERROR_ROPE_NOT_INITIALIZED == 90201


def test_out_of_range_kernel_index_and_double_twin(lib):
    from mycaffe_b200 import _lib, function_ids as ids
    err = C.create_string_buffer(256)
    out = np.zeros(1, np.float32)
    pp = C.cast(out.ctypes.data, C.POINTER(C.c_float))
    n = _lib.LONG(1)
    # kernel index beyond the 2048-slot table: ERROR_PARAM_OUT_OF_RANGE (CudaDnnDLL.cpp:144-145)
    assert lib.DLL_InvokeFloat(5000, ids.CUDNN_FN_ATTN_CREATE, None, 0, C.byref(pp), C.byref(n), err, 256) == 90001
    # never-initialised slot: ERROR_PARAM_NULL (CudaDnnDLL.cpp:296-301)
    assert lib.DLL_InvokeFloat(7, ids.CUDNN_FN_ATTN_CREATE, None, 0, C.byref(pp), C.byref(n), err, 256) == 90002
    assert b"null" in err.value
    assert lib.DLL_InvokeDouble(0, ids.CUDNN_FN_ATTN_CREATE, None, 0, None, None, err, 256) == ids.ERROR_NOT_IMPLEMENTED


def test_rope_tables_host_match_oracle(lib):
    import oracle
    T, D = 33, 16
    c = np.empty((T, D // 2), np.float32)
    s = np.empty((T, D // 2), np.float32)
    fp = C.POINTER(C.c_float)
    assert lib.mca_rope_tables_host(T, D, 10000.0, c.ctypes.data_as(fp), s.ctypes.data_as(fp)) == 0
    oc, os_ = oracle.rope_tables(T, D, 10000.0)
    np.testing.assert_array_equal(c, oc)
    np.testing.assert_array_equal(s, os_)


def test_decode_plan_is_consistent(lib):
    sl, ns, sc = C.c_int(), C.c_int(), C.c_int64()
    for B, nh, nkv, L in [(1, 32, 32, 4096), (64, 32, 32, 4096), (16, 32, 8, 513), (1, 8, 8, 1)]:
        assert lib.mca_decode_plan(B, nh, nkv, 128, L, C.byref(sl), C.byref(ns), C.byref(sc)) == 0
        assert sl.value % 16 == 0 and 16 <= sl.value <= 1024
        assert ns.value == -(-L // sl.value)
        assert sc.value == B * nh * ns.value * 130
    assert lib.mca_decode_plan(1, 32, 5, 128, 10, C.byref(sl), C.byref(ns), C.byref(sc)) == 90001
    # one sequence: the splits fill one wave of the 296 resident CTAs instead of spilling into a third
    assert lib.mca_decode_plan(1, 32, 32, 128, 2339, C.byref(sl), C.byref(ns), C.byref(sc)) == 0
    assert 32 * ns.value <= 296 and ns.value == 9


def test_no_gpu_fails_loudly(lib):
    """Without a CUDA device INITIALIZE must return an error and a message, never fall back."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from mycaffe_b200 import CudaDnn, CudaDnnError
    with pytest.raises(CudaDnnError) as ei:
        CudaDnn(0)
    assert ei.value.code != 0 and ei.value.native_message

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
        assert sl.value % 128 == 0 and 128 <= sl.value <= 1024
        assert ns.value == -(-L // sl.value)
        assert sc.value == B * nh * ns.value * 130
    assert lib.mca_decode_plan(1, 32, 5, 128, 10, C.byref(sl), C.byref(ns), C.byref(sc)) == 90001


def test_no_gpu_fails_loudly(lib):
    """Without a CUDA device INITIALIZE must return an error and a message, never fall back."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from mycaffe_b200 import CudaDnn, CudaDnnError
    with pytest.raises(CudaDnnError) as ei:
        CudaDnn(0)
    assert ei.value.code != 0 and ei.value.native_message

"""CPU: the C-ABI library loads, exports what include/amosb.h declares, and validates arguments
before touching a device."""
import ctypes
import os
import re

import numpy as np
import pytest

from amos_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "amosb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(amosb_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    declared = _declared_symbols()
    assert len(declared) >= 9
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in amosb.h but not exported"
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared


def test_struct_layout_matches_header(built_lib):
    # 8 int32 + 4 int64 + 9 int64 + 8 int32 + 4 int32
    assert ctypes.sizeof(_lib.AmosbOpDesc) == 8 * 4 + 13 * 8 + 8 * 4 + 4 * 4
    assert ctypes.sizeof(_lib.AmosbTensor) == 8 + 4 * 3 + 4 + 8 + 8 + 8


def test_version_and_error_string(built_lib):
    lib = _lib.load()
    assert lib.amosb_version() >= 100
    assert isinstance(_lib.last_error(), str)


def test_workspace_bytes(built_lib):
    assert _lib.workspace_bytes_min(_lib.gemm_desc(128, 128, 128)) == 0
    d = _lib.conv2d_desc(256, 128, 28, 28, 128, 3, 3, pad=1)
    act = 256 * 28 * 28 * 128 * 2
    flt = 128 * 9 * 128 * 2
    assert _lib.workspace_bytes_min(d) == (act + 1023) // 1024 * 1024 + (flt + 1023) // 1024 * 1024
    # channel padding: activation to a multiple of 8, filter to a multiple of 64
    d = _lib.conv2d_desc(1, 3, 8, 8, 16, 3, 3, pad=1)
    assert _lib.workspace_bytes_min(d) == 1024 + (16 * 9 * 64 * 2 + 1023) // 1024 * 1024
    # the optional part: partial sums of a shared-out last round, one accumulator tile per CTA.  By
    # default only where it clearly pays (7x7, C512 -> K512: 98 pair tiles on 74 pairs) ...
    d = _lib.conv2d_desc(256, 512, 7, 7, 512, 3, 3, pad=1)
    assert _lib.workspace_bytes(d) - _lib.workspace_bytes_min(d) == 148 * 128 * 256 * 4
    d = _lib.conv2d_desc(256, 128, 28, 28, 128, 3, 3, pad=1)
    assert _lib.workspace_bytes(d) == _lib.workspace_bytes_min(d)
    assert _lib.workspace_bytes(_lib.gemm_desc(4096, 4096, 4096)) == 0
    # ... and wherever a round is short when forced, never when forbidden
    os.environ["AMOSB_TAIL_SHARING"] = "1"
    try:
        assert _lib.workspace_bytes(d) - _lib.workspace_bytes_min(d) == 148 * 256 * 128 * 4
        big = _lib.gemm_desc(512, 4096, 4096)
        assert _lib.workspace_bytes_min(big) == 0 and _lib.workspace_bytes(big) == 148 * 128 * 256 * 4
        os.environ["AMOSB_NO_TAIL_SHARING"] = "1"
        assert _lib.workspace_bytes(big) == 0
    finally:
        del os.environ["AMOSB_TAIL_SHARING"]
        os.environ.pop("AMOSB_NO_TAIL_SHARING", None)
    bad = _lib.AmosbOpDesc()
    with pytest.raises(_lib.AmosbError):
        _lib.workspace_bytes(bad)


def test_describe_plan(built_lib):
    text = _lib.describe_plan(_lib.gemm_desc(8192, 8192, 8192, in_dtype=_lib.AMOSB_S8))
    assert "i8" in text and "BN=256" in text and "MN-major" in text
    text = _lib.describe_plan(_lib.gemm_desc(4096, 4096, 4096))
    assert "umma_pair" in text and "BN=256" in text and "256 tiles on 74 CTA pairs" in text
    text = _lib.describe_plan(_lib.gemm_desc(512, 64, 512, batch=96, out_dtype=_lib.AMOSB_F16))
    assert "batched_gemm" in text and "BN=64" in text and "umma_persistent" in text
    # pinned choices are honoured
    text = _lib.describe_plan(_lib.gemm_desc(4096, 4096, 4096, tile_n=128, cta_pair=1))
    assert "BN=128" in text and "umma_persistent" in text
    text = _lib.describe_plan(_lib.conv2d_desc(256, 64, 56, 56, 256, 1, 1))
    assert "batched GEMM" in text and "no re-layout" in text


def _host_tensor(arr, dtype_code):
    return _lib.make_tensor(arr.ctypes.data, 0, dtype_code, list(arr.shape))


def _run(desc, a, b, c, codes):
    lib = _lib.load()
    ta, ka = _host_tensor(a, codes[0])
    tb, kb = _host_tensor(b, codes[1])
    tc, kc = _host_tensor(c, codes[2])
    ins = (_lib.AmosbTensor * 2)(ta, tb)
    outs = (_lib.AmosbTensor * 1)(tc)
    return lib.amosb_run(ctypes.byref(desc), ins, 2, outs, 1, None, 0, None)


def test_argument_validation_happens_before_any_device_call(built_lib):
    """Shape / dtype / rank / stride / alignment checks mirror the asserts of the reference's
    generated host function; they fail with -1 and a message, on a machine with no GPU too."""
    d = _lib.gemm_desc(64, 32, 48)
    a = np.zeros((64, 48), np.float16)
    b = np.zeros((48, 32), np.float16)
    c = np.zeros((64, 32), np.float32)
    f16, f32 = _lib.AMOSB_F16, _lib.AMOSB_F32
    assert _run(d, np.zeros((64, 40), np.float16), b, c, (f16, f16, f32)) == _lib.AMOSB_ERR_ARG
    assert "arg0.shape[1]" in _lib.last_error()
    assert _run(d, a, b, c, (f16, f32, f32)) == _lib.AMOSB_ERR_ARG
    assert "arg1.dtype is expected to be float16" in _lib.last_error()
    assert _run(d, a, b, np.zeros((64, 32, 1), np.float32), (f16, f16, f32)) == _lib.AMOSB_ERR_ARG
    assert "arg2.ndim is expected to equal 2" in _lib.last_error()
    lib = _lib.load()
    # wrong argument count
    ta, ka = _host_tensor(a, f16)
    ins = (_lib.AmosbTensor * 1)(ta)
    tc, kc = _host_tensor(c, f32)
    outs = (_lib.AmosbTensor * 1)(tc)
    assert lib.amosb_run(ctypes.byref(d), ins, 1, outs, 1, None, 0, None) == _lib.AMOSB_ERR_ARG
    # non-compact strides
    ta, ka = _lib.make_tensor(a.ctypes.data, 0, f16, [64, 48], strides=[96, 2])
    tb, kb = _host_tensor(b, f16)
    ins = (_lib.AmosbTensor * 2)(ta, tb)
    assert lib.amosb_run(ctypes.byref(d), ins, 2, outs, 1, None, 0, None) == _lib.AMOSB_ERR_ARG
    assert "compact" in _lib.last_error()
    # misaligned data pointer
    ta, ka = _lib.make_tensor(a.ctypes.data, 0, f16, [64, 48], byte_offset=2)
    ins = (_lib.AmosbTensor * 2)(ta, tb)
    assert lib.amosb_run(ctypes.byref(d), ins, 2, outs, 1, None, 0, None) == _lib.AMOSB_ERR_ARG
    assert "16-byte aligned" in _lib.last_error()
    # NULL data
    ta, ka = _lib.make_tensor(0, 0, f16, [64, 48])
    ins = (_lib.AmosbTensor * 2)(ta, tb)
    assert lib.amosb_run(ctypes.byref(d), ins, 2, outs, 1, None, 0, None) == _lib.AMOSB_ERR_ARG
    # tensors on different devices
    ta, ka = _lib.make_tensor(a.ctypes.data, 1, f16, [64, 48])
    ins = (_lib.AmosbTensor * 2)(ta, tb)
    assert lib.amosb_run(ctypes.byref(d), ins, 2, outs, 1, None, 0, None) == _lib.AMOSB_ERR_ARG
    assert "device_id mismatch" in _lib.last_error()


def test_no_cpu_path(built_lib):
    """Without a CUDA device a well-formed call fails with a CUDA error; nothing computes it on
    the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    d = _lib.gemm_desc(64, 32, 48)
    a = np.zeros((64, 48), np.float16)
    b = np.zeros((48, 32), np.float16)
    c = np.full((64, 32), 7.0, np.float32)
    rc = _run(d, a, b, c, (_lib.AMOSB_F16, _lib.AMOSB_F16, _lib.AMOSB_F32))
    assert rc == _lib.AMOSB_ERR_CUDA
    assert (c == 7.0).all()
    from amos_b200 import device
    with pytest.raises(_lib.AmosbError):
        device.tensor_arg(torch.zeros(4, 4, dtype=torch.float16))


def test_dltensor_layout_is_the_reference_one(built_lib):
    # data 0, ctx 8, ndim 16, dtype 20, shape 24, strides 32, byte_offset 40: 48 bytes
    T = _lib.AmosbDLTensor
    assert ctypes.sizeof(T) == 48 and ctypes.sizeof(_lib.AmosbTVMValue) == 8
    assert [getattr(T, f).offset for f in ("data", "ctx", "ndim", "dtype", "shape", "strides",
                                           "byte_offset")] == [0, 8, 16, 20, 24, 32, 40]


def _dl(arr, code, **kw):
    return _lib.make_dl_tensor(arr.ctypes.data, 0, code, list(arr.shape), **kw)


def test_packed_call_checks_what_the_generated_prologue_checks(built_lib):
    """The PackedFunc-shaped entry refuses, with -1 and a message that carries the library's own
    code, everything the reference's generated host function asserts: argument count, handle type
    codes, device_type, device_id, dtype code / bits / lanes, shapes, strides."""
    d = _lib.gemm_desc(64, 32, 48)
    a = np.zeros((64, 48), np.float16)
    b = np.zeros((48, 32), np.float16)
    c = np.zeros((64, 32), np.float32)
    f16, f32 = _lib.AMOSB_F16, _lib.AMOSB_F32
    ta, ka = _dl(a, f16)
    tb, kb = _dl(b, f16)
    tc, kc = _dl(c, f32)
    assert _lib.packed_call(d, [ta, tb]) == -1
    assert "num_args should be 3" in _lib.last_error() and "[amosb -1]" in _lib.last_error()
    assert _lib.packed_call(d, [ta, tb, tc], [7, 0, 7]) == -1  # an int where a tensor is expected
    assert "Expect arg[1] to be pointer" in _lib.last_error()
    assert _lib.packed_call(d, [ta, None, tc]) == -1
    assert "NULL tensor handle" in _lib.last_error()
    cpu, _k = _dl(a, f16, device_type=1)  # kDLCPU
    assert _lib.packed_call(d, [cpu, tb, tc]) == -1
    assert "arg0.device_type" in _lib.last_error()
    other, _k2 = _lib.make_dl_tensor(b.ctypes.data, 1, f16, list(b.shape))
    assert _lib.packed_call(d, [ta, other, tc]) == -1
    assert "arg1.device_id" in _lib.last_error()
    lanes2, _k3 = _dl(a, f16, lanes=2)
    assert _lib.packed_call(d, [lanes2, tb, tc]) == -1
    assert "lanes 2" in _lib.last_error()
    wrong, _k4 = _dl(np.zeros((64, 48), np.float32), f32)
    assert _lib.packed_call(d, [wrong, tb, tc]) == -1
    assert "arg0.dtype is expected to be float16" in _lib.last_error()
    short, _k5 = _dl(np.zeros((64, 40), np.float16), f16)
    assert _lib.packed_call(d, [short, tb, tc]) == -1
    assert "arg0.shape[1]" in _lib.last_error()
    strided, _k6 = _dl(a, f16, strides=[96, 2])
    assert _lib.packed_call(d, [strided, tb, tc]) == -1
    assert "compact" in _lib.last_error()
    # both handle kinds are tensors
    # both handle kinds are tensors: this call gets past the prologue and stops at the memory check
    # (host arrays: -1 with a GPU, -3 without a driver to ask)
    rc = _lib.packed_call(d, [ta, tb, tc], [7, 13, 13])
    assert rc == -1 and ("[amosb -1]" in _lib.last_error() or "[amosb -3]" in _lib.last_error())
    lib = _lib.load()
    assert lib.amosb_set_stream(0, None) == 0 and lib.amosb_set_stream(99, None) == _lib.AMOSB_ERR_ARG


def test_host_memory_is_refused_by_the_device_entry_points(built_lib):
    """amosb_run and amosb_packed_call never hand a host pointer to the copy engine: with a GPU the
    CUDA runtime says what the memory is (-1), without one the query itself fails (-3)."""
    import torch
    d = _lib.gemm_desc(64, 32, 48)
    a = np.zeros((64, 48), np.float16)
    b = np.zeros((48, 32), np.float16)
    c = np.full((64, 32), 7.0, np.float32)
    rc = _run(d, a, b, c, (_lib.AMOSB_F16, _lib.AMOSB_F16, _lib.AMOSB_F32))
    if torch.cuda.is_available():
        assert rc == _lib.AMOSB_ERR_ARG and "device_type is expected to be cuda" in _lib.last_error()
    else:
        assert rc == _lib.AMOSB_ERR_CUDA
    assert (c == 7.0).all()

"""GPU: the reference-shaped entry point (TVMValue array + DLTensors) and the give-up path of the
kernels' bounded waits."""
import ctypes
import os

import numpy as np
import pytest
import torch

from amos_b200 import _lib, device

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dl(t: torch.Tensor, **kw):
    code = device._TORCH_TO_CODE[t.dtype]
    return _lib.make_dl_tensor(t.data_ptr(), 0, code, list(t.shape), list(t.stride()), **kw)


def test_packed_call_runs_a_gemm(oracle):
    rng = np.random.default_rng(31)
    a = rng.uniform(-1, 1, (264, 200)).astype(np.float16)
    b = rng.uniform(-1, 1, (200, 136)).astype(np.float16)
    ta, tb = torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)
    tc = torch.full((264, 136), 7.0, dtype=torch.float32, device=DEV)
    d = _lib.gemm_desc(264, 136, 200)
    (da, ka), (db, kb), (dc, kc) = _dl(ta), _dl(tb), _dl(tc)
    assert _lib.packed_call(d, [da, db, dc]) == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert oracle.rel_l2(tc.cpu().numpy(), oracle.c_gemm(a, b, "te_llvm")) <= 1e-3
    # the same call on a stream of the caller's, set the way TVMSetStream would
    st = torch.cuda.Stream(DEV)
    tc.fill_(7.0)
    torch.cuda.synchronize()
    lib = _lib.load()
    assert lib.amosb_set_stream(0, ctypes.c_void_p(st.cuda_stream)) == 0
    try:
        assert _lib.packed_call(d, [da, db, dc], [13, 13, 13]) == 0, _lib.last_error()
        st.synchronize()
    finally:
        lib.amosb_set_stream(0, None)
    assert oracle.rel_l2(tc.cpu().numpy(), oracle.c_gemm(a, b, "te_llvm")) <= 1e-3


def test_packed_call_bfloat16_and_conv_scratch(oracle):
    """bfloat16 tensors (kDLBfloat) and an NCHW conv, whose scratch the library provides itself."""
    rng = np.random.default_rng(32)
    a = torch.from_numpy(rng.uniform(-1, 1, (136, 72)).astype(np.float32)).to(DEV).bfloat16()
    b = torch.from_numpy(rng.uniform(-1, 1, (72, 80)).astype(np.float32)).to(DEV).bfloat16()
    c = torch.empty((136, 80), dtype=torch.float32, device=DEV)
    d = _lib.gemm_desc(136, 80, 72, in_dtype=_lib.AMOSB_BF16)
    (da, ka), (db, kb), (dc, kc) = _dl(a), _dl(b), _dl(c)
    assert da.dtype.code == _lib.DL_BFLOAT
    assert _lib.packed_call(d, [da, db, dc]) == 0, _lib.last_error()
    torch.cuda.synchronize()
    ref = a.float().cpu().numpy().astype(np.float64) @ b.float().cpu().numpy().astype(np.float64)
    assert oracle.rel_l2(c.cpu().numpy(), ref) <= 2e-5

    x = rng.uniform(-1, 1, (3, 24, 10, 10)).astype(np.float16)
    w = rng.normal(0, 0.05, (40, 24, 3, 3)).astype(np.float16)
    tx, tw = torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV)
    ty = torch.empty((3, 40, 10, 10), dtype=torch.float32, device=DEV)
    dconv = _lib.conv2d_desc(3, 24, 10, 10, 40, 3, 3, pad=1)
    assert _lib.workspace_bytes_min(dconv) > 0
    (dx, kx), (dw, kw), (dy, ky) = _dl(tx), _dl(tw), _dl(ty)
    for _ in range(2):
        assert _lib.packed_call(dconv, [dx, dw, dy]) == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert oracle.rel_l2(ty.cpu().numpy(), oracle.c_conv2d_nchw(x, w, 1, 1, 1, "te_llvm")) <= 1e-3


def test_packed_call_refuses_host_and_wrong_device_memory():
    a = torch.zeros((64, 48), dtype=torch.float16).pin_memory()
    b = torch.zeros((48, 32), dtype=torch.float16, device=DEV)
    c = torch.full((64, 32), 7.0, dtype=torch.float32, device=DEV)
    d = _lib.gemm_desc(64, 32, 48)
    (da, ka), (db, kb), (dc, kc) = _dl(a), _dl(b), _dl(c)
    assert _lib.packed_call(d, [da, db, dc]) == -1
    assert "device_type is expected to be cuda" in _lib.last_error()
    torch.cuda.synchronize()
    assert (c == 7.0).all()


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(oracle):
    """The copy-issuing threads are told to issue nothing (a launch parameter), so nothing is in
    flight; the MMA thread's wait for a filled stage runs out after a few milliseconds, the CTA
    records status 102, frees its TMEM and returns.  The host sees -4 once, the context is intact
    and the next ordinary call is bit-correct."""
    lib = _lib.load()
    assert lib.amosb_sync_check(0) == 0
    rng = np.random.default_rng(33)
    a = rng.uniform(-1, 1, (128, 128)).astype(np.float16)
    b = rng.uniform(-1, 1, (128, 128)).astype(np.float16)
    ta, tb = torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)
    tc = torch.zeros((128, 128), dtype=torch.float32, device=DEV)
    d = _lib.gemm_desc(128, 128, 128, tile_n=128, cta_pair=1)  # one CTA of the single-CTA kernel
    os.environ["AMOSB_WAIT_BUDGET_NS"] = "3000000"
    os.environ["AMOSB_DIAG_NO_LOADS"] = "1"
    try:
        assert device.run(d, [ta, tb], [tc]) == 1
    finally:
        del os.environ["AMOSB_WAIT_BUDGET_NS"]
        del os.environ["AMOSB_DIAG_NO_LOADS"]
    torch.cuda.synchronize()  # the kernel returned by itself; no error is pending
    assert lib.amosb_status_peek(0, 0) == 102
    assert lib.amosb_sync_check(0) == _lib.AMOSB_ERR_DEVICE_TIMEOUT
    assert "status 102" in _lib.last_error()
    assert lib.amosb_sync_check(0) == 0  # reported once, then clear
    tc.zero_()
    device.run(d, [ta, tb], [tc])
    torch.cuda.synchronize()
    assert oracle.rel_l2(tc.cpu().numpy(), oracle.c_gemm(a, b, "te_llvm")) <= 1e-3
    assert np.array_equal(tc.cpu().numpy(), _again(d, ta, tb))


def _again(d, ta, tb):
    out = torch.zeros((128, 128), dtype=torch.float32, device=DEV)
    device.run(d, [ta, tb], [out])
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_host_buffer_call_returns_the_timeout_code():
    """amosb_run_host reads the status word behind its last copy: a kernel that gave up a wait makes
    the call fail with -4 instead of handing back numbers."""
    from amos_b200 import runtime
    a = np.ones((128, 128), np.float16)
    b = np.ones((128, 128), np.float16)
    c = np.zeros((128, 128), np.float32)
    mod = runtime.Module(_lib.gemm_desc(128, 128, 128, tile_n=128, cta_pair=1))
    os.environ["AMOSB_WAIT_BUDGET_NS"] = "3000000"
    os.environ["AMOSB_DIAG_NO_LOADS"] = "1"
    try:
        with pytest.raises(_lib.AmosbError) as err:
            mod(a, b, c)
    finally:
        del os.environ["AMOSB_WAIT_BUDGET_NS"]
        del os.environ["AMOSB_DIAG_NO_LOADS"]
    assert err.value.code == _lib.AMOSB_ERR_DEVICE_TIMEOUT
    assert _lib.load().amosb_sync_check(0) == 0
    mod(a, b, c)
    assert (c == 128.0).all()

"""GPU: the conv2d entry point that allocates nothing (amosb_conv2d_nchw_static).

It serves callers that cannot obtain device memory at call time -- a host process that handed the
whole GPU to its own arena, a plugin interface without an allocator, a loop that must not hit the
device-wide synchronisation of cudaMalloc -- by keeping the conv scratch in an array built into
the library.  The test calls it through the C ABI twice in a row (different data the second time,
so that anything left in the shared array by the first call would show) and requires the same
bits as the existing entry point amosb_run, which gets its scratch from the caller.

Collected last (file name) so that a run that stops at the first failure has already run every
other test; it passes alone in a fresh process and after the rest of the suite.
"""
import ctypes

import numpy as np
import pytest
import torch

from amos_b200 import _lib, device

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _static_call(desc, x, w, out):
    lib = _lib.load()
    keep = []
    ins = (_lib.AmosbTensor * 2)()
    for i, t in enumerate((x, w)):
        ins[i], k = device.tensor_arg(t)
        keep.append(k)
    outs = (_lib.AmosbTensor * 1)()
    outs[0], k = device.tensor_arg(out)
    keep.append(k)
    stream = torch.cuda.current_stream(0)
    rc = lib.amosb_conv2d_nchw_static(ctypes.byref(desc), ins, 2, outs, 1,
                                      ctypes.c_void_p(stream.cuda_stream))
    return rc


def test_static_scratch_matches_caller_scratch_twice(oracle):
    rng = np.random.default_rng(99)
    desc = _lib.conv2d_desc(1, 64, 56, 56, 64, 3, 3, stride=1, pad=1)
    assert 0 < _lib.workspace_bytes_min(desc) <= _lib.STATIC_SCRATCH_BYTES
    for call in range(2):
        x_np = rng.uniform(-1, 1, (1, 64, 56, 56)).astype(np.float16)
        w_np = rng.uniform(-1, 1, (64, 64, 3, 3)).astype(np.float16)
        x = torch.from_numpy(x_np).to(DEV)
        w = torch.from_numpy(w_np).to(DEV)
        ref = torch.full((1, 64, 56, 56), float("nan"), dtype=torch.float32, device=DEV)
        device.run(desc, [x, w], [ref])  # existing entry point, caller-provided workspace
        got = torch.full((1, 64, 56, 56), float("nan"), dtype=torch.float32, device=DEV)
        rc = _static_call(desc, x, w, got)
        assert rc == _lib.AMOSB_OK, _lib.last_error()
        assert _lib.load().amosb_last_launch_count() == 2
        assert device.status_peek(0) == 0
        # same kernels, same inputs: the same bits
        assert torch.equal(got, ref), f"call {call}: outputs differ"
        # and both agree with the oracle within the tolerance of the parity tests
        err = oracle.rel_l2(got.cpu().numpy(), oracle.c_conv2d_nchw(x_np, w_np, 1, 1, 1, "te_llvm"))
        assert err <= 1e-3


def test_static_scratch_second_shape_and_limits():
    # a different geometry right after: channel padding (C=24 -> 64 in the filter) must not pick
    # up what the previous call left in the array
    rng = np.random.default_rng(100)
    desc = _lib.conv2d_desc(3, 24, 10, 9, 40, 3, 3, stride=1, pad=1)
    x = torch.from_numpy(rng.uniform(-1, 1, (3, 24, 10, 9)).astype(np.float16)).to(DEV)
    w = torch.from_numpy(rng.normal(0, 0.05, (40, 24, 3, 3)).astype(np.float16)).to(DEV)
    ref = torch.empty(3, 40, 10, 9, dtype=torch.float32, device=DEV)
    got = torch.empty_like(ref)
    device.run(desc, [x, w], [ref])
    assert _static_call(desc, x, w, got) == _lib.AMOSB_OK, _lib.last_error()
    assert device.status_peek(0) == 0
    assert torch.equal(got, ref)
    # beyond the built-in maximum: refused with a message, nothing launched
    big = _lib.conv2d_desc(256, 128, 28, 28, 128, 3, 3, stride=1, pad=1)
    assert _lib.workspace_bytes_min(big) > _lib.STATIC_SCRATCH_BYTES
    xb = torch.zeros(256, 128, 28, 28, dtype=torch.float16, device=DEV)
    wb = torch.zeros(128, 128, 3, 3, dtype=torch.float16, device=DEV)
    ob = torch.full((256, 128, 28, 28), 5.0, dtype=torch.float32, device=DEV)
    assert _static_call(big, xb, wb, ob) == _lib.AMOSB_ERR_UNSUPPORTED
    assert "AMOSB_STATIC_SCRATCH_BYTES" in _lib.last_error()
    torch.cuda.synchronize()
    assert (ob == 5.0).all()
    # a GEMM descriptor is not accepted by this entry point
    g = _lib.gemm_desc(64, 64, 64)
    assert _static_call(g, xb, wb, ob) == _lib.AMOSB_ERR_ARG

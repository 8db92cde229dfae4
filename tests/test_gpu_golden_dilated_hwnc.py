"""GPU: the kernels on the committed inputs of tests/golden/ref_topi_dilated_and_hwnc.npz against
what the reference's own test helpers gave for them: dilated layers (`dilate_python` on the filter +
the undilated conv helper) in NCHW and NHWC, and the HWNC layout (`conv2d_hwcn_python` with the
last two axes exchanged).  int8 bit for bit; float16 within 2e-5 of the exact sums."""
import os

import numpy as np
import pytest
import torch

from amos_b200 import _lib, device

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_EXACT = 2e-5


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def _run(desc, a, w, shape):
    i8 = a.dtype == np.int8
    out = torch.full(shape, 77 if i8 else float("nan"), dtype=torch.int32 if i8 else torch.float32,
                     device=DEV)
    device.run(desc, [_t(a), _t(w)], [out])
    assert device.status_peek(0) == 0
    return out.cpu().numpy()


def _check(got, ref, i8, what):
    assert got.shape == ref.shape, what
    if i8:
        assert np.array_equal(got, ref.astype(np.int64)), what
    else:
        err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
        assert err <= TOL_EXACT, (what, err)


def test_dilated_layers_against_the_reference_helpers(golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_topi_dilated_and_hwnc.npz"))
    for i in range(int(g["num_dil"])):
        a, w, ref = g[f"dil{i}_a"], g[f"dil{i}_w"], g[f"dil{i}_out"]
        stride, pad, dil = (int(v) for v in g[f"dil{i}_geom"])
        i8 = a.dtype == np.int8
        in_dtype = _lib.AMOSB_S8 if i8 else _lib.AMOSB_F16
        if str(g[f"dil{i}_layout"]) == "nchw":
            n, c, h, wd = a.shape
            k, _, r, s = w.shape
            d = _lib.conv2d_desc(n, c, h, wd, k, r, s, stride, pad, dil)
            _lib._set_conv_in_dtype(d, in_dtype)
            shape = (n, k, d.conv_p, d.conv_q)
        else:
            n, h, wd, c = a.shape
            r, s, _, k = w.shape
            d = _lib.conv2d_nhwc_desc(n, h, wd, c, k, r, s, stride, pad, dil, in_dtype=in_dtype)
            shape = (n, d.conv_p, d.conv_q, k)
        _check(_run(d, a, w, shape), ref, i8, f"dilated case {i}")


@pytest.mark.parametrize("packing", [True, False])
def test_hwnc_against_the_reference_hwcn_helper(golden_dir, packing):
    g = np.load(os.path.join(golden_dir, "ref_topi_dilated_and_hwnc.npz"))
    if not packing:
        os.environ["AMOSB_HWNC_NO_PACKING"] = "1"
    try:
        for i in range(int(g["num_hwnc"])):
            a, w, ref = g[f"hwnc{i}_a"], g[f"hwnc{i}_w"], g[f"hwnc{i}_out"]
            stride, pad, dil = (int(v) for v in g[f"hwnc{i}_geom"])
            i8 = a.dtype == np.int8
            h, wd, n, c = a.shape
            r, s, _, k = w.shape
            d = _lib.conv2d_hwnc_desc(h, wd, n, c, k, r, s, stride, pad, dil,
                                      in_dtype=_lib.AMOSB_S8 if i8 else _lib.AMOSB_F16)
            _check(_run(d, a, w, (d.conv_p, d.conv_q, n, k)), ref, i8, f"hwnc case {i}")
    finally:
        os.environ.pop("AMOSB_HWNC_NO_PACKING", None)

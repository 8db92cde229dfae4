"""GPU: the CUDA path, called through the C ABI, against the CPU oracle.

Bars: int8 -> int32 bit exact against the oracle's `exact` mode; fp16 relative L2 error <= 1e-3
against the oracle's `te_llvm` mode (the reference's own CPU build of the same `te` compute), and,
as a tighter sanity bound, <= 2e-5 against `exact` (fp32 vs fp64 accumulation of exact products).
"""
import os

import numpy as np
import pytest
import torch

from amos_b200 import _lib, device

pytestmark = pytest.mark.gpu

TOL_TE_LLVM = 1e-3
TOL_EXACT = 2e-5
DEV = "cuda:0"


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def _run_gemm(a, b, out_dtype, trans_b=False, tile_n=0, cta_pair=0, trans_a=False):
    i8 = a.dtype == np.int8
    batched = a.ndim == 3
    m, k = a.shape[-2:]
    if trans_a:
        k, m = m, k
    n = b.shape[-2] if trans_b else b.shape[-1]
    d = _lib.gemm_desc(m, n, k, in_dtype=_lib.AMOSB_S8 if i8 else _lib.AMOSB_F16,
                       out_dtype=_lib.DTYPE_CODES[out_dtype], batch=a.shape[0] if batched else 1,
                       trans_b=trans_b, batched=batched, tile_n=tile_n, cta_pair=cta_pair,
                       trans_a=trans_a)
    shape = (a.shape[0], m, n) if batched else (m, n)
    # guard band around the output: nothing outside the tensor may be written
    tdt = device.CODE_TO_TORCH[d.out_dtype]
    numel = int(np.prod(shape))
    buf = torch.full((numel + 2048,), 77, dtype=tdt, device=DEV)
    out = buf[1024:1024 + numel].view(shape)
    launches = device.run(d, [_t(a), _t(b)], [out])
    assert launches == 1
    assert device.status_peek(0) == 0
    assert (buf[:1024] == 77).all() and (buf[1024 + numel:] == 77).all(), "wrote outside C"
    return out.cpu().numpy()


def _run_conv(x, w, stride, pad, dil, out_dtype="float32", tile_n=0, cta_pair=0,
              launches_expected=None):
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    d = _lib.conv2d_desc(n, c, h, wd, k, r, s, stride, pad, dil,
                         out_dtype=_lib.DTYPE_CODES[out_dtype], tile_n=tile_n, cta_pair=cta_pair)
    shape = (n, k, d.conv_p, d.conv_q)
    numel = int(np.prod(shape))
    tdt = device.CODE_TO_TORCH[d.out_dtype]
    buf = torch.full((numel + 2048,), 77, dtype=tdt, device=DEV)
    out = buf[1024:1024 + numel].view(shape)
    launches = device.run(d, [_t(x), _t(w)], [out])
    # a 1x1 / stride 1 / unpadded layer whose planes are multiples of 4 pixels runs in place (as one
    # batched GEMM when the planes are 16-byte multiples, else with the activation copied in by
    # cp.async); every other geometry re-lays-out both operands first (one launch) and then runs
    # the implicit GEMM
    pointwise = (r == 1 and s == 1 and stride == 1 and pad == 0 and (h * wd) % 4 == 0
                 and c % 8 == 0 and "AMOSB_CONV_NO_POINTWISE" not in os.environ)
    if launches_expected is None:
        launches_expected = 1 if pointwise else 2
    assert launches == launches_expected
    assert device.status_peek(0) == 0
    assert (buf[:1024] == 77).all() and (buf[1024 + numel:] == 77).all(), "wrote outside Out"
    return out.cpu().numpy()


# ------------------------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("shape", [(128, 64, 64), (1, 8, 8), (7, 24, 16), (200, 136, 72),
                                   (256, 256, 256), (1000, 520, 264), (129, 264, 1032)])
@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_f16(oracle, shape, trans_b):
    m, n, k = shape
    rng = np.random.default_rng(m * 31 + n)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (n, k) if trans_b else (k, n)).astype(np.float16)
    got = _run_gemm(a, b, "float32", trans_b)
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "te_llvm", trans_b=trans_b)) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "exact", trans_b=trans_b)) <= TOL_EXACT


@pytest.mark.parametrize("n", [77, 130, 3])
def test_gemm_rows_of_c_not_16_byte_multiples(oracle, n):
    """B given as [N,K]: N is then free of TMA alignment rules, and C rows that are not 16-byte
    multiples take the plain-store epilogue instead of TMA stores."""
    rng = np.random.default_rng(n)
    a = rng.uniform(-1, 1, (150, 72)).astype(np.float16)
    b = rng.uniform(-1, 1, (n, 72)).astype(np.float16)
    got = _run_gemm(a, b, "float32", trans_b=True)
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "te_llvm", trans_b=True)) <= TOL_TE_LLVM
    got16 = _run_gemm(a, b, "float16", trans_b=True)
    assert np.array_equal(got16, got.astype(np.float16))
    ai = rng.integers(-128, 128, (150, 80), dtype=np.int8)
    bi = rng.integers(-128, 128, (n, 80), dtype=np.int8)
    assert np.array_equal(_run_gemm(ai, bi, "int32", trans_b=True),
                          oracle.c_gemm(ai, bi, "exact", trans_b=True))


@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_gemm_f16_tile_variants_and_cast(oracle, tile_n):
    rng = np.random.default_rng(tile_n)
    a = rng.uniform(-1, 1, (384, 320)).astype(np.float16)
    b = rng.uniform(-1, 1, (320, 520)).astype(np.float16)
    got32 = _run_gemm(a, b, "float32", tile_n=tile_n)
    got16 = _run_gemm(a, b, "float16", tile_n=tile_n)
    assert got16.dtype == np.float16
    # the fp16 output is the fp32 result rounded once (the trailing astype stage)
    assert np.array_equal(got16, got32.astype(np.float16))
    ref16 = oracle.c_gemm(a, b, "te_llvm", out_dtype="float16")
    assert oracle.rel_l2(got16, ref16) <= TOL_TE_LLVM


@pytest.mark.parametrize("shape", [(128, 128, 128), (1, 16, 16), (200, 144, 80), (256, 256, 512),
                                   (1000, 528, 272), (130, 272, 2064)])
@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_s8_bit_exact(oracle, shape, trans_b):
    m, n, k = shape
    rng = np.random.default_rng(m * 17 + k)
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (n, k) if trans_b else (k, n), dtype=np.int8)
    got = _run_gemm(a, b, "int32", trans_b)
    assert np.array_equal(got, oracle.c_gemm(a, b, "exact", trans_b=trans_b))


def test_gemm_s8_extremes(oracle):
    """Largest magnitudes: 2064 * (-128 * -128) and 2064 * (-128 * 127)."""
    a = np.full((130, 2064), -128, dtype=np.int8)
    b = np.full((2064, 144), -128, dtype=np.int8)
    b[:, ::2] = 127
    got = _run_gemm(a, b, "int32")
    assert np.array_equal(got, oracle.c_gemm(a, b, "exact"))
    assert got.max() == 2064 * 16384 and got.min() == 2064 * -16256


@pytest.mark.parametrize("tile_n", [128, 256])
def test_gemm_s8_tile_variants(oracle, tile_n):
    rng = np.random.default_rng(3)
    a = rng.integers(-128, 128, (300, 400), dtype=np.int8)
    b = rng.integers(-128, 128, (400, 528), dtype=np.int8)
    assert np.array_equal(_run_gemm(a, b, "int32", tile_n=tile_n), oracle.c_gemm(a, b, "exact"))


@pytest.mark.parametrize("cta_pair", [1, 2])
def test_single_cta_and_cta_pair_kernels_agree(oracle, cta_pair):
    """Both kernel families (one CTA per 128-row tile, CTA pairs per 256-row tile) on the same
    problems, forced through the descriptor; ragged M/N/K, both B layouts, all output types."""
    rng = np.random.default_rng(41)
    a = rng.uniform(-1, 1, (300, 200)).astype(np.float16)
    b = rng.uniform(-1, 1, (200, 264)).astype(np.float16)
    ref = oracle.c_gemm(a, b, "te_llvm")
    for tile_n in (128, 256):
        got = _run_gemm(a, b, "float32", tile_n=tile_n, cta_pair=cta_pair)
        assert oracle.rel_l2(got, ref) <= TOL_TE_LLVM
        got_t = _run_gemm(a, np.ascontiguousarray(b.T), "float32", trans_b=True, tile_n=tile_n,
                          cta_pair=cta_pair)
        assert np.array_equal(got, got_t)
        assert np.array_equal(_run_gemm(a, b, "float16", tile_n=tile_n, cta_pair=cta_pair),
                              got.astype(np.float16))
    ai = rng.integers(-128, 128, (520, 400), dtype=np.int8)
    bi = rng.integers(-128, 128, (400, 528), dtype=np.int8)
    assert np.array_equal(_run_gemm(ai, bi, "int32", cta_pair=cta_pair),
                          oracle.c_gemm(ai, bi, "exact"))
    assert np.array_equal(_run_gemm(ai, np.ascontiguousarray(bi.T), "int32", trans_b=True,
                                    tile_n=128, cta_pair=cta_pair), oracle.c_gemm(ai, bi, "exact"))
    x = rng.uniform(-1, 1, (3, 72, 9, 11)).astype(np.float16)
    w = rng.normal(0, 0.05, (300, 72, 3, 3)).astype(np.float16)
    got = _run_conv(x, w, 1, 1, 1, cta_pair=cta_pair)
    assert oracle.rel_l2(got, oracle.c_conv2d_nchw(x, w, 1, 1, 1, "te_llvm")) <= TOL_TE_LLVM


def test_cta_pair_partial_last_wave(oracle):
    """80-96 pair tiles on 74 pairs: one full wave and a partial one (K-major and MN-major B, int8,
    conv)."""
    rng = np.random.default_rng(43)
    a = rng.uniform(-1, 1, (2560, 192)).astype(np.float16)
    b = rng.uniform(-1, 1, (192, 2112)).astype(np.float16)
    got = _run_gemm(a, b, "float32", cta_pair=2)
    ref = torch.from_numpy(a).to(DEV).float() @ torch.from_numpy(b).to(DEV).float()
    assert oracle.rel_l2(got, ref.cpu().numpy()) <= TOL_EXACT
    rows = [0, 255, 256, 1279, 2559]
    assert oracle.rel_l2(got[rows], oracle.c_gemm(a[rows], b, "te_llvm")) <= TOL_TE_LLVM
    got_t = _run_gemm(a, np.ascontiguousarray(b.T), "float32", trans_b=True, cta_pair=2)
    assert np.array_equal(got, got_t)
    ai = rng.integers(-128, 128, (1320, 320), dtype=np.int8)
    bi = rng.integers(-128, 128, (320, 4096), dtype=np.int8)
    ref_i = (torch.from_numpy(ai).to(DEV).double() @ torch.from_numpy(bi).to(DEV).double())
    ref_i = ref_i.to(torch.int32).cpu().numpy()
    assert np.array_equal(_run_gemm(ai, bi, "int32", cta_pair=2), ref_i)
    assert np.array_equal(_run_gemm(ai, np.ascontiguousarray(bi.T), "int32", trans_b=True,
                                    cta_pair=2), ref_i)
    x = rng.uniform(-1, 1, (40, 64, 16, 16)).astype(np.float16)
    w = rng.normal(0, 0.05, (512, 64, 3, 3)).astype(np.float16)
    got = _run_conv(x, w, 1, 1, 1, cta_pair=2)
    imgs = [0, 17, 39]
    assert oracle.rel_l2(got[imgs], oracle.c_conv2d_nchw(x[imgs], w, 1, 1, 1, "te_llvm")) \
        <= TOL_TE_LLVM
    assert np.array_equal(got, _run_conv(x, w, 1, 1, 1, cta_pair=1))


def test_one_hot_operands_locate_every_element():
    """A = I picks rows of B exactly: any mis-addressed tile or swizzle shows up as a moved value."""
    n = 256
    a = np.eye(n, dtype=np.float16)
    b = (np.arange(n * n, dtype=np.float32).reshape(n, n) % 2039).astype(np.float16)
    assert np.array_equal(_run_gemm(a, b, "float32"), b.astype(np.float32))
    ai = np.eye(n, dtype=np.int8)
    bi = ((np.arange(n * n).reshape(n, n) % 251) - 125).astype(np.int8)
    assert np.array_equal(_run_gemm(ai, bi, "int32"), bi.astype(np.int32))


@pytest.mark.parametrize("shape", [(4, 512, 512, 64), (4, 512, 64, 512), (3, 100, 72, 40),
                                   (5, 130, 264, 72)])
def test_batched_gemm(oracle, shape):
    bt, m, n, k = shape
    rng = np.random.default_rng(bt * 1000 + m)
    a = rng.normal(0, 1, (bt, m, k)).astype(np.float16)
    b = rng.normal(0, 1, (bt, k, n)).astype(np.float16)
    got = _run_gemm(a, b, "float16")
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "te_llvm", out_dtype="float16")) <= TOL_TE_LLVM
    got32 = _run_gemm(a, b, "float32")
    assert oracle.rel_l2(got32, oracle.c_gemm(a, b, "exact")) <= TOL_EXACT


# --------------------------------------------------------------------- fused trailing stages
def _fused_ref(acc, addend, relu, out_dtype):
    """te semantics of the trailing stages: each is its own element-wise stage on the
    materialised accumulator: add in the accumulator dtype, max with 0, then the cast."""
    x = acc
    if addend is not None:
        x = (x + addend.astype(acc.dtype)).astype(acc.dtype)
    if relu:
        x = np.maximum(x, 0)
    return x.astype(out_dtype)


@pytest.mark.parametrize("cta_pair", [1, 2])
@pytest.mark.parametrize("bias", ["vector", "full"])
def test_gemm_fused_bias_relu_cast(oracle, bias, cta_pair):
    rng = np.random.default_rng(7 + cta_pair)
    m, n, k = 300, 264, 200
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    for addend_dtype, out_dtype, relu in (("float32", "float32", True), ("float16", "float16", True),
                                          ("float32", "float16", False)):
        add = rng.uniform(-2, 2, (n,) if bias == "vector" else (m, n)).astype(addend_dtype)
        d = _lib.gemm_desc(m, n, k, out_dtype=_lib.DTYPE_CODES[out_dtype], cta_pair=cta_pair)
        d.epilogue = (_lib.EPI_ADD_VECTOR if bias == "vector" else _lib.EPI_ADD_FULL) | \
            (_lib.EPI_RELU if relu else 0)
        d.addend_dtype = _lib.DTYPE_CODES[addend_dtype]
        d.arg_c = 2
        out = torch.full((m, n), float("nan"), dtype=device.CODE_TO_TORCH[d.out_dtype], device=DEV)
        assert device.run(d, [_t(a), _t(b), _t(add)], [out]) == 1
        assert device.status_peek(0) == 0
        addb = add[None, :] if bias == "vector" else add
        ref = _fused_ref(oracle.c_gemm(a, b, "te_llvm"), addb, relu, out_dtype)
        assert oracle.rel_l2(out.cpu().numpy(), ref) <= TOL_TE_LLVM
        exact = _fused_ref(oracle.c_gemm(a, b, "exact"), addb, relu, "float32")
        assert oracle.rel_l2(out.cpu().numpy(), exact) <= (3e-4 if out_dtype == "float16" else TOL_EXACT)
        if relu:
            assert (out >= 0).all()


def test_gemm_s8_fused_bias_relu_bit_exact(oracle):
    rng = np.random.default_rng(9)
    a = rng.integers(-128, 128, (260, 400), dtype=np.int8)
    b = rng.integers(-128, 128, (400, 272), dtype=np.int8)
    bias = rng.integers(-100000, 100000, (272,), dtype=np.int32)
    full = rng.integers(-100000, 100000, (260, 272), dtype=np.int32)
    acc = oracle.c_gemm(a, b, "exact")
    for cta_pair in (1, 2):
        for flags, add, addb in ((_lib.EPI_ADD_VECTOR | _lib.EPI_RELU, bias, bias[None, :]),
                                 (_lib.EPI_ADD_FULL, full, full)):
            d = _lib.gemm_desc(260, 272, 400, in_dtype=_lib.AMOSB_S8, cta_pair=cta_pair)
            d.epilogue, d.addend_dtype, d.arg_c = flags, _lib.AMOSB_S32, 2
            out = torch.zeros(260, 272, dtype=torch.int32, device=DEV)
            device.run(d, [_t(a), _t(b), _t(add)], [out])
            ref = acc + addb
            if flags & _lib.EPI_RELU:
                ref = np.maximum(ref, 0)
            assert np.array_equal(out.cpu().numpy(), ref)


@pytest.mark.parametrize("cfg", [(3, 72, 9, 11, 300, 3, 3, 1), (2, 64, 16, 16, 64, 3, 3, 1),
                                 (2, 64, 8, 8, 136, 1, 1, 0), (2, 200, 10, 10, 72, 1, 1, 0)])
@pytest.mark.parametrize("bias", ["vector", "full"])
def test_conv2d_fused_bias_relu(oracle, cfg, bias):
    """Per-channel bias (and a residual of the output's shape) + ReLU on both conv paths: the
    im2col kernel and the 1x1 layers that run as batched GEMMs (bias then follows the GEMM rows)."""
    n, c, h, w, k, r, s, pad = cfg
    rng = np.random.default_rng(n * 7 + k)
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float16)
    wt = rng.normal(0, 0.05, (k, c, r, s)).astype(np.float16)
    for cta_pair in (1, 2):
        d = _lib.conv2d_desc(n, c, h, w, k, r, s, 1, pad, 1, cta_pair=cta_pair)
        add = rng.uniform(-1, 1, (k,) if bias == "vector" else (n, k, d.conv_p, d.conv_q)) \
            .astype(np.float32)
        d.epilogue = (_lib.EPI_ADD_VECTOR if bias == "vector" else _lib.EPI_ADD_FULL) | _lib.EPI_RELU
        d.addend_dtype, d.arg_c = _lib.AMOSB_F32, 2
        out = torch.full((n, k, d.conv_p, d.conv_q), float("nan"), dtype=torch.float32, device=DEV)
        device.run(d, [_t(x), _t(wt), _t(add)], [out])
        assert device.status_peek(0) == 0
        addb = add[None, :, None, None] if bias == "vector" else add
        ref = _fused_ref(oracle.c_conv2d_nchw(x, wt, 1, pad, 1, "te_llvm"), addb, True, "float32")
        assert oracle.rel_l2(out.cpu().numpy(), ref) <= TOL_TE_LLVM


def test_unsupported_shapes_fail_cleanly():
    a = torch.zeros(64, 36, dtype=torch.float16, device=DEV)  # K*2 bytes not a multiple of 16
    b = torch.zeros(36, 64, dtype=torch.float16, device=DEV)
    c = torch.zeros(64, 64, dtype=torch.float32, device=DEV)
    with pytest.raises(_lib.AmosbError) as e:
        device.run(_lib.gemm_desc(64, 64, 36), [a, b], [c])
    assert e.value.code == _lib.AMOSB_ERR_UNSUPPORTED
    # conv without workspace
    lib = _lib.load()
    x = torch.zeros(1, 64, 8, 8, dtype=torch.float16, device=DEV)
    w = torch.zeros(64, 64, 3, 3, dtype=torch.float16, device=DEV)
    y = torch.zeros(1, 64, 8, 8, dtype=torch.float32, device=DEV)
    import ctypes
    cd = _lib.conv2d_desc(1, 64, 8, 8, 64, 3, 3, pad=1)
    ins = (_lib.AmosbTensor * 2)(device.tensor_arg(x)[0], device.tensor_arg(w)[0])
    outs = (_lib.AmosbTensor * 1)(device.tensor_arg(y)[0])
    assert lib.amosb_run(ctypes.byref(cd), ins, 2, outs, 1, None, 0, None) == _lib.AMOSB_ERR_ARG
    assert "workspace" in _lib.last_error()
    assert device.status_peek(0) == 0


# ---------------------------------------------------------------------------- transposed A
@pytest.mark.parametrize("shape", [(128, 64, 64), (8, 8, 8), (200, 136, 72), (1000, 520, 264),
                                   (136, 264, 1032)])
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("tile_n", [0, 64, 256])
def test_gemm_f16_a_stored_k_by_m(oracle, shape, trans_b, tile_n):
    """A[k, i] (stored [K, M]) is consumed in place as an MN-major operand; the result is the one
    of the same GEMM on the transposed copy, bit for bit (same products, same order)."""
    m, n, k = shape
    rng = np.random.default_rng(m * 17 + n + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (n, k) if trans_b else (k, n)).astype(np.float16)
    at_ = np.ascontiguousarray(a.T)
    got = _run_gemm(at_, b, "float32", trans_b, tile_n=tile_n, trans_a=True)
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "te_llvm", trans_b=trans_b)) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "exact", trans_b=trans_b)) <= TOL_EXACT
    tn = tile_n if tile_n else 0
    assert np.array_equal(got, _run_gemm(a, b, "float32", trans_b, tile_n=tn, cta_pair=1))
    got16 = _run_gemm(at_, b, "float16", trans_b, tile_n=tile_n, trans_a=True)
    assert np.array_equal(got16, got.astype(np.float16))


@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_i8_a_stored_k_by_m(oracle, trans_b):
    rng = np.random.default_rng(99)
    a = rng.integers(-128, 128, (272, 400), dtype=np.int8)
    b = rng.integers(-128, 128, (144, 400) if trans_b else (400, 144), dtype=np.int8)
    got = _run_gemm(np.ascontiguousarray(a.T), b, "int32", trans_b, trans_a=True)
    assert np.array_equal(got, oracle.c_gemm(a, b, "exact", trans_b=trans_b))


def test_batched_gemm_a_stored_k_by_m(oracle):
    rng = np.random.default_rng(98)
    a = rng.normal(0, 1, (6, 264, 72)).astype(np.float16)
    b = rng.normal(0, 1, (6, 72, 136)).astype(np.float16)
    got = _run_gemm(np.ascontiguousarray(a.transpose(0, 2, 1)), b, "float16", trans_a=True)
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "te_llvm", out_dtype="float16")) <= TOL_TE_LLVM


def test_a_stored_k_by_m_needs_16_byte_rows():
    a = torch.zeros(64, 36, dtype=torch.float16, device=DEV)   # [K, M] with M*2 = 72 bytes
    b = torch.zeros(64, 64, dtype=torch.float16, device=DEV)
    c = torch.zeros(36, 64, dtype=torch.float32, device=DEV)
    with pytest.raises(_lib.AmosbError) as e:
        device.run(_lib.gemm_desc(36, 64, 64, trans_a=True), [a, b], [c])
    assert e.value.code == _lib.AMOSB_ERR_UNSUPPORTED
    with pytest.raises(_lib.AmosbError):
        device.run(_lib.gemm_desc(64, 64, 64, trans_a=True, cta_pair=2),
                   [torch.zeros(64, 64, dtype=torch.float16, device=DEV), b],
                   [torch.zeros(64, 64, dtype=torch.float32, device=DEV)])
    assert device.status_peek(0) == 0


# ------------------------------------------------------------------------------ tall tiles
@pytest.mark.parametrize("shape", [(300, 136, 72), (256, 128, 64), (1000, 264, 520), (129, 72, 200),
                                   (2048, 128, 1024)])
@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_tall_tiles(oracle, shape, trans_b):
    """cta_pair = 3: one CTA per 256 x 128 tile, two accumulators sharing every B stage; ragged M
    leaves the second accumulator partly or wholly past the last row."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (n, k) if trans_b else (k, n)).astype(np.float16)
    assert "tall" in _lib.describe_plan(_lib.gemm_desc(m, n, k, trans_b=trans_b, tile_n=128,
                                                       cta_pair=3))
    got = _run_gemm(a, b, "float32", trans_b, tile_n=128, cta_pair=3)
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "te_llvm", trans_b=trans_b)) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "exact", trans_b=trans_b)) <= TOL_EXACT
    # same products, same order of accumulation as the 128-row tiles of the same width
    assert np.array_equal(got, _run_gemm(a, b, "float32", trans_b, tile_n=128, cta_pair=1))
    got16 = _run_gemm(a, b, "float16", trans_b, tile_n=128, cta_pair=3)
    assert np.array_equal(got16, got.astype(np.float16))


def test_batched_gemm_tall_tiles(oracle):
    rng = np.random.default_rng(77)
    a = rng.normal(0, 1, (5, 384, 64)).astype(np.float16)
    b = rng.normal(0, 1, (5, 64, 136)).astype(np.float16)
    got = _run_gemm(a, b, "float16", tile_n=128, cta_pair=3)
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "te_llvm", out_dtype="float16")) <= TOL_TE_LLVM


@pytest.mark.parametrize("cfg", [(3, 72, 9, 11, 40, 3, 3, 1, 1, 1), (2, 64, 14, 14, 64, 3, 3, 1, 1, 1),
                                 (5, 128, 7, 7, 136, 3, 3, 1, 1, 1), (2, 64, 15, 15, 64, 3, 3, 2, 1, 1),
                                 (9, 64, 12, 12, 128, 3, 3, 1, 1, 1)])
def test_conv2d_tall_tiles(oracle, cfg):
    n, c, h, w, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n * 100 + c + 1)
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float16)
    wt = rng.normal(0, 0.05, (k, c, r, s)).astype(np.float16)
    got = _run_conv(x, wt, st, pad, dil, tile_n=128, cta_pair=3)
    assert oracle.rel_l2(got, oracle.c_conv2d_nchw(x, wt, st, pad, dil, "te_llvm")) <= TOL_TE_LLVM
    assert np.array_equal(got, _run_conv(x, wt, st, pad, dil, tile_n=128, cta_pair=1))


# ------------------------------------------------------------------------------------------ conv
CONV_CASES = [
    # N, C, H, W, K, R, S, stride, pad, dil
    (1, 64, 8, 8, 64, 1, 1, 1, 0, 1),
    (1, 64, 16, 16, 64, 3, 3, 1, 1, 1),
    (2, 64, 14, 14, 64, 3, 3, 1, 1, 1),      # 392 pixels: tiles straddle images
    (3, 72, 9, 11, 40, 3, 3, 1, 1, 1),       # ragged channels and filters
    (2, 3, 17, 17, 16, 7, 7, 2, 3, 1),       # first-layer style: C=3, 7x7, stride 2
    (2, 64, 15, 15, 64, 3, 3, 2, 1, 1),
    (2, 64, 15, 15, 64, 3, 3, 1, 2, 2),
    (5, 128, 7, 7, 136, 3, 3, 1, 1, 1),      # 49 pixels per image
    (2, 200, 10, 10, 300, 1, 1, 1, 0, 1),
    (1, 8, 5, 5, 8, 5, 5, 1, 0, 1),          # single output pixel
]


@pytest.mark.parametrize("cfg", CONV_CASES)
def test_conv2d_nchw(oracle, cfg):
    n, c, h, w, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n * 100 + c)
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float16)
    wt = rng.normal(0, 0.05, (k, c, r, s)).astype(np.float16)
    got = _run_conv(x, wt, st, pad, dil)
    assert oracle.rel_l2(got, oracle.c_conv2d_nchw(x, wt, st, pad, dil, "te_llvm")) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, oracle.c_conv2d_nchw(x, wt, st, pad, dil, "exact")) <= TOL_EXACT


# 1x1 / stride 1 / unpadded layers whose planes are a multiple of 4 pixels but not of 8: consumed in
# place, the activation copied into the stages by cp.async (one launch, no workspace)
POINTWISE_INPLACE_CASES = [
    # N, C, H, W, K
    (1, 64, 2, 2, 64),        # 4 pixels per image: one ragged tile
    (3, 72, 6, 6, 40),        # ragged channels (two k-blocks, the second 8 wide) and filters
    (5, 128, 14, 14, 264),    # 196-pixel planes, tiles straddle images, three 128-wide column tiles
    (7, 200, 10, 10, 136),    # 700 pixels: last tile ragged
    (2, 8, 18, 2, 16),        # a single 8-channel k-block
    (16, 1024, 14, 14, 256),  # the ResNet-50 layer at a small batch
]


@pytest.mark.parametrize("cfg", POINTWISE_INPLACE_CASES)
def test_conv2d_nchw_pointwise_in_place(oracle, cfg):
    n, c, h, w, k = cfg
    rng = np.random.default_rng(n * 1000 + c)
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float16)
    wt = rng.normal(0, 0.05, (k, c, 1, 1)).astype(np.float16)
    d = _lib.conv2d_desc(n, c, h, w, k, 1, 1)
    assert _lib.workspace_bytes_min(d) == 0 and "conv-1x1-inplace" in _lib.describe_plan(d)
    got = _run_conv(x, wt, 1, 0, 1, launches_expected=1)
    assert oracle.rel_l2(got, oracle.c_conv2d_nchw(x, wt, 1, 0, 1, "te_llvm")) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, oracle.c_conv2d_nchw(x, wt, 1, 0, 1, "exact")) <= TOL_EXACT
    # the re-layout path (what these layers ran on before) gives the same bits
    os.environ["AMOSB_CONV_NO_POINTWISE"] = "1"
    try:
        two = _run_conv(x, wt, 1, 0, 1, launches_expected=2)
    finally:
        del os.environ["AMOSB_CONV_NO_POINTWISE"]
    assert np.array_equal(got, two)


@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_conv2d_nchw_pointwise_in_place_tiles_and_fp16_out(oracle, tile_n):
    rng = np.random.default_rng(tile_n + 5)
    x = rng.uniform(-1, 1, (4, 136, 10, 10)).astype(np.float16)
    wt = rng.normal(0, 0.05, (300, 136, 1, 1)).astype(np.float16)
    ref = oracle.c_conv2d_nchw(x, wt, 1, 0, 1, "te_llvm")
    got = _run_conv(x, wt, 1, 0, 1, tile_n=tile_n, launches_expected=1)
    assert oracle.rel_l2(got, ref) <= TOL_TE_LLVM
    half = _run_conv(x, wt, 1, 0, 1, out_dtype="float16", tile_n=tile_n, launches_expected=1)
    assert np.array_equal(half, got.astype(np.float16))


@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_conv2d_tile_variants_and_fp16_out(oracle, tile_n):
    rng = np.random.default_rng(tile_n + 1)
    x = rng.uniform(-1, 1, (3, 64, 12, 12)).astype(np.float16)
    wt = rng.normal(0, 0.05, (320, 64, 3, 3)).astype(np.float16)
    got = _run_conv(x, wt, 1, 1, 1, tile_n=tile_n)
    assert oracle.rel_l2(got, oracle.c_conv2d_nchw(x, wt, 1, 1, 1, "te_llvm")) <= TOL_TE_LLVM
    got16 = _run_conv(x, wt, 1, 1, 1, out_dtype="float16", tile_n=tile_n)
    assert np.array_equal(got16, got.astype(np.float16))


@pytest.mark.parametrize("cfg", [
    # n, c, h, w, k, r, pad, cta_pair: planes of 4n pixels that tiles cut across, ragged channels
    (5, 64, 10, 10, 300, 3, 1, 1), (5, 64, 10, 10, 300, 3, 1, 2), (3, 136, 14, 14, 72, 1, 0, 0),
    (40, 72, 6, 6, 264, 3, 1, 0), (2, 64, 9, 9, 80, 3, 1, 0)])
@pytest.mark.parametrize("out_dtype", ["float32", "float16"])
def test_conv2d_nchw_four_pixel_stores_match_element_stores(oracle, cfg, out_dtype):
    """The NCHW epilogue that stores 4 pixels per lane (after a transposition among lanes) writes
    exactly what the element-wise epilogue writes; planes that are not whole 4-pixel groups (9x9)
    keep the element-wise form either way."""
    n, c, h, w, k, r, pad, cta_pair = cfg
    rng = np.random.default_rng(n * 1000 + k)
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float16)
    wt = rng.normal(0, 0.05, (k, c, r, r)).astype(np.float16)
    got = {}
    for mode in ("0", "1"):
        os.environ["AMOSB_NCHW_QUADS"] = mode
        try:
            got[mode] = _run_conv(x, wt, 1, pad, 1, out_dtype=out_dtype, cta_pair=cta_pair,
                                  launches_expected=1 if r == 1 else 2)
        finally:
            del os.environ["AMOSB_NCHW_QUADS"]
    assert np.array_equal(got["0"], got["1"])
    ref = oracle.c_conv2d_nchw(x, wt, 1, pad, 1, "te_llvm")
    assert oracle.rel_l2(got["1"].astype(np.float32), ref) <= (TOL_TE_LLVM if out_dtype == "float32" else 1e-3)


# ------------------------------------------------------------------------------ golden fixtures
def test_golden_reference_helpers(golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_topi_conv2d_nchw.npz"))
    for i in range(int(g["num_cases"])):
        stride, pad, dil = (int(v) for v in g[f"case{i}_geom"])
        got = _run_conv(g[f"case{i}_a"], g[f"case{i}_w"], stride, pad, dil)
        ref = g[f"case{i}_out"]
        err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
        assert err <= TOL_EXACT, (i, err)
    g = np.load(os.path.join(golden_dir, "ref_topi_batch_matmul.npz"))
    for i in range(int(g["num_cases"])):
        x, y = g[f"case{i}_x"], g[f"case{i}_y"]
        if x.shape[2] % 8 == 0:
            got = _run_gemm(x, y, "float32", trans_b=True)
            ref = g[f"case{i}_out"]
            assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= TOL_EXACT
        xi, yi = g[f"case{i}_xi"], g[f"case{i}_yi"]
        if xi.shape[2] % 16 == 0:
            assert np.array_equal(_run_gemm(xi, yi, "int32", trans_b=True),
                                  g[f"case{i}_outi"].astype(np.int32))


def test_golden_known_answers(golden_dir, oracle):
    k = np.load(os.path.join(golden_dir, "kat_oracle.npz"))
    assert np.array_equal(_run_gemm(k["gemm8_a"], k["gemm8_b"], "int32"), k["gemm8_exact"])
    got = _run_gemm(k["gemm_a"], k["gemm_b"], "float32")
    assert oracle.rel_l2(got, k["gemm_te_llvm"]) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, k["gemm_exact"]) <= TOL_EXACT
    got = _run_gemm(k["bgemm_a"], k["bgemm_b"], "float16")
    assert oracle.rel_l2(got, k["bgemm_te_llvm_f16out"]) <= TOL_TE_LLVM
    got = _run_conv(k["conv_a"], k["conv_w"], 1, 1, 1)
    assert oracle.rel_l2(got, k["conv_te_llvm"]) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, k["conv_exact"]) <= TOL_EXACT
    assert oracle.rel_l2(_run_conv(k["conv_a"], k["conv_w"], 2, 1, 1), k["conv_s2_te_llvm"]) \
        <= TOL_TE_LLVM
    assert oracle.rel_l2(_run_conv(k["conv_a"], k["conv_w"], 1, 2, 2), k["conv_d2_te_llvm"]) \
        <= TOL_TE_LLVM


# ------------------------------------------------------------------- full-size configurations
def test_full_gemm_f16_4096(oracle):
    """M=N=K=4096: sampled rows against the oracle, and the row-sum identity on every element."""
    rng = np.random.default_rng(20260001)
    a = rng.uniform(-1, 1, (4096, 4096)).astype(np.float16)
    b = rng.uniform(-1, 1, (4096, 4096)).astype(np.float16)
    ta, tb = _t(a), _t(b)
    c = torch.empty(4096, 4096, dtype=torch.float16, device=DEV)
    device.run(_lib.gemm_desc(4096, 4096, 4096, out_dtype=_lib.AMOSB_F16), [ta, tb], [c])
    c32 = torch.empty(4096, 4096, dtype=torch.float32, device=DEV)
    device.run(_lib.gemm_desc(4096, 4096, 4096), [ta, tb], [c32])
    assert device.status_peek(0) == 0
    rows = np.sort(rng.choice(4096, 48, replace=False))
    ref = oracle.c_gemm(a[rows], b, "te_llvm", out_dtype="float16")
    assert oracle.rel_l2(c[torch.from_numpy(rows).to(DEV)].cpu().numpy(), ref) <= TOL_TE_LLVM
    # sum_j C[i,j] == A[i,:] . (sum_j B[:,j])  (fp64 on the device, fp32-accumulated C)
    lhs = c32.double().sum(dim=1)
    rhs = ta.double() @ tb.double().sum(dim=1)
    assert (lhs - rhs).norm() / rhs.norm() < 1e-5
    assert torch.equal(c, c32.to(torch.float16))


def test_full_gemm_s8_8192(oracle):
    rng = np.random.default_rng(20260003)
    a = rng.integers(-128, 128, (8192, 8192), dtype=np.int8)
    b = rng.integers(-128, 128, (8192, 8192), dtype=np.int8)
    ta, tb = _t(a), _t(b)
    c = torch.empty(8192, 8192, dtype=torch.int32, device=DEV)
    device.run(_lib.gemm_desc(8192, 8192, 8192, in_dtype=_lib.AMOSB_S8), [ta, tb], [c])
    assert device.status_peek(0) == 0
    rows = np.sort(rng.choice(8192, 24, replace=False))
    ref = oracle.c_gemm(a[rows], b, "exact")
    assert np.array_equal(c[torch.from_numpy(rows).to(DEV)].cpu().numpy(), ref)
    # exact integer identities over every element: row sums and column sums
    bsum = tb.long().sum(dim=1)
    assert torch.equal(c.long().sum(dim=1), (ta.long() * bsum[None, :]).sum(dim=1))
    asum = ta.long().sum(dim=0)
    assert torch.equal(c.long().sum(dim=0), (asum[:, None] * tb.long()).sum(dim=0))


def test_full_batched_gemm(oracle):
    rng = np.random.default_rng(20260004)
    q = rng.normal(0, 1, (96, 512, 64)).astype(np.float16)
    kt = rng.normal(0, 1, (96, 64, 512)).astype(np.float16)
    got = _run_gemm(q, kt, "float16")
    assert oracle.rel_l2(got, oracle.c_gemm(q, kt, "te_llvm", out_dtype="float16")) <= TOL_TE_LLVM
    p = rng.normal(0, 1, (96, 512, 512)).astype(np.float16)
    v = rng.normal(0, 1, (96, 512, 64)).astype(np.float16)
    got = _run_gemm(p, v, "float16")
    assert oracle.rel_l2(got, oracle.c_gemm(p, v, "te_llvm", out_dtype="float16")) <= TOL_TE_LLVM


def test_full_conv_c1(oracle):
    rng = np.random.default_rng(20260000)
    x = rng.uniform(-1, 1, (1, 64, 56, 56)).astype(np.float16)
    w = rng.uniform(-1, 1, (64, 64, 3, 3)).astype(np.float16)
    got = _run_conv(x, w, 1, 1, 1)
    assert oracle.rel_l2(got, oracle.c_conv2d_nchw(x, w, 1, 1, 1, "te_llvm")) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, oracle.c_conv2d_nchw(x, w, 1, 1, 1, "exact")) <= TOL_EXACT


@pytest.mark.parametrize("cfg", [(256, 64, 56, 56, 256, 1, 1, 0), (256, 128, 28, 28, 128, 3, 3, 1),
                                 (256, 256, 14, 14, 256, 3, 3, 1), (256, 1024, 14, 14, 256, 1, 1, 0),
                                 (256, 512, 7, 7, 512, 3, 3, 1)])
def test_full_conv_batch256(oracle, cfg):
    """Batch-256 layers: sampled images against the oracle; and the whole output through the
    image-permutation property conv(x[perm]) == conv(x)[perm] (bit for bit)."""
    n, c, h, w, k, r, s, pad = cfg
    rng = np.random.default_rng(20260002)
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float16)
    wt = rng.normal(0, 0.05, (k, c, r, s)).astype(np.float16)
    d = _lib.conv2d_desc(n, c, h, w, k, r, s, 1, pad, 1)
    tx, tw = _t(x), _t(wt)
    out = torch.empty(n, k, d.conv_p, d.conv_q, dtype=torch.float32, device=DEV)
    device.run(d, [tx, tw], [out])
    assert device.status_peek(0) == 0
    imgs = [0, 1, 127, 255]
    ref = oracle.c_conv2d_nchw(x[imgs], wt, 1, pad, 1, "te_llvm")
    assert oracle.rel_l2(out[imgs].cpu().numpy(), ref) <= TOL_TE_LLVM
    # bit for bit when every tile is computed whole; where the schedule shares out the tiles of a
    # short last round (the 7x7 layer does), an image's sums may be added in another order
    perm = torch.from_numpy(rng.permutation(n)).to(DEV)
    out2 = torch.empty_like(out)
    device.run(d, [tx[perm].contiguous(), tw], [out2])
    shares = _lib.workspace_bytes(d) > _lib.workspace_bytes_min(d)
    if shares:
        diff = (out2.double() - out[perm].double()).norm() / out.double().norm()
        assert float(diff) <= 1e-5
        os.environ["AMOSB_NO_TAIL_SHARING"] = "1"
        try:
            device.run(d, [tx, tw], [out])
            device.run(d, [tx[perm].contiguous(), tw], [out2])
        finally:
            del os.environ["AMOSB_NO_TAIL_SHARING"]
    assert torch.equal(out2, out[perm])

"""GPU: float32 inputs -> float32 on the tf32 tensor-core path (reference: the wmma_tf32_fp32
intrinsic family, python/tvm/auto_tensorize/hw_abs_dag/cuda/wmma_tf32.py:11-60), through the C ABI,
against the numpy oracle.  The operands stay float32 in memory and are consumed in place; the TMA
copy into shared memory rounds every element to tf32 (nearest, ties to even).

Bars: relative L2 <= 2e-5 against the oracle's `tf32` mode (the reference's CUDA kernels: operands
converted with `__float_to_tf32`, nearest with ties away from zero -- the two roundings differ on
exact ties only, one value in 8192) and against `tf32_rne` (what runs here, to float32 summation
order); <= 1e-3 against `te_llvm` (the reference's llvm build: plain float32).
"""
import numpy as np
import pytest
import torch

from amos_b200 import _lib, device

pytestmark = pytest.mark.gpu

HW_MODE = "tf32_rne"
TOL_HW = 2e-5
TOL_REFERENCE = 1e-3
DEV = "cuda:0"


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def _gemm(a, b, trans_a=False, trans_b=False, tile_n=0, cta_pair=0):
    batched = a.ndim == 3
    m, k = a.shape[-2:]
    if trans_a:
        k, m = m, k
    n = b.shape[-2] if trans_b else b.shape[-1]
    d = _lib.gemm_desc(m, n, k, in_dtype=_lib.AMOSB_F32, batch=a.shape[0] if batched else 1,
                       trans_a=trans_a, trans_b=trans_b, batched=batched, tile_n=tile_n,
                       cta_pair=cta_pair)
    assert d.out_dtype == _lib.AMOSB_F32
    shape = (a.shape[0], m, n) if batched else (m, n)
    numel = int(np.prod(shape))
    buf = torch.full((numel + 2048,), 77, dtype=torch.float32, device=DEV)
    out = buf[1024:1024 + numel].view(shape)
    assert device.run(d, [_t(a), _t(b)], [out]) == 1
    assert device.status_peek(0) == 0
    assert (buf[:1024] == 77).all() and (buf[1024 + numel:] == 77).all(), "wrote outside C"
    return out.cpu().numpy()


def _check(oracle, got, a, b, **layout):
    assert oracle.rel_l2(got, oracle.np_gemm_f32(a, b, HW_MODE, **layout)) <= TOL_HW
    assert oracle.rel_l2(got, oracle.np_gemm_f32(a, b, "tf32", **layout)) <= TOL_HW
    assert oracle.rel_l2(got, oracle.np_gemm_f32(a, b, "te_llvm", **layout)) <= TOL_REFERENCE


@pytest.mark.parametrize("shape", [(128, 64, 32), (8, 8, 8), (200, 136, 72), (1000, 520, 264),
                                   (132, 36, 4)])
@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_tf32(oracle, shape, trans_b):
    m, n, k = shape
    rng = np.random.default_rng(m + 3 * n + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, k) if trans_b else (k, n)).astype(np.float32)
    got = _gemm(a, b, trans_b=trans_b)
    _check(oracle, got, a, b, trans_b=trans_b)
    # A given as [K, M]: the same products in the same order
    got_t = _gemm(np.ascontiguousarray(a.T), b, trans_a=True, trans_b=trans_b)
    assert np.array_equal(got_t, got)


@pytest.mark.parametrize("shape", [(512, 256, 64), (1000, 520, 264), (300, 136, 100), (2048, 1024, 512)])
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("tile_n", [0, 128, 256])
def test_gemm_tf32_cta_pairs(oracle, shape, trans_b, tile_n):
    """CTA-pair tiles (256 rows, tcgen05.mma.cta_group::2.kind::tf32): the same products in the same
    order as the single-CTA tiles, ragged edges and partial last rounds included."""
    m, n, k = shape
    rng = np.random.default_rng(7 * m + n + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, k) if trans_b else (k, n)).astype(np.float32)
    pair = _gemm(a, b, trans_b=trans_b, tile_n=tile_n, cta_pair=2)
    single = _gemm(a, b, trans_b=trans_b, tile_n=tile_n, cta_pair=1)
    assert np.array_equal(pair, single)
    _check(oracle, pair, a, b, trans_b=trans_b)


def test_batched_gemm_tf32_cta_pairs(oracle):
    rng = np.random.default_rng(11)
    a = rng.uniform(-1, 1, (3, 300, 72)).astype(np.float32)
    b = rng.uniform(-1, 1, (3, 72, 264)).astype(np.float32)
    pair = _gemm(a, b, cta_pair=2)
    assert np.array_equal(pair, _gemm(a, b, cta_pair=1))
    for i in range(3):
        _check(oracle, pair[i], a[i], b[i])


@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_gemm_tf32_tile_widths(oracle, tile_n):
    rng = np.random.default_rng(tile_n)
    a = rng.normal(0, 1, (520, 264)).astype(np.float32)
    b = rng.normal(0, 1, (264, 528)).astype(np.float32)
    _check(oracle, _gemm(a, b, tile_n=tile_n), a, b)
    bt = np.ascontiguousarray(b.T)
    _check(oracle, _gemm(a, bt, trans_b=True, tile_n=tile_n), a, bt, trans_b=True)


def test_operands_are_rounded_not_truncated(oracle):
    """Operands that already are tf32 values make every mode of the oracle agree, so this case is
    held to the tight bar against the reference's own float32 arithmetic; and adding less than half
    a tf32 step to every operand changes no bit of the result (truncation would let `a - tiny`
    drop to the next value down)."""
    rng = np.random.default_rng(77)
    a = oracle.to_tf32(rng.uniform(-1, 1, (264, 200)).astype(np.float32))
    b = oracle.to_tf32(rng.uniform(-1, 1, (200, 136)).astype(np.float32))
    got = _gemm(a, b)
    assert oracle.rel_l2(got, oracle.np_gemm_f32(a, b, "te_llvm")) <= TOL_HW
    assert oracle.rel_l2(got, oracle.np_gemm_f32(a, b, "tf32")) <= TOL_HW

    def nudge(x):  # +/- up to 0.4 of a tf32 step, in float32 bits
        d = rng.integers(-0x0CCC, 0x0CCD, x.shape).astype(np.int64)
        y = (x.view(np.uint32).astype(np.int64) + d).astype(np.uint32).view(np.float32)
        return np.where(x == 0, x, y)
    a2, b2 = nudge(a), nudge(b)
    assert np.array_equal(oracle.to_tf32(a2, "rne"), a) and not np.array_equal(a2, a)
    assert np.array_equal(_gemm(a2, b2), got)


def test_batched_gemm_tf32(oracle):
    rng = np.random.default_rng(8)
    a = rng.normal(0, 1, (5, 264, 64)).astype(np.float32)
    b = rng.normal(0, 1, (5, 64, 136)).astype(np.float32)
    _check(oracle, _gemm(a, b), a, b)
    bt = np.ascontiguousarray(b.transpose(0, 2, 1))
    _check(oracle, _gemm(a, bt, trans_b=True), a, bt, trans_b=True)


@pytest.mark.parametrize("relu", [False, True])
def test_fused_bias_relu_tf32(oracle, relu):
    rng = np.random.default_rng(21)
    m, n, k = 264, 136, 96
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    bias = rng.uniform(-1, 1, (n,)).astype(np.float32)
    d = _lib.gemm_desc(m, n, k, in_dtype=_lib.AMOSB_F32)
    d.epilogue = _lib.EPI_ADD_VECTOR | (_lib.EPI_RELU if relu else 0)
    d.addend_dtype, d.arg_c = _lib.AMOSB_F32, 2
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    device.run(d, [_t(a), _t(b), _t(bias)], [out])
    assert device.status_peek(0) == 0
    ref = oracle.np_gemm_f32(a, b, HW_MODE) + bias
    if relu:
        ref = np.maximum(ref, 0)
    assert oracle.rel_l2(out.cpu().numpy(), ref) <= TOL_HW


def test_full_size_gemm_tf32(oracle):
    """4096^3: sampled rows against the oracle (float64 sums), and linearity in A on the whole
    output -- A scaled by a power of two scales every product exactly."""
    rng = np.random.default_rng(20260004)
    a = rng.normal(0, 1, (4096, 4096)).astype(np.float32)
    b = rng.normal(0, 1, (4096, 4096)).astype(np.float32)
    d = _lib.gemm_desc(4096, 4096, 4096, in_dtype=_lib.AMOSB_F32)
    ta, tb = _t(a), _t(b)
    out = torch.empty(4096, 4096, dtype=torch.float32, device=DEV)
    device.run(d, [ta, tb], [out])
    assert device.status_peek(0) == 0
    rows = [0, 1, 127, 128, 2049, 4095]
    ref = oracle.np_gemm_f32(a[rows], b, HW_MODE, sequential=False)
    assert oracle.rel_l2(out[rows].cpu().numpy(), ref) <= TOL_HW
    assert oracle.rel_l2(out[rows].cpu().numpy(),
                         oracle.np_gemm_f32(a[rows], b, "tf32", sequential=False)) <= TOL_HW
    out2 = torch.empty_like(out)
    device.run(d, [ta * 4.0, tb], [out2])
    assert torch.equal(out2, out * 4.0)


def test_tf32_limits():
    a = torch.zeros(64, 64, dtype=torch.float32, device=DEV)
    # narrowing output and tall tiles: refused, not emulated
    d = _lib.gemm_desc(64, 64, 64, in_dtype=_lib.AMOSB_F32, out_dtype=_lib.AMOSB_F16)
    with pytest.raises(_lib.AmosbError) as e:
        device.run(d, [a, a.clone()], [torch.zeros(64, 64, dtype=torch.float16, device=DEV)])
    assert e.value.code == _lib.AMOSB_ERR_UNSUPPORTED
    for pin in (3,):
        d = _lib.gemm_desc(512, 256, 64, in_dtype=_lib.AMOSB_F32, cta_pair=pin)
        x = torch.zeros(512, 64, dtype=torch.float32, device=DEV)
        y = torch.zeros(64, 256, dtype=torch.float32, device=DEV)
        with pytest.raises(_lib.AmosbError) as e:
            device.run(d, [x, y], [torch.zeros(512, 256, dtype=torch.float32, device=DEV)])
        assert e.value.code == _lib.AMOSB_ERR_UNSUPPORTED
    # rows of A[M,K] must be 16-byte multiples: K % 4
    d = _lib.gemm_desc(64, 64, 6, in_dtype=_lib.AMOSB_F32)
    with pytest.raises(_lib.AmosbError) as e:
        device.run(d, [torch.zeros(64, 6, dtype=torch.float32, device=DEV),
                       torch.zeros(6, 64, dtype=torch.float32, device=DEV)],
                   [torch.zeros(64, 64, dtype=torch.float32, device=DEV)])
    assert e.value.code == _lib.AMOSB_ERR_UNSUPPORTED
    assert device.status_peek(0) == 0


def test_tf32_through_the_te_front_end(oracle):
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import ops
    from amos_b200 import tvm
    from amos_b200.tvm import auto_tensorize as at
    A, B, C = ops.gemm(264, 136, 200, "float32", "float32")
    r = at.auto_tensorize(at.compute_dag_from_tensors([C]), "cuda", None,
                          at.MeasureOptions(target="cuda", number=10, min_repeat_ms=5), trials=3)
    assert r.defined() and r.mapping.hw_abs_dag == "tcgen05_tf32_fp32"
    func = tvm.build(*at.get_schedule(r.sch_app, r.params), "cuda")
    rng = np.random.default_rng(13)
    a = rng.uniform(-1, 1, (264, 200)).astype(np.float32)
    b = rng.uniform(-1, 1, (200, 136)).astype(np.float32)
    ctx = tvm.gpu(0)
    c = tvm.nd.empty((264, 136), "float32", ctx)
    func(tvm.nd.array(a, ctx), tvm.nd.array(b, ctx), c)
    ctx.sync()
    _check(oracle, c.asnumpy(), a, b)


CONV_CASES = [
    # N, H, W, C, K, R, S, stride, pad, dil
    (2, 14, 14, 64, 64, 3, 3, 1, 1, 1),
    (3, 9, 11, 36, 40, 3, 3, 1, 1, 1),       # ragged channels and filters (multiples of 4)
    (2, 15, 15, 32, 64, 3, 3, 2, 1, 1),
    (2, 15, 15, 64, 32, 3, 3, 1, 2, 2),
    (2, 10, 10, 100, 304, 1, 1, 1, 0, 1),
    (2, 12, 12, 16, 24, 3, 3, 1, 1, 1),      # C < 32: a k-block spans rows of the next filter tap
]


@pytest.mark.parametrize("cfg", CONV_CASES)
def test_conv2d_nhwc_tf32(oracle, cfg):
    n, h, w, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n * 100 + c)
    x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
    wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float32)
    d = _lib.conv2d_nhwc_desc(n, h, w, c, k, r, s, st, pad, dil)
    d.in_dtype = _lib.AMOSB_F32
    assert _lib.workspace_bytes_min(d) == 0
    out = torch.full((n, d.conv_p, d.conv_q, k), float("nan"), dtype=torch.float32, device=DEV)
    assert device.run(d, [_t(x), _t(wt)], [out]) == 1
    assert device.status_peek(0) == 0
    got = out.cpu().numpy()
    assert oracle.rel_l2(got, oracle.np_conv2d_nhwc_f32(x, wt, st, pad, dil, HW_MODE)) <= TOL_HW
    assert oracle.rel_l2(got, oracle.np_conv2d_nhwc_f32(x, wt, st, pad, dil, "tf32")) <= TOL_HW
    assert oracle.rel_l2(got, oracle.np_conv2d_nhwc_f32(x, wt, st, pad, dil, "te_llvm")) \
        <= TOL_REFERENCE


@pytest.mark.parametrize("cfg", [
    (5, 15, 15, 36, 272, 3, 3, 2, 1, 1),     # ragged channel chunk, ragged second filter tile
    (5, 14, 14, 32, 256, 3, 3, 1, 1, 1),     # 980 pixels: four pair tiles, the last one ragged
    (2, 10, 10, 100, 304, 1, 1, 1, 0, 1),
    (40, 14, 14, 32, 512, 3, 3, 1, 1, 1),    # 62 pair tiles
])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_conv2d_nhwc_tf32_cta_pairs(oracle, cfg, tile_n):
    """float32 NHWC on CTA pairs: the same products in the same order as the single-CTA tiles."""
    n, h, w, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n * 10 + k)
    x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
    wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float32)
    outs = []
    for pair in (2, 1):
        d = _lib.conv2d_nhwc_desc(n, h, w, c, k, r, s, st, pad, dil, tile_n=tile_n, cta_pair=pair)
        d.in_dtype = _lib.AMOSB_F32
        assert ("umma_pair" in _lib.describe_plan(d)) == (pair == 2)
        out = torch.full((n, d.conv_p, d.conv_q, k), float("nan"), dtype=torch.float32, device=DEV)
        assert device.run(d, [_t(x), _t(wt)], [out]) == 1
        assert device.status_peek(0) == 0
        outs.append(out.cpu().numpy())
    assert np.array_equal(outs[0], outs[1])
    assert oracle.rel_l2(outs[0], oracle.np_conv2d_nhwc_f32(x, wt, st, pad, dil, HW_MODE)) <= TOL_HW


@pytest.mark.parametrize("cfg", [(6, 6, 128, 32, 32, 3, 3, 1, 1, 1), (5, 7, 256, 36, 72, 3, 3, 2, 1, 1),
                                 (4, 4, 128, 64, 40, 1, 1, 1, 0, 1)])
def test_conv2d_hwnc_tf32(oracle, cfg):
    h, w, n, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(h * 10 + c)
    x = rng.uniform(-1, 1, (h, w, n, c)).astype(np.float32)
    wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float32)
    d = _lib.conv2d_hwnc_desc(h, w, n, c, k, r, s, st, pad, dil)
    d.in_dtype = _lib.AMOSB_F32
    out = torch.full((d.conv_p, d.conv_q, n, k), float("nan"), dtype=torch.float32, device=DEV)
    assert device.run(d, [_t(x), _t(wt)], [out]) == 1
    assert device.status_peek(0) == 0
    got = out.cpu().numpy()
    assert oracle.rel_l2(got, oracle.np_conv2d_nhwc_f32(x, wt, st, pad, dil, HW_MODE, hwnc=True)) \
        <= TOL_HW
    # the NHWC kernel on the transposed tensors accumulates the same products in the same order
    d2 = _lib.conv2d_nhwc_desc(n, h, w, c, k, r, s, st, pad, dil)
    d2.in_dtype = _lib.AMOSB_F32
    out2 = torch.empty(n, d.conv_p, d.conv_q, k, dtype=torch.float32, device=DEV)
    device.run(d2, [_t(x.transpose(2, 0, 1, 3)), _t(wt)], [out2])
    assert torch.equal(out2.permute(1, 2, 0, 3), out)


def test_conv2d_tf32_limits_and_front_end(oracle):
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import ops
    from amos_b200 import tvm
    from amos_b200.tvm import auto_tensorize as at
    # tall tiles are not built for float32 tensors (CTA pairs are, for NHWC)
    d = _lib.conv2d_nhwc_desc(4, 8, 8, 32, 128, 3, 3, pad=1, in_dtype=_lib.AMOSB_F32, cta_pair=3)
    with pytest.raises(_lib.AmosbError) as e:
        device.run(d, [torch.zeros(4, 8, 8, 32, dtype=torch.float32, device=DEV),
                       torch.zeros(3, 3, 32, 128, dtype=torch.float32, device=DEV)],
                   [torch.zeros(4, 8, 8, 128, dtype=torch.float32, device=DEV)])
    assert e.value.code == _lib.AMOSB_ERR_UNSUPPORTED
    # the NHWC text on float32 tensors through the tuning flow
    A, B, Conv = ops.conv2d_nhwc(2, 14, 14, 32, 64, 3, 3, 1, 1, 1, in_dtype="float32")
    r = at.auto_tensorize(at.compute_dag_from_tensors([Conv]), "cuda", None,
                          at.MeasureOptions(target="cuda", number=10, min_repeat_ms=5), trials=3)
    assert r.defined() and r.mapping.hw_abs_dag == "tcgen05_tf32_fp32"
    func = tvm.build(*at.get_schedule(r.sch_app, r.params), "cuda")
    rng = np.random.default_rng(3)
    xh = rng.uniform(-1, 1, (2, 14, 14, 32)).astype(np.float32)
    wh = rng.normal(0, 0.05, (3, 3, 32, 64)).astype(np.float32)
    ctx = tvm.gpu(0)
    out = tvm.nd.empty((2, 14, 14, 64), "float32", ctx)
    func(tvm.nd.array(xh, ctx), tvm.nd.array(wh, ctx), out)
    ctx.sync()
    assert oracle.rel_l2(out.asnumpy(), oracle.np_conv2d_nhwc_f32(xh, wh, 1, 1, 1, HW_MODE)) <= TOL_HW


@pytest.mark.parametrize("cfg", [(2, 64, 14, 14, 64, 3, 3, 1, 1, 1), (3, 10, 9, 11, 40, 3, 3, 1, 1, 1),
                                 (2, 3, 17, 17, 16, 7, 7, 2, 3, 1), (2, 100, 10, 10, 304, 1, 1, 1, 0, 1),
                                 (5, 36, 7, 7, 64, 3, 3, 1, 1, 1)])
def test_conv2d_nchw_tf32(oracle, cfg):
    """NCHW / KCRS float32 tensors: re-layout pass on 32-bit elements, then the same main loop."""
    n, c, h, w, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n * 10 + c)
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
    f = rng.normal(0, 0.05, (k, c, r, s)).astype(np.float32)
    d = _lib.conv2d_desc(n, c, h, w, k, r, s, st, pad, dil)
    d.in_dtype = _lib.AMOSB_F32
    out = torch.full((n, k, d.conv_p, d.conv_q), float("nan"), dtype=torch.float32, device=DEV)
    ws = device.get_workspace(_lib.workspace_bytes(d), 0)
    assert device.run(d, [_t(x), _t(f)], [out], workspace=ws) == 2
    assert device.status_peek(0) == 0
    xh = np.ascontiguousarray(x.transpose(0, 2, 3, 1))
    fh = np.ascontiguousarray(f.transpose(2, 3, 1, 0))
    got = out.permute(0, 2, 3, 1).cpu().numpy()
    assert oracle.rel_l2(got, oracle.np_conv2d_nhwc_f32(xh, fh, st, pad, dil, HW_MODE)) <= TOL_HW
    assert oracle.rel_l2(got, oracle.np_conv2d_nhwc_f32(xh, fh, st, pad, dil, "te_llvm")) \
        <= TOL_REFERENCE

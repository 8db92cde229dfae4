"""GPU: int8 conv2d -> int32 in the two in-place layouts, NHWC and HWNC (reference: the
("int8", "int32") pair of benchmark/amos/mapping_conv2d_tensorcore.py:214-224 on the te texts of
:43-104) and in NCHW / KCRS (reference: tests/python/auto_tensorize/semi_auto_mappings/cuda/
tune_tensorcore_conv2d_int8.py:11-49), through the C ABI.  Bit for bit against the oracle's
`exact` mode (int32 products, what the reference's tensor-core path computes; its llvm build wraps every product to 8 bits and
disagrees with that on the same text -- `te_llvm` is checked to differ, so the test knows which
of the two it pins)."""
import numpy as np
import pytest
import torch

from amos_b200 import _lib, device

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def _run(desc, ins, shape):
    numel = int(np.prod(shape))
    buf = torch.full((numel + 2048,), 77, dtype=torch.int32, device=DEV)
    out = buf[1024:1024 + numel].view(shape)
    assert _lib.workspace_bytes_min(desc) == 0
    assert device.run(desc, [_t(x) for x in ins], [out]) == 1
    assert device.status_peek(0) == 0
    assert (buf[:1024] == 77).all() and (buf[1024 + numel:] == 77).all(), "wrote outside Out"
    return out.cpu().numpy()


CASES = [
    # N, H, W, C, K, R, S, stride, pad, dil
    (2, 14, 14, 128, 128, 3, 3, 1, 1, 1),
    (3, 9, 11, 48, 144, 3, 3, 1, 1, 1),      # C < 128: a k-block spans rows of the next filter taps
    (2, 15, 15, 160, 272, 3, 3, 2, 1, 1),    # ragged channel chunk and filter tile
    (2, 15, 15, 128, 128, 3, 3, 1, 2, 2),
    (2, 10, 10, 256, 304, 1, 1, 1, 0, 1),
    (1, 17, 17, 16, 16, 7, 7, 2, 3, 1),
]


@pytest.mark.parametrize("cfg", CASES)
@pytest.mark.parametrize("tile_n", [0, 128, 256])
def test_conv2d_nhwc_int8(oracle, cfg, tile_n):
    n, h, w, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n * 100 + c)
    x = rng.integers(-128, 128, (n, h, w, c), dtype=np.int8)
    wt = rng.integers(-128, 128, (r, s, c, k), dtype=np.int8)
    d = _lib.conv2d_nhwc_desc(n, h, w, c, k, r, s, st, pad, dil, in_dtype=_lib.AMOSB_S8,
                              tile_n=tile_n)
    assert (d.acc_dtype, d.out_dtype) == (_lib.AMOSB_S32, _lib.AMOSB_S32)
    got = _run(d, [x, wt], (n, d.conv_p, d.conv_q, k))
    want = oracle.np_conv2d_nhwc(x, wt, st, pad, dil, "exact")
    assert np.array_equal(got, want)
    if tile_n == 0:
        assert not np.array_equal(got, oracle.np_conv2d_nhwc(x, wt, st, pad, dil, "te_llvm"))


@pytest.mark.parametrize("cfg", [
    # N, H, W, C, K, R, S, stride, pad, dil: CTA-pair tiles are 256 pixels x 256 filters
    (5, 15, 15, 160, 272, 3, 3, 2, 1, 1),    # ragged channel chunk, ragged second filter tile
    (5, 14, 14, 128, 256, 3, 3, 1, 1, 1),    # 980 pixels: four pair tiles, the last one ragged
    (2, 10, 10, 256, 304, 1, 1, 1, 0, 1),
    (40, 14, 14, 128, 512, 3, 3, 1, 1, 1),   # 62 pair tiles: most of the 74 pairs busy
])
def test_conv2d_nhwc_int8_cta_pairs(oracle, cfg):
    """int8 NHWC on CTA pairs (tcgen05.mma.cta_group::2.kind::i8): bit for bit the oracle's sums."""
    n, h, w, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n * 10 + k)
    x = rng.integers(-128, 128, (n, h, w, c), dtype=np.int8)
    wt = rng.integers(-128, 128, (r, s, c, k), dtype=np.int8)
    d = _lib.conv2d_nhwc_desc(n, h, w, c, k, r, s, st, pad, dil, in_dtype=_lib.AMOSB_S8,
                              tile_n=256, cta_pair=2)
    assert "umma_pair" in _lib.describe_plan(d)
    got = _run(d, [x, wt], (n, d.conv_p, d.conv_q, k))
    assert np.array_equal(got, oracle.np_conv2d_nhwc(x, wt, st, pad, dil, "exact"))


@pytest.mark.parametrize("cfg", [(6, 6, 128, 128, 128, 3, 3, 1, 1, 1),
                                 (5, 7, 256, 48, 144, 3, 3, 2, 1, 1),
                                 (4, 4, 128, 256, 48, 1, 1, 1, 0, 1)])
def test_conv2d_hwnc_int8(oracle, cfg):
    h, w, n, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(h * 10 + c)
    x = rng.integers(-128, 128, (h, w, n, c), dtype=np.int8)
    wt = rng.integers(-128, 128, (r, s, c, k), dtype=np.int8)
    d = _lib.conv2d_hwnc_desc(h, w, n, c, k, r, s, st, pad, dil, in_dtype=_lib.AMOSB_S8)
    got = _run(d, [x, wt], (d.conv_p, d.conv_q, n, k))
    want = oracle.np_conv2d_nhwc(np.ascontiguousarray(x.transpose(2, 0, 1, 3)), wt, st, pad, dil,
                                 "exact").transpose(1, 2, 0, 3)
    assert np.array_equal(got, want)


NCHW_CASES = [
    # N, C, H, W, K, R, S, stride, pad, dil
    (2, 128, 14, 14, 128, 3, 3, 1, 1, 1),
    (3, 40, 9, 11, 72, 3, 3, 1, 1, 1),       # channels padded to 48 per pixel / 128 per filter tap
    (2, 3, 17, 17, 16, 7, 7, 2, 3, 1),       # first-layer style
    (2, 160, 15, 15, 272, 3, 3, 1, 2, 2),
    (2, 256, 10, 10, 304, 1, 1, 1, 0, 1),    # 1x1: still through the re-layout (8-bit planes)
    (5, 64, 7, 7, 64, 3, 3, 1, 1, 1),        # 49 pixels per image
]


@pytest.mark.parametrize("cfg", NCHW_CASES)
def test_conv2d_nchw_int8(oracle, cfg):
    n, c, h, w, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n * 100 + c)
    x = rng.integers(-128, 128, (n, c, h, w), dtype=np.int8)
    f = rng.integers(-128, 128, (k, c, r, s), dtype=np.int8)
    d = _lib.conv2d_desc(n, c, h, w, k, r, s, st, pad, dil)
    d.in_dtype, d.acc_dtype, d.out_dtype = _lib.AMOSB_S8, _lib.AMOSB_S32, _lib.AMOSB_S32
    shape = (n, k, d.conv_p, d.conv_q)
    numel = int(np.prod(shape))
    buf = torch.full((numel + 2048,), 77, dtype=torch.int32, device=DEV)
    out = buf[1024:1024 + numel].view(shape)
    ws = device.get_workspace(_lib.workspace_bytes(d), 0)
    assert device.run(d, [_t(x), _t(f)], [out], workspace=ws) == 2
    assert device.status_peek(0) == 0
    assert (buf[:1024] == 77).all() and (buf[1024 + numel:] == 77).all(), "wrote outside Out"
    want = oracle.np_conv2d_nhwc(np.ascontiguousarray(x.transpose(0, 2, 3, 1)),
                                 np.ascontiguousarray(f.transpose(2, 3, 1, 0)), st, pad, dil, "exact")
    assert np.array_equal(out.cpu().numpy(), want.transpose(0, 3, 1, 2))


def test_fused_bias_relu_int8():
    rng = np.random.default_rng(9)
    n, h, w, c, k = 3, 9, 11, 48, 144
    x = rng.integers(-128, 128, (n, h, w, c), dtype=np.int8)
    wt = rng.integers(-128, 128, (3, 3, c, k), dtype=np.int8)
    bias = rng.integers(-50000, 50000, (k,), dtype=np.int32)
    d = _lib.conv2d_nhwc_desc(n, h, w, c, k, 3, 3, 1, 1, 1, in_dtype=_lib.AMOSB_S8)
    plain = _run(d, [x, wt], (n, h, w, k))
    d.epilogue = _lib.EPI_ADD_VECTOR | _lib.EPI_RELU
    d.addend_dtype, d.arg_c = _lib.AMOSB_S32, 2
    got = _run(d, [x, wt, bias], (n, h, w, k))
    assert np.array_equal(got, np.maximum(plain + bias, 0))


def test_limits():
    x = torch.zeros(1, 8, 8, 24, dtype=torch.int8, device=DEV)       # C not a multiple of 16
    w = torch.zeros(3, 3, 24, 16, dtype=torch.int8, device=DEV)
    y = torch.zeros(1, 8, 8, 16, dtype=torch.int32, device=DEV)
    with pytest.raises(_lib.AmosbError) as e:
        device.run(_lib.conv2d_nhwc_desc(1, 8, 8, 24, 16, 3, 3, pad=1, in_dtype=_lib.AMOSB_S8),
                   [x, w], [y])
    assert e.value.code == _lib.AMOSB_ERR_UNSUPPORTED
    # tall tiles are not built for int8 (CTA pairs are, for NHWC)
    d = _lib.conv2d_nhwc_desc(4, 8, 8, 32, 128, 3, 3, pad=1, in_dtype=_lib.AMOSB_S8, cta_pair=3)
    with pytest.raises(_lib.AmosbError) as e:
        device.run(d, [torch.zeros(4, 8, 8, 32, dtype=torch.int8, device=DEV),
                       torch.zeros(3, 3, 32, 128, dtype=torch.int8, device=DEV)],
                   [torch.zeros(4, 8, 8, 128, dtype=torch.int32, device=DEV)])
    assert e.value.code == _lib.AMOSB_ERR_UNSUPPORTED
    assert device.status_peek(0) == 0


def test_through_the_te_front_end(oracle):
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import ops
    from amos_b200 import tvm
    from amos_b200.tvm import auto_tensorize as at
    A, B, Conv = ops.conv2d_nhwc(2, 14, 14, 32, 128, 3, 3, 1, 1, 1, in_dtype="int8",
                                 out_dtype="int32")
    r = at.auto_tensorize(at.compute_dag_from_tensors([Conv]), "cuda", None,
                          at.MeasureOptions(target="cuda", number=10, min_repeat_ms=5), trials=3)
    assert r.defined() and r.mapping.hw_abs_dag == "tcgen05_int8_int32"
    func = tvm.build(*at.get_schedule(r.sch_app, r.params), "cuda")
    rng = np.random.default_rng(3)
    x = rng.integers(-128, 128, (2, 14, 14, 32), dtype=np.int8)
    wt = rng.integers(-128, 128, (3, 3, 32, 128), dtype=np.int8)
    ctx = tvm.gpu(0)
    out = tvm.nd.empty((2, 14, 14, 128), "int32", ctx)
    func(tvm.nd.array(x, ctx), tvm.nd.array(wt, ctx), out)
    ctx.sync()
    assert np.array_equal(out.asnumpy(), oracle.np_conv2d_nhwc(x, wt, 1, 1, 1, "exact"))

"""GPU: HWNC / RSCK conv2d (reference: benchmark/amos/mapping_conv2d_tensorcore.py:74-104) through
the C ABI against the CPU oracle.  A[H,W,N,C] and B[R,S,C,K] are consumed where they lie; a 128-row
tile is one output pixel x 128 images (other image counts are padded to 128 per pixel inside the
kernel; a single image runs as the NHWC operator).  Bars as for the other layouts: relative L2 <= 1e-3 against `te_llvm`, <= 2e-5 against `exact`."""
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


def _run(x, w, stride, pad, dil, out_dtype="float32", tile_n=0, cta_pair=0):
    h, wd, n, c = x.shape
    r, s, _, k = w.shape
    d = _lib.conv2d_hwnc_desc(h, wd, n, c, k, r, s, stride, pad, dil,
                              out_dtype=_lib.DTYPE_CODES[out_dtype], tile_n=tile_n,
                              cta_pair=cta_pair)
    shape = (d.conv_p, d.conv_q, n, k)
    numel = int(np.prod(shape))
    tdt = device.CODE_TO_TORCH[d.out_dtype]
    buf = torch.full((numel + 2048,), 77, dtype=tdt, device=DEV)
    out = buf[1024:1024 + numel].view(shape)
    assert device.run(d, [_t(x), _t(w)], [out]) == 1
    assert device.status_peek(0) == 0
    assert (buf[:1024] == 77).all() and (buf[1024 + numel:] == 77).all(), "wrote outside Out"
    return out.cpu().numpy()


CASES = [
    # H, W, N, C, K, R, S, stride, pad, dil
    (4, 4, 128, 64, 64, 1, 1, 1, 0, 1),
    (6, 5, 128, 64, 64, 3, 3, 1, 1, 1),
    (7, 7, 256, 72, 40, 3, 3, 1, 1, 1),       # ragged channels and filters (multiples of 8)
    (9, 9, 128, 8, 16, 7, 7, 2, 3, 1),        # few channels, 7x7, stride 2
    (9, 8, 128, 64, 136, 3, 3, 2, 1, 1),
    (9, 9, 128, 64, 64, 3, 3, 1, 2, 2),       # dilation
    (5, 5, 128, 32, 24, 3, 3, 1, 1, 1),       # C < 64
    (5, 5, 384, 64, 304, 3, 3, 1, 0, 1),      # three image groups per pixel, no padding
]


@pytest.mark.parametrize("cfg", CASES)
@pytest.mark.parametrize("cta_pair", [1, 2, 3])
def test_conv2d_hwnc(oracle, cfg, cta_pair):
    h, w, n, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(h * 100 + c + k)
    x = rng.uniform(-1, 1, (h, w, n, c)).astype(np.float16)
    wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float16)
    got = _run(x, wt, st, pad, dil, cta_pair=cta_pair)
    assert oracle.rel_l2(got, oracle.c_conv2d_hwnc(x, wt, st, pad, dil, "te_llvm")) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, oracle.c_conv2d_hwnc(x, wt, st, pad, dil, "exact")) <= TOL_EXACT


@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_tile_variants_fp16_out_and_the_nhwc_operator(oracle, tile_n):
    rng = np.random.default_rng(tile_n + 2)
    x = rng.uniform(-1, 1, (6, 6, 128, 64)).astype(np.float16)
    wt = rng.normal(0, 0.05, (3, 3, 64, 320)).astype(np.float16)
    got = _run(x, wt, 1, 1, 1, tile_n=tile_n)
    assert oracle.rel_l2(got, oracle.c_conv2d_hwnc(x, wt, 1, 1, 1, "te_llvm")) <= TOL_TE_LLVM
    got16 = _run(x, wt, 1, 1, 1, out_dtype="float16", tile_n=tile_n)
    assert np.array_equal(got16, got.astype(np.float16))
    # the NHWC kernel on the transposed tensors accumulates the same products in the same order
    d = _lib.conv2d_nhwc_desc(128, 6, 6, 64, 320, 3, 3, pad=1, tile_n=tile_n, cta_pair=1)
    out = torch.empty(128, 6, 6, 320, dtype=torch.float32, device=DEV)
    device.run(d, [_t(x.transpose(2, 0, 1, 3)), _t(wt)], [out])
    assert np.array_equal(got, out.permute(1, 2, 0, 3).cpu().numpy())


def test_fused_bias_relu_and_bf16(oracle):
    rng = np.random.default_rng(17)
    h, w, n, c, k = 5, 6, 128, 72, 296
    x = rng.uniform(-1, 1, (h, w, n, c)).astype(np.float16)
    wt = rng.normal(0, 0.05, (3, 3, c, k)).astype(np.float16)
    bias = rng.uniform(-1, 1, (k,)).astype(np.float32)
    d = _lib.conv2d_hwnc_desc(h, w, n, c, k, 3, 3, 1, 1, 1)
    d.epilogue = _lib.EPI_ADD_VECTOR | _lib.EPI_RELU
    d.addend_dtype, d.arg_c = _lib.AMOSB_F32, 2
    out = torch.full((h, w, n, k), float("nan"), dtype=torch.float32, device=DEV)
    device.run(d, [_t(x), _t(wt), _t(bias)], [out])
    ref = np.maximum(oracle.c_conv2d_hwnc(x, wt, 1, 1, 1, "te_llvm") + bias, 0)
    assert oracle.rel_l2(out.cpu().numpy(), ref) <= TOL_TE_LLVM
    # bfloat16 inputs
    xb = oracle.to_bf16(x.astype(np.float32))
    wb = oracle.to_bf16(wt.astype(np.float32))
    d2 = _lib.conv2d_hwnc_desc(h, w, n, c, k, 3, 3, 1, 1, 1)
    d2.in_dtype = _lib.AMOSB_BF16
    out2 = torch.empty(h, w, n, k, dtype=torch.float32, device=DEV)
    device.run(d2, [_t(xb).to(torch.bfloat16), _t(wb).to(torch.bfloat16)], [out2])
    assert oracle.rel_l2(out2.cpu().numpy(), oracle.np_conv2d_hwnc(xb, wb, 1, 1, 1, "te_llvm")) \
        <= TOL_EXACT
    assert device.status_peek(0) == 0


@pytest.mark.parametrize("cfg", [
    # H, W, N, C, K, R, S, stride, pad, dil
    (8, 8, 96, 64, 64, 3, 3, 1, 1, 1),       # fewer images than a tile
    (6, 7, 16, 64, 72, 3, 3, 1, 1, 1),       # the benchmark script's small batches
    (5, 5, 200, 72, 40, 3, 3, 2, 1, 1),      # one full group of 128 and a ragged one per pixel
    (6, 6, 130, 64, 40, 1, 1, 1, 0, 1),
    (4, 4, 33, 64, 40, 3, 3, 1, 1, 1),
])
def test_image_counts_that_are_not_multiples_of_128(oracle, cfg):
    """Images are padded to 128 per output pixel inside the kernel: the padding images load as
    zeros and their rows are not stored (guards around the output stay untouched)."""
    h, w, n, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n + c)
    x = rng.uniform(-1, 1, (h, w, n, c)).astype(np.float16)
    wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float16)
    ref = oracle.c_conv2d_hwnc(x, wt, st, pad, dil, "te_llvm")
    import os
    for out_dtype in ("float32", "float16"):
        got = _run(x, wt, st, pad, dil, out_dtype=out_dtype)
        want = ref if out_dtype == "float32" else ref.astype(np.float16)
        assert oracle.rel_l2(got, want) <= TOL_TE_LLVM
    os.environ["AMOSB_DIRECT_STORE"] = "1"      # the epilogue without TMA stores: same bits
    try:
        assert np.array_equal(_run(x, wt, st, pad, dil, out_dtype="float16"), got)
    finally:
        del os.environ["AMOSB_DIRECT_STORE"]
    # fused full-shape addend + ReLU: the addend is indexed by the rows that exist
    d = _lib.conv2d_hwnc_desc(h, w, n, c, k, r, s, st, pad, dil)
    d.epilogue = _lib.EPI_ADD_FULL | _lib.EPI_RELU
    d.addend_dtype, d.arg_c = _lib.AMOSB_F32, 2
    res = rng.uniform(-1, 1, ref.shape).astype(np.float32)
    out = torch.full(ref.shape, float("nan"), dtype=torch.float32, device=DEV)
    device.run(d, [_t(x), _t(wt), _t(res)], [out])
    assert device.status_peek(0) == 0
    assert oracle.rel_l2(out.cpu().numpy(), np.maximum(ref + res, 0)) <= TOL_TE_LLVM


@pytest.mark.parametrize("cfg", [
    # H, W, N, C, K, R, S, stride_h (stride_w = 1 through the square stride 1), pad, dil
    (6, 7, 8, 64, 72, 3, 3, 1, 1, 1),        # 16 pixels x 8 images per tile; 7 pixels per row: ragged groups
    (9, 21, 12, 64, 40, 3, 3, 1, 1, 1),      # 12 images in boxes of 16; rows of 21 = 2 groups of 8 + 5
    (5, 9, 32, 72, 136, 3, 3, 1, 2, 2),      # 4 pixels x 32 images; dilation; ragged channels
    (4, 6, 64, 64, 264, 1, 1, 1, 0, 1),      # 2 pixels x 64 images; 1x1; three 128-wide filter tiles
    (7, 5, 50, 32, 24, 5, 5, 1, 2, 1),       # 50 images in boxes of 64; 5x5 filter
    (12, 12, 24, 128, 128, 3, 3, 1, 1, 1),
])
@pytest.mark.parametrize("cta_pair", [0, 2, 3])
def test_few_images_pack_pixels_into_a_tile(oracle, cfg, cta_pair):
    """With at most 64 images (and a filter that moves one pixel at a time along a row) a 128-row tile
    is several consecutive pixels of an output row x the images, instead of one pixel x images padded
    to 128: the same sums as the padded form, bit for bit, TMA-store and plain-store epilogues."""
    import os
    h, w, n, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n * 7 + c)
    x = rng.uniform(-1, 1, (h, w, n, c)).astype(np.float16)
    wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float16)
    d = _lib.conv2d_hwnc_desc(h, w, n, c, k, r, s, st, pad, dil, cta_pair=cta_pair)
    assert "consecutive pixels of an output row" in _lib.describe_plan(d)
    got = _run(x, wt, st, pad, dil, cta_pair=cta_pair)
    assert oracle.rel_l2(got, oracle.c_conv2d_hwnc(x, wt, st, pad, dil, "te_llvm")) <= TOL_TE_LLVM
    os.environ["AMOSB_HWNC_NO_PACKING"] = "1"
    try:
        assert "one output pixel x 128 images" in _lib.describe_plan(d)
        padded = _run(x, wt, st, pad, dil, cta_pair=cta_pair)
    finally:
        del os.environ["AMOSB_HWNC_NO_PACKING"]
    assert np.array_equal(got, padded)
    os.environ["AMOSB_DIRECT_STORE"] = "1"
    try:
        assert np.array_equal(_run(x, wt, st, pad, dil, cta_pair=cta_pair), got)
    finally:
        del os.environ["AMOSB_DIRECT_STORE"]
    got16 = _run(x, wt, st, pad, dil, out_dtype="float16", cta_pair=cta_pair)
    assert np.array_equal(got16, got.astype(np.float16))


@pytest.mark.parametrize("n", [256, 200, 24])
def test_cta_pairs_match_single_cta_tiles(oracle, n):
    """HWNC on CTA pairs (each CTA of a pair holds one 128-row group: 128 images of a pixel, or a
    group of pixels x few images): bit-identical to the single-CTA tiles, for float16, int8 and
    float32 tensors."""
    rng = np.random.default_rng(n)
    h, w, c, k = 6, 7, 64, 272
    for kind in ("f16", "s8", "f32"):
        if kind == "s8":
            x = rng.integers(-128, 128, (h, w, n, c), dtype=np.int8)
            wt = rng.integers(-128, 128, (3, 3, c, k), dtype=np.int8)
            in_dtype, odt = _lib.AMOSB_S8, torch.int32
        elif kind == "f32":
            x = rng.uniform(-1, 1, (h, w, n, c)).astype(np.float32)
            wt = rng.normal(0, 0.05, (3, 3, c, k)).astype(np.float32)
            in_dtype, odt = _lib.AMOSB_F32, torch.float32
        else:
            x = rng.uniform(-1, 1, (h, w, n, c)).astype(np.float16)
            wt = rng.normal(0, 0.05, (3, 3, c, k)).astype(np.float16)
            in_dtype, odt = _lib.AMOSB_F16, torch.float32
        outs = []
        for pair in (2, 1):
            d = _lib.conv2d_hwnc_desc(h, w, n, c, k, 3, 3, 1, 1, 1, tile_n=256, cta_pair=pair,
                                      in_dtype=in_dtype)
            assert ("umma_pair" in _lib.describe_plan(d)) == (pair == 2)
            out = torch.full((h, w, n, k), 77, dtype=odt, device=DEV)
            assert device.run(d, [_t(x), _t(wt)], [out]) == 1
            assert device.status_peek(0) == 0
            outs.append(out.cpu().numpy())
        assert np.array_equal(outs[0], outs[1]), kind
        if kind == "s8":
            want = oracle.np_conv2d_nhwc(np.ascontiguousarray(x.transpose(2, 0, 1, 3)), wt, 1, 1, 1,
                                         "exact").transpose(1, 2, 0, 3)
            assert np.array_equal(outs[0], want)
        elif kind == "f16":
            assert oracle.rel_l2(outs[0], oracle.c_conv2d_hwnc(x, wt, 1, 1, 1, "te_llvm")) <= TOL_TE_LLVM


def test_ragged_image_count_int8_and_tf32(oracle):
    rng = np.random.default_rng(3)
    h, w, n, c, k = 5, 6, 40, 32, 48
    xi = rng.integers(-128, 128, (h, w, n, c), dtype=np.int8)
    wi = rng.integers(-128, 128, (3, 3, c, k), dtype=np.int8)
    d = _lib.conv2d_hwnc_desc(h, w, n, c, k, 3, 3, 1, 1, 1, in_dtype=_lib.AMOSB_S8)
    out = torch.full((h, w, n, k), 77, dtype=torch.int32, device=DEV)
    device.run(d, [_t(xi), _t(wi)], [out])
    want = oracle.np_conv2d_nhwc(np.ascontiguousarray(xi.transpose(2, 0, 1, 3)), wi, 1, 1, 1,
                                 "exact").transpose(1, 2, 0, 3)
    assert np.array_equal(out.cpu().numpy(), want)
    xf = rng.uniform(-1, 1, (h, w, n, c)).astype(np.float32)
    wf = rng.normal(0, 0.05, (3, 3, c, k)).astype(np.float32)
    d = _lib.conv2d_hwnc_desc(h, w, n, c, k, 3, 3, 1, 1, 1, in_dtype=_lib.AMOSB_F32)
    outf = torch.full((h, w, n, k), float("nan"), dtype=torch.float32, device=DEV)
    device.run(d, [_t(xf), _t(wf)], [outf])
    assert device.status_peek(0) == 0
    assert oracle.rel_l2(outf.cpu().numpy(),
                         oracle.np_conv2d_nhwc_f32(xf, wf, 1, 1, 1, "tf32_rne", hwnc=True)) <= TOL_EXACT


def test_full_size_layer_and_the_te_front_end(oracle):
    """Batch-256 3x3 C128->K128 28x28 in HWNC: sampled pixels against the oracle of the NHWC
    operator on the same values, the whole output against the NHWC kernel."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import ops
    from amos_b200 import tvm
    from amos_b200.tvm import auto_tensorize as at
    H = W = 28
    N, C, K = 256, 128, 128
    A, B, Conv = ops.conv2d_hwnc(H, W, N, C, K, 3, 3, 1, 1, 1)
    r = at.auto_tensorize(at.compute_dag_from_tensors([Conv]), "cuda", None,
                          at.MeasureOptions(target="cuda", number=5, min_repeat_ms=5), trials=2)
    assert r.defined()
    func = tvm.build(*at.get_schedule(r.sch_app, r.params), "cuda")
    rng = np.random.default_rng(20260004)
    x = rng.uniform(-1, 1, (H, W, N, C)).astype(np.float16)
    wt = rng.normal(0, 0.05, (3, 3, C, K)).astype(np.float16)
    out = tvm.nd.empty((H, W, N, K), "float32")
    tx, tw = tvm.nd.array(x), tvm.nd.array(wt)
    func(tx, tw, out)
    got = out.torch()
    d = _lib.conv2d_nhwc_desc(N, H, W, C, K, 3, 3, pad=1)
    ref = torch.empty(N, H, W, K, dtype=torch.float32, device=DEV)
    device.run(d, [tx.torch().permute(2, 0, 1, 3).contiguous(), tw.torch()], [ref])
    assert oracle.rel_l2(got.cpu().numpy(), ref.permute(1, 2, 0, 3).cpu().numpy()) <= 1e-6
    imgs = [0, 127, 128, 255]
    cpu = oracle.c_conv2d_nhwc(np.ascontiguousarray(x[:, :, imgs].transpose(2, 0, 1, 3)), wt,
                               1, 1, 1, "te_llvm")
    assert oracle.rel_l2(got[:, :, imgs].permute(2, 0, 1, 3).cpu().numpy(), cpu) <= TOL_TE_LLVM
    assert device.status_peek(0) == 0


@pytest.mark.parametrize("cfg", [(14, 14, 64, 64, 3, 3, 1, 1, 1), (15, 15, 64, 128, 3, 3, 2, 1, 1),
                                 (7, 7, 512, 512, 3, 3, 1, 1, 1), (10, 10, 200, 304, 1, 1, 1, 0, 1)])
def test_single_image(oracle, cfg):
    """Batch 1, the default of the reference's benchmark script (its layer list has N = 1): one
    image in HWNC is the same memory as one image in NHWC, and runs as that operator."""
    h, w, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(h + c)
    x = rng.uniform(-1, 1, (h, w, 1, c)).astype(np.float16)
    wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float16)
    d = _lib.conv2d_hwnc_desc(h, w, 1, c, k, r, s, st, pad, dil)
    assert "conv2d_nhwc" in _lib.describe_plan(d)
    out = torch.full((d.conv_p, d.conv_q, 1, k), float("nan"), dtype=torch.float32, device=DEV)
    assert device.run(d, [_t(x), _t(wt)], [out]) == 1
    assert device.status_peek(0) == 0
    ref = oracle.c_conv2d_hwnc(x, wt, st, pad, dil, "te_llvm")
    assert oracle.rel_l2(out.cpu().numpy(), ref) <= TOL_TE_LLVM

"""GPU: NHWC / RSCK conv2d (reference: benchmark/amos/mapping_conv2d_tensorcore.py:43-72), called
through the C ABI, against the CPU oracle.  Both operands are consumed where they lie: one launch,
no workspace.  Bars as for the NCHW operator: relative L2 <= 1e-3 against the oracle's `te_llvm`
mode, <= 2e-5 against `exact`.
"""
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
    n, h, wd, c = x.shape
    r, s, _, k = w.shape
    d = _lib.conv2d_nhwc_desc(n, h, wd, c, k, r, s, stride, pad, dil,
                              out_dtype=_lib.DTYPE_CODES[out_dtype], tile_n=tile_n,
                              cta_pair=cta_pair)
    assert _lib.workspace_bytes_min(d) == 0
    shape = (n, d.conv_p, d.conv_q, k)
    numel = int(np.prod(shape))
    tdt = device.CODE_TO_TORCH[d.out_dtype]
    buf = torch.full((numel + 2048,), 77, dtype=tdt, device=DEV)
    out = buf[1024:1024 + numel].view(shape)
    launches = device.run(d, [_t(x), _t(w)], [out])
    assert launches == 1
    assert device.status_peek(0) == 0
    assert (buf[:1024] == 77).all() and (buf[1024 + numel:] == 77).all(), "wrote outside Out"
    return out.cpu().numpy()


CASES = [
    # N, H, W, C, K, R, S, stride, pad, dil
    (1, 8, 8, 64, 64, 1, 1, 1, 0, 1),
    (1, 16, 16, 64, 64, 3, 3, 1, 1, 1),
    (2, 14, 14, 64, 64, 3, 3, 1, 1, 1),      # 392 pixels: tiles straddle images
    (3, 9, 11, 72, 40, 3, 3, 1, 1, 1),       # ragged channels and filters (multiples of 8)
    (2, 17, 17, 8, 16, 7, 7, 2, 3, 1),       # first-layer style: few channels, 7x7, stride 2
    (2, 15, 15, 64, 64, 3, 3, 2, 1, 1),
    (2, 15, 15, 64, 64, 3, 3, 1, 2, 2),
    (5, 7, 7, 128, 136, 3, 3, 1, 1, 1),      # 49 pixels per image
    (2, 10, 10, 200, 304, 1, 1, 1, 0, 1),
    (1, 5, 5, 8, 8, 5, 5, 1, 0, 1),          # single output pixel
    (2, 12, 12, 32, 24, 3, 3, 1, 1, 1),      # C < 64: a k-block spans rows of the next filter tap
]


@pytest.mark.parametrize("cfg", CASES)
@pytest.mark.parametrize("cta_pair", [1, 2, 3])
def test_conv2d_nhwc(oracle, cfg, cta_pair):
    n, h, w, c, k, r, s, st, pad, dil = cfg
    rng = np.random.default_rng(n * 100 + c)
    x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float16)
    wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float16)
    got = _run(x, wt, st, pad, dil, cta_pair=cta_pair)
    assert oracle.rel_l2(got, oracle.c_conv2d_nhwc(x, wt, st, pad, dil, "te_llvm")) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, oracle.c_conv2d_nhwc(x, wt, st, pad, dil, "exact")) <= TOL_EXACT


@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_tile_variants_and_fp16_out(oracle, tile_n):
    rng = np.random.default_rng(tile_n + 1)
    x = rng.uniform(-1, 1, (3, 12, 12, 64)).astype(np.float16)
    wt = rng.normal(0, 0.05, (3, 3, 64, 320)).astype(np.float16)
    got = _run(x, wt, 1, 1, 1, tile_n=tile_n)
    assert oracle.rel_l2(got, oracle.c_conv2d_nhwc(x, wt, 1, 1, 1, "te_llvm")) <= TOL_TE_LLVM
    got16 = _run(x, wt, 1, 1, 1, out_dtype="float16", tile_n=tile_n)
    assert np.array_equal(got16, got.astype(np.float16))


def test_same_numbers_as_the_nchw_operator(oracle):
    """Same layer given in both layouts: the two kernels accumulate the same exact products in
    fp32, in a different order -- they agree to fp32 rounding."""
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, (4, 14, 14, 128)).astype(np.float16)
    wt = rng.normal(0, 0.05, (3, 3, 128, 128)).astype(np.float16)
    got = _run(x, wt, 1, 1, 1)
    d = _lib.conv2d_desc(4, 128, 14, 14, 128, 3, 3, pad=1)
    out = torch.empty(4, 128, 14, 14, dtype=torch.float32, device=DEV)
    device.run(d, [_t(x.transpose(0, 3, 1, 2)), _t(wt.transpose(3, 2, 0, 1))], [out])
    assert oracle.rel_l2(got, out.permute(0, 2, 3, 1).cpu().numpy()) <= 1e-6


@pytest.mark.parametrize("relu", [False, True])
def test_fused_bias_relu(oracle, relu):
    rng = np.random.default_rng(9)
    n, h, w, c, k = 3, 9, 11, 72, 296
    x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float16)
    wt = rng.normal(0, 0.05, (3, 3, c, k)).astype(np.float16)
    bias = rng.uniform(-1, 1, (k,)).astype(np.float32)
    for cta_pair in (1, 2, 3):
        d = _lib.conv2d_nhwc_desc(n, h, w, c, k, 3, 3, 1, 1, 1, cta_pair=cta_pair)
        d.epilogue = _lib.EPI_ADD_VECTOR | (_lib.EPI_RELU if relu else 0)
        d.addend_dtype, d.arg_c = _lib.AMOSB_F32, 2
        out = torch.full((n, d.conv_p, d.conv_q, k), float("nan"), dtype=torch.float32, device=DEV)
        device.run(d, [_t(x), _t(wt), _t(bias)], [out])
        assert device.status_peek(0) == 0
        ref = oracle.c_conv2d_nhwc(x, wt, 1, 1, 1, "te_llvm") + bias
        if relu:
            ref = np.maximum(ref, 0)
        assert oracle.rel_l2(out.cpu().numpy(), ref) <= TOL_TE_LLVM
        # full-size residual
        res = rng.uniform(-1, 1, ref.shape).astype(np.float32)
        d.epilogue = _lib.EPI_ADD_FULL | (_lib.EPI_RELU if relu else 0)
        device.run(d, [_t(x), _t(wt), _t(res)], [out])
        ref = oracle.c_conv2d_nhwc(x, wt, 1, 1, 1, "te_llvm") + res
        if relu:
            ref = np.maximum(ref, 0)
        assert oracle.rel_l2(out.cpu().numpy(), ref) <= TOL_TE_LLVM


def test_channels_not_multiple_of_8_fail_cleanly():
    d = _lib.conv2d_nhwc_desc(1, 8, 8, 3, 16, 3, 3, pad=1)
    x = torch.zeros(1, 8, 8, 3, dtype=torch.float16, device=DEV)
    w = torch.zeros(3, 3, 3, 16, dtype=torch.float16, device=DEV)
    y = torch.zeros(1, 8, 8, 16, dtype=torch.float32, device=DEV)
    with pytest.raises(_lib.AmosbError) as e:
        device.run(d, [x, w], [y])
    assert e.value.code == _lib.AMOSB_ERR_UNSUPPORTED
    assert device.status_peek(0) == 0


@pytest.mark.parametrize("cfg", [(256, 28, 28, 128, 128, 3, 3, 1), (256, 14, 14, 256, 256, 3, 3, 1),
                                 (256, 7, 7, 512, 512, 3, 3, 1), (256, 56, 56, 64, 256, 1, 1, 0)])
def test_full_size_layers(oracle, cfg):
    """Batch-256 layers in NHWC: sampled images against the oracle, and the whole output through
    the image-permutation property conv(x[perm]) == conv(x)[perm] (bit for bit)."""
    n, h, w, c, k, r, s, pad = cfg
    rng = np.random.default_rng(20260003)
    x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float16)
    wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float16)
    d = _lib.conv2d_nhwc_desc(n, h, w, c, k, r, s, 1, pad, 1)
    tx, tw = _t(x), _t(wt)
    out = torch.empty(n, d.conv_p, d.conv_q, k, dtype=torch.float32, device=DEV)
    device.run(d, [tx, tw], [out])
    assert device.status_peek(0) == 0
    imgs = [0, 1, 127, 255]
    ref = oracle.c_conv2d_nhwc(x[imgs], wt, 1, pad, 1, "te_llvm")
    assert oracle.rel_l2(out[imgs].cpu().numpy(), ref) <= TOL_TE_LLVM
    perm = torch.from_numpy(rng.permutation(n)).to(DEV)
    out2 = torch.empty_like(out)
    device.run(d, [tx[perm].contiguous(), tw], [out2])
    if _lib.workspace_bytes(d) > _lib.workspace_bytes_min(d):
        # the schedule shares out the tiles of its short last round (the 7x7 layer): the sums of an
        # image that lands in such a tile are added in another order; bit for bit with whole tiles
        import os
        diff = (out2.double() - out[perm].double()).norm() / out.double().norm()
        assert float(diff) <= 1e-5
        os.environ["AMOSB_NO_TAIL_SHARING"] = "1"
        try:
            device.run(d, [tx, tw], [out])
            device.run(d, [tx[perm].contiguous(), tw], [out2])
        finally:
            del os.environ["AMOSB_NO_TAIL_SHARING"]
    assert torch.equal(out2, out[perm])


def test_through_the_tuning_flow(oracle, tmp_path):
    """The reference benchmark's flow on the NHWC text: auto_tensorize -> get_schedule ->
    tvm.build -> call (benchmark/amos/mapping_conv2d_tensorcore.py:88-135)."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import ops
    from amos_b200 import tvm
    from amos_b200.tvm import auto_tensorize as at
    A, B, Conv = ops.conv2d_nhwc(2, 14, 14, 64, 64, 3, 3, 1, 1, 1)
    target_dag = at.compute_dag_from_tensors([Conv])
    measure_opt = at.MeasureOptions(target="cuda", timeout=100, number=20, min_repeat_ms=20)
    result = at.auto_tensorize(target_dag, "cuda", str(tmp_path / "nhwc.log"), measure_opt,
                               trials=6)
    assert result.defined() and 0 < result.perf < 1.0
    sch, args = at.get_schedule(result.sch_app, result.params)
    func = tvm.build(sch, args, "cuda")
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, (2, 14, 14, 64)).astype(np.float16)
    wt = rng.normal(0, 0.05, (3, 3, 64, 64)).astype(np.float16)
    ctx = tvm.gpu(0)
    out = tvm.nd.empty((2, 14, 14, 64), "float32", ctx)
    assert func(tvm.nd.array(x, ctx), tvm.nd.array(wt, ctx), out) is None
    ctx.sync()
    assert oracle.rel_l2(out.asnumpy(), oracle.c_conv2d_nhwc(x, wt, 1, 1, 1, "te_llvm")) \
        <= TOL_TE_LLVM


def test_golden_outputs_of_the_reference_nhwc_helper(oracle, golden_dir):
    """The kernels on the committed inputs of tests/golden/ref_topi_conv2d_nhwc.npz against the
    outputs the reference's conv2d_nhwc_python produced for them: float16 and tf32-representable
    float32 to float32 rounding of the sums, int8 bit for bit (through NHWC where C and K are
    multiples of 16, else through the NCHW operator on the transposed tensors)."""
    import os
    g = np.load(os.path.join(golden_dir, "ref_topi_conv2d_nhwc.npz"))
    for i in range(int(g["num_cases"])):
        a, w = g[f"case{i}_a"], g[f"case{i}_w"]
        stride, pad, dil = (int(v) for v in g[f"case{i}_geom"])
        ref = g[f"case{i}_out"]
        n, h, wd, c = a.shape
        r, s, _, k = w.shape
        code = {"float16": _lib.AMOSB_F16, "int8": _lib.AMOSB_S8, "float32": _lib.AMOSB_F32}[str(a.dtype)]
        odt = torch.int32 if a.dtype == np.int8 else torch.float32
        if a.dtype == np.int8 and (c % 16 or k % 16):
            d = _lib.conv2d_desc(n, c, h, wd, k, r, s, stride, pad, dil)
            d.in_dtype, d.acc_dtype, d.out_dtype = code, _lib.AMOSB_S32, _lib.AMOSB_S32
            out = torch.empty(n, k, d.conv_p, d.conv_q, dtype=odt, device=DEV)
            device.run(d, [_t(a.transpose(0, 3, 1, 2)), _t(w.transpose(3, 2, 0, 1))], [out],
                       workspace=device.get_workspace(_lib.workspace_bytes(d), 0))
            got = out.permute(0, 2, 3, 1).cpu().numpy()
        else:
            d = _lib.conv2d_nhwc_desc(n, h, wd, c, k, r, s, stride, pad, dil, in_dtype=code)
            out = torch.empty(n, d.conv_p, d.conv_q, k, dtype=odt, device=DEV)
            device.run(d, [_t(a), _t(w)], [out])
            got = out.cpu().numpy()
        assert device.status_peek(0) == 0
        if a.dtype == np.int8:
            assert np.array_equal(got, ref.astype(np.int64))
        else:
            assert oracle.rel_l2(got, ref) <= TOL_EXACT

"""CPU: the `te` front end, the native recogniser and the `at` surface (no GPU needed)."""
import json
import os

import pytest

from amos_b200 import _lib, tvm
from amos_b200.tvm import auto_tensorize as at

import ops

te = tvm.te


def _desc(tensors):
    return _lib.recognize(at.compute_dag_from_tensors([tensors[-1]]).serialise())


def test_placeholder_defaults_and_compute_axes(built_lib):
    A = te.placeholder((4, 5), name="A")
    assert A.dtype == "float32" and A.shape == (4, 5)
    C = te.compute((4, 5), lambda x, y: A[x, y] * 2.0, name="C")
    assert [a.var.name for a in C.op.axis] == ["x", "y"]
    assert C.op.axis[0].dom.extent == 4 and C.op.reduce_axis == []
    assert C.op.input_tensors == [A] and C.op.output(0) is C
    k = te.reduce_axis([0, 7], name="k")
    assert k.dom.min == 0 and k.dom.extent == 7
    with pytest.raises(ValueError):
        te.reduce_axis(7, name="k")


def test_binary_ops_keep_operand_dtype(built_lib):
    A = te.placeholder((4, 4), dtype="float16", name="A")
    B = te.placeholder((4, 4), dtype="float16", name="B")
    prod = A[0, 0] * B[0, 0]
    assert prod.dtype == "float16"  # this is what makes the llvm build round products to fp16
    assert prod.astype("float32").dtype == "float32"
    I = te.placeholder((4, 4), dtype="int8", name="I")
    assert (I[0, 0] * I[1, 1]).dtype == "int8"
    with pytest.raises(TypeError):
        _ = A[0, 0] * I[0, 0]


def test_dag_inputs_order_and_args(built_lib):
    A, B, Conv = ops.conv2d(1, 64, 56, 56, 64, 3, 3, 1, 1, 1)
    dag = at.compute_dag_from_tensors([Conv])
    assert dag.get_inputs() == [A, B]
    assert [op.name for op in dag.op_lst] == ["Pad", "Conv"]
    assert dag.tensors == [Conv]


def test_recognise_gemm_variants(built_lib):
    d = _desc(ops.gemm(4096, 4096, 4096))
    assert (d.kind, d.m, d.n, d.k, d.trans_b) == (_lib.OP_GEMM, 4096, 4096, 4096, 0)
    assert (d.in_dtype, d.acc_dtype, d.out_dtype) == (_lib.AMOSB_F16, _lib.AMOSB_F32, _lib.AMOSB_F32)
    assert (d.arg_a, d.arg_b) == (0, 1)
    d = _desc(ops.gemm_nt(128, 256, 64))
    assert (d.m, d.n, d.k, d.trans_b) == (128, 256, 64, 1)
    d = _desc(ops.gemm_cast(128, 256, 64))
    assert d.out_dtype == _lib.AMOSB_F16 and d.acc_dtype == _lib.AMOSB_F32
    d = _desc(ops.gemm(8192, 8192, 8192, "int8", "int32"))
    assert (d.in_dtype, d.acc_dtype, d.out_dtype) == (_lib.AMOSB_S8, _lib.AMOSB_S32, _lib.AMOSB_S32)


def test_recognise_operands_swapped_in_the_product(built_lib):
    A = te.placeholder([64, 32], dtype="float16", name="A")
    B = te.placeholder([32, 48], dtype="float16", name="B")
    k = te.reduce_axis([0, 32], name="k")
    C = te.compute([64, 48], lambda i, j: te.sum((B[k, j] * A[i, k]).astype("float32"), axis=k),
                   name="C")
    dag = at.compute_dag_from_tensors([C])
    assert dag.get_inputs() == [B, A]
    d = _lib.recognize(dag.serialise())
    assert (d.m, d.n, d.k) == (64, 48, 32)
    assert (d.arg_a, d.arg_b) == (1, 0)  # the callable takes (B, A, C); A is its second input


def test_recognise_transposed_a(built_lib):
    """gemm1 / gemm2 / batch_gemm2 of the reference's functional module: A indexed [k, i]."""
    d = _desc(ops.gemm_tn(300, 136, 72))
    assert (d.kind, d.trans_a, d.trans_b, d.m, d.n, d.k) == (_lib.OP_GEMM, 1, 0, 300, 136, 72)
    d = _desc(ops.gemm_tt(300, 136, 72, "int8", "int32"))
    assert (d.trans_a, d.trans_b, d.in_dtype) == (1, 1, _lib.AMOSB_S8)
    d = _desc(ops.batch_gemm_tn(4, 256, 64, 128))
    assert (d.kind, d.trans_a, d.batch, d.m, d.n, d.k) == (_lib.OP_BATCHED_GEMM, 1, 4, 256, 64, 128)
    text = _lib.describe_plan(d)
    assert "A MN-major" in text and "umma_persistent" in text
    # pairs and tall tiles do not exist for this layout: the plan stays on single-CTA tiles
    big = _lib.gemm_desc(4096, 4096, 4096, trans_a=True)
    assert "umma_pair" not in _lib.describe_plan(big)
    cands = at.ScheduleGenerator(big, None).candidates()
    assert cands and all(c.cta_pair == 1 for c in cands)


def test_recognise_bfloat16(built_lib):
    """("bfloat16", "float32") is one of the dtype pairs the reference's benchmark scripts accept
    (benchmark/amos/mapping_conv2d_tensorcore.py:217); its intrinsic family is wmma_bf16_fp32
    (python/tvm/auto_tensorize/hw_abs_dag/cuda/wmma_bf16.py:11-50)."""
    d = _desc(ops.gemm(256, 128, 64, "bfloat16", "float32"))
    assert (d.kind, d.in_dtype, d.acc_dtype, d.out_dtype) == \
        (_lib.OP_GEMM, _lib.AMOSB_BF16, _lib.AMOSB_F32, _lib.AMOSB_F32)
    d = _desc(ops.conv2d_nhwc(2, 14, 14, 64, 64, 3, 3, 1, 1, 1, in_dtype="bfloat16"))
    assert (d.kind, d.in_dtype) == (_lib.OP_CONV2D_NHWC, _lib.AMOSB_BF16)
    d = _desc(ops.conv2d(2, 64, 14, 14, 64, 3, 3, 1, 1, 1, in_dtype="bfloat16"))
    assert (d.kind, d.in_dtype) == (_lib.OP_CONV2D_NCHW, _lib.AMOSB_BF16)
    assert "bf16" in _lib.describe_plan(_desc(ops.gemm(256, 128, 64, "bfloat16", "float32")))
    m = at.get_match_results(at.compute_dag_from_tensors([ops.gemm(256, 128, 64, "bfloat16")[-1]]))
    assert m and m[0].hw_abs_dag == "tcgen05_bf16_fp32"
    # a narrowing cast after a bfloat16 GEMM has no kernel
    with pytest.raises(_lib.AmosbError):
        A, B, C = ops.gemm(64, 64, 64, "bfloat16", "float32")
        D = te.compute([64, 64], lambda i, j: C[i, j].astype("float16"), name="D")
        _desc([A, B, D])


def test_recognise_float32_as_tf32(built_lib):
    """float32 operands are what the reference maps to its tf32 intrinsic family wmma_tf32_fp32
    (python/tvm/auto_tensorize/hw_abs_dag/cuda/wmma_tf32.py:11-60: float32 in memory, tf32 in the
    fragments, compute keys nnn / nnt)."""
    for build, ta, tb in ((ops.gemm, 0, 0), (ops.gemm_nt, 0, 1), (ops.gemm_tn, 1, 0),
                          (ops.gemm_tt, 1, 1)):
        d = _desc(build(256, 128, 64, "float32", "float32"))
        assert (d.kind, d.in_dtype, d.acc_dtype, d.out_dtype, d.trans_a, d.trans_b) == \
            (_lib.OP_GEMM, _lib.AMOSB_F32, _lib.AMOSB_F32, _lib.AMOSB_F32, ta, tb)
    d = _desc(ops.batch_gemm(6, 256, 128, 64, "float32", "float32"))
    assert (d.kind, d.batch, d.in_dtype) == (_lib.OP_BATCHED_GEMM, 6, _lib.AMOSB_F32)
    plan = _lib.describe_plan(d)
    assert "tf32" in plan and "x32," in plan          # 32 float32 = one 128-byte k-block
    m = at.get_match_results(at.compute_dag_from_tensors([ops.gemm(256, 128, 64, "float32")[-1]]))
    assert m and m[0].hw_abs_dag == "tcgen05_tf32_fp32" and m[0].shape_key.endswith("x8")
    # conv2d on float32 tensors: the in-place layouts are mapped ...
    d = _desc(ops.conv2d_nhwc(2, 14, 14, 32, 64, 3, 3, 1, 1, 1, in_dtype="float32"))
    assert (d.kind, d.in_dtype, d.out_dtype) == (_lib.OP_CONV2D_NHWC, _lib.AMOSB_F32, _lib.AMOSB_F32)
    d = _desc(ops.conv2d_hwnc(14, 14, 128, 32, 64, 3, 3, 1, 1, 1, in_dtype="float32"))
    assert (d.kind, d.in_dtype) == (_lib.OP_CONV2D_HWNC, _lib.AMOSB_F32)
    assert "tf32" in _lib.describe_plan(d) and "32 channels" in _lib.describe_plan(d)
    # ... and so is NCHW (re-layout pass on 32-bit elements, channels padded to 4 / 32)
    d = _desc(ops.conv2d(1, 64, 8, 8, 64, 3, 3, 1, 1, 1, in_dtype="float32"))
    assert (d.kind, d.in_dtype) == (_lib.OP_CONV2D_NCHW, _lib.AMOSB_F32)
    assert _lib.workspace_bytes_min(d) == (64 * 64 + 64 * 9 * 64) * 4
    # float64 tensors have no mapping: the reference's message, not a fallback
    with pytest.raises(_lib.AmosbError) as e:
        _desc(ops.conv2d(1, 64, 8, 8, 64, 3, 3, 1, 1, 1, in_dtype="float64", out_dtype="float64"))
    assert "no matched intrinsic" in str(e.value)


def test_recognise_int8_conv_in_the_in_place_layouts(built_lib):
    """("int8", "int32") on the NHWC / HWNC texts of benchmark/amos/mapping_conv2d_tensorcore.py
    (:43-104, dtype pairs :214-224), and on the NCHW text."""
    d = _desc(ops.conv2d_nhwc(2, 14, 14, 32, 128, 3, 3, 1, 1, 1, in_dtype="int8", out_dtype="int32"))
    assert (d.kind, d.in_dtype, d.acc_dtype, d.out_dtype) == \
        (_lib.OP_CONV2D_NHWC, _lib.AMOSB_S8, _lib.AMOSB_S32, _lib.AMOSB_S32)
    plan = _lib.describe_plan(d)
    assert "<i8," in plan and "x128," in plan
    d = _desc(ops.conv2d_hwnc(6, 6, 128, 32, 128, 3, 3, 1, 1, 1, in_dtype="int8", out_dtype="int32"))
    assert (d.kind, d.in_dtype) == (_lib.OP_CONV2D_HWNC, _lib.AMOSB_S8)
    # NCHW / KCRS (the reference's own int8 conv script,
    # tests/python/auto_tensorize/semi_auto_mappings/cuda/tune_tensorcore_conv2d_int8.py:11-49)
    d = _desc(ops.conv2d(1, 64, 8, 8, 64, 3, 3, 1, 1, 1, in_dtype="int8", out_dtype="int32"))
    assert (d.kind, d.in_dtype, d.out_dtype) == (_lib.OP_CONV2D_NCHW, _lib.AMOSB_S8, _lib.AMOSB_S32)
    # scratch: N*H*W pixels of 64 -> 64 channels, 64 filters of 9 taps x 128 padded channels, 1 byte each
    assert _lib.workspace_bytes_min(d) == 64 * 64 + 64 * 9 * 128


def test_recognise_float16_sums(built_lib):
    """("float16", "float16"), the first dtype pair of the reference's benchmark scripts
    (benchmark/amos/mapping_conv2d_tensorcore.py:214-224, mapping_gemm_tensorcore.py): accepted, and
    run with a float32 accumulator whose value is rounded to float16 once."""
    for t in (ops.gemm(256, 128, 64, "float16", "float16"),
              ops.conv2d(1, 64, 14, 14, 64, 3, 3, 1, 1, 1, out_dtype="float16"),
              ops.conv2d_nhwc(2, 14, 14, 64, 64, 3, 3, 1, 1, 1, out_dtype="float16")):
        d = _desc(t)
        assert (d.in_dtype, d.acc_dtype, d.out_dtype) == (_lib.AMOSB_F16, _lib.AMOSB_F32, _lib.AMOSB_F16)
    # a float16 sum widened afterwards would need the float16-rounded sum: not offered
    A, B, C = ops.gemm(64, 64, 64, "float16", "float16")
    with pytest.raises(_lib.AmosbError):
        _desc([A, B, te.compute([64, 64], lambda i, j: C[i, j].astype("float32"), name="D")])


def test_recognise_batched(built_lib):
    d = _desc(ops.batch_gemm(96, 512, 512, 64, final_dtype="float16"))
    assert (d.kind, d.batch, d.m, d.n, d.k) == (_lib.OP_BATCHED_GEMM, 96, 512, 512, 64)
    assert d.out_dtype == _lib.AMOSB_F16


@pytest.mark.parametrize("cfg", [
    (1, 64, 56, 56, 64, 3, 3, 1, 1, 1),
    (256, 64, 56, 56, 256, 1, 1, 1, 0, 1),
    (2, 3, 224, 224, 64, 7, 7, 2, 3, 1),
    (1, 16, 20, 20, 8, 3, 3, 1, 2, 2),
])
def test_recognise_conv(built_lib, cfg):
    N, C, H, W, K, R, S, st, pad, dil = cfg
    d = _desc(ops.conv2d(N, C, H, W, K, R, S, st, pad, dil))
    assert d.kind == _lib.OP_CONV2D_NCHW
    assert (d.conv_n, d.conv_c, d.conv_h, d.conv_w, d.conv_k, d.conv_r, d.conv_s) == \
        (N, C, H, W, K, R, S)
    assert (d.stride_h, d.stride_w, d.pad_h, d.pad_w, d.dil_h, d.dil_w) == \
        (st, st, pad, pad, dil, dil)
    assert d.conv_p == (H + 2 * pad - dil * (R - 1) - 1) // st + 1


@pytest.mark.parametrize("cfg", [
    (1, 56, 56, 64, 64, 3, 3, 1, 1, 1),
    (256, 56, 56, 64, 256, 1, 1, 1, 0, 1),
    (2, 224, 224, 8, 64, 7, 7, 2, 3, 1),
    (1, 20, 20, 16, 8, 3, 3, 1, 2, 2),
])
def test_recognise_conv_nhwc(built_lib, cfg):
    """The NHWC / RSCK text of the reference's conv2d benchmark
    (benchmark/amos/mapping_conv2d_tensorcore.py:43-72)."""
    N, H, W, C, K, R, S, st, pad, dil = cfg
    d = _desc(ops.conv2d_nhwc(N, H, W, C, K, R, S, st, pad, dil))
    assert d.kind == _lib.OP_CONV2D_NHWC
    assert (d.conv_n, d.conv_c, d.conv_h, d.conv_w, d.conv_k, d.conv_r, d.conv_s) == \
        (N, C, H, W, K, R, S)
    assert (d.stride_h, d.stride_w, d.pad_h, d.pad_w, d.dil_h, d.dil_w) == \
        (st, st, pad, pad, dil, dil)
    assert d.conv_p == (H + 2 * pad - dil * (R - 1) - 1) // st + 1
    assert _lib.workspace_bytes_min(d) == 0  # both operands are consumed where they lie
    fused = _desc(ops.conv2d_nhwc_bias_relu(N, H, W, C, K, R, S, st, pad, dil))
    assert fused.kind == _lib.OP_CONV2D_NHWC
    assert fused.epilogue == _lib.EPI_ADD_VECTOR | _lib.EPI_RELU and fused.arg_c == 2


@pytest.mark.parametrize("cfg", [
    (28, 28, 256, 128, 128, 3, 3, 1, 1, 1),
    (15, 15, 128, 32, 48, 3, 3, 2, 1, 2),
    (8, 8, 128, 64, 64, 1, 1, 1, 0, 1),
])
def test_recognise_conv_hwnc(built_lib, cfg):
    """The HWNC / RSCK text of the reference's conv2d benchmark
    (benchmark/amos/mapping_conv2d_tensorcore.py:74-104)."""
    H, W, N, C, K, R, S, st, pad, dil = cfg
    d = _desc(ops.conv2d_hwnc(H, W, N, C, K, R, S, st, pad, dil))
    assert d.kind == _lib.OP_CONV2D_HWNC
    assert (d.conv_n, d.conv_c, d.conv_h, d.conv_w, d.conv_k, d.conv_r, d.conv_s) == \
        (N, C, H, W, K, R, S)
    assert (d.stride_h, d.pad_h, d.dil_h) == (st, pad, dil)
    assert d.conv_p == (H + 2 * pad - dil * (R - 1) - 1) // st + 1
    assert _lib.workspace_bytes_min(d) == 0
    text = _lib.describe_plan(d)
    assert "conv-hwnc" in text and "umma_pair" not in text
    from amos_b200 import shard
    half, start, count = shard.local_desc(d, 2, 1)  # images are split; the layout stays HWNC
    assert half.kind == _lib.OP_CONV2D_HWNC and (start, count) == (N // 2, N - N // 2)


def test_recognise_fused_trailing_stages(built_lib):
    A, B, D, E = ops.gemm_bias_relu(128, 256, 64, bias="vector", relu=True, final_dtype="float16")
    dag = at.compute_dag_from_tensors([E])
    assert dag.get_inputs() == [A, B, D]
    d = _lib.recognize(dag.serialise())
    assert d.kind == _lib.OP_GEMM and d.out_dtype == _lib.AMOSB_F16
    assert d.epilogue == _lib.EPI_ADD_VECTOR | _lib.EPI_RELU
    assert (d.arg_a, d.arg_b, d.arg_c, d.addend_dtype) == (0, 1, 2, _lib.AMOSB_F32)
    assert d.n_inputs == 3
    # the reference's own trailing op: E = C + D with a full matrix, no ReLU
    d = _desc(ops.gemm_bias_relu(128, 128, 128, bias="full", relu=False))
    assert d.epilogue == _lib.EPI_ADD_FULL and d.out_dtype == _lib.AMOSB_F32
    # fp16 bias read through a cast; int32 bias on the int8 GEMM
    d = _desc(ops.gemm_bias_relu(64, 64, 64, bias_dtype="float16"))
    assert d.addend_dtype == _lib.AMOSB_F16
    d = _desc(ops.gemm_bias_relu(64, 64, 64, in_dtype="int8", acc_dtype="int32"))
    assert d.addend_dtype == _lib.AMOSB_S32 and d.epilogue & _lib.EPI_RELU
    d = _desc(ops.conv2d_bias_relu(2, 64, 14, 14, 64, 3, 3, 1, 1, 1))
    assert d.kind == _lib.OP_CONV2D_NCHW and d.epilogue == _lib.EPI_ADD_VECTOR | _lib.EPI_RELU
    d = _desc(ops.conv2d_bias_relu(2, 64, 14, 14, 64, 3, 3, 1, 1, 1, bias="full", relu=False))
    assert d.epilogue == _lib.EPI_ADD_FULL
    # a bias over the M axis, arithmetic after a narrowing cast, or two addends do not fuse
    A, B, C = ops.gemm(64, 64, 64)
    D = te.placeholder([64], dtype="float32", name="D")
    with pytest.raises(_lib.AmosbError):
        _desc([A, B, D, te.compute([64, 64], lambda i, j: C[i, j] + D[i], name="E")])
    with pytest.raises(_lib.AmosbError):
        H = te.compute([64, 64], lambda i, j: C[i, j].astype("float16"), name="H")
        D16 = te.placeholder([64], dtype="float16", name="D16")
        _desc([A, B, D16, te.compute([64, 64], lambda i, j: H[i, j] + D16[j], name="E")])
    with pytest.raises(_lib.AmosbError):
        D2 = te.placeholder([64], dtype="float32", name="D2")
        _desc([A, B, D, D2, te.compute([64, 64], lambda i, j: C[i, j] + D[j] + D2[j], name="E")])


def test_unmatched_workloads(built_lib, capsys):
    mo = at.MeasureOptions(target="cuda")
    # element-wise op: no reduction
    X = te.placeholder([8, 8], dtype="float16", name="X")
    Y = te.compute([8, 8], lambda i, j: X[i, j] + X[j, i], name="Y")
    r = at.auto_tensorize(at.compute_dag_from_tensors([Y]), "cuda", "", mo, trials=0)
    assert not r.defined()
    assert "This workload has no matched intrinsic for target: cuda" in capsys.readouterr().out
    # int32 inputs have no mapping here
    with pytest.raises(_lib.AmosbError) as e:
        _desc(ops.gemm(64, 64, 64, "int32", "int32"))
    assert e.value.code == _lib.AMOSB_ERR_UNSUPPORTED
    assert "no matched intrinsic" in e.value.message
    # non-affine / non-GEMM index pattern
    A = te.placeholder([16, 16], dtype="float16", name="A")
    B = te.placeholder([16, 16], dtype="float16", name="B")
    k = te.reduce_axis([0, 16], name="k")
    C = te.compute([16, 16], lambda i, j: te.sum((A[i, k] * B[i, k]).astype("float32"), axis=k),
                   name="C")
    with pytest.raises(_lib.AmosbError):
        _desc([A, B, C])
    # a padding stage whose predicate does not guard the bounds
    with pytest.raises(_lib.AmosbError):
        A = te.placeholder([1, 8, 6, 6], dtype="float16", name="A")
        W = te.placeholder([8, 8, 3, 3], dtype="float16", name="W")
        Pad = te.compute([1, 8, 8, 8], lambda n, c, h, w: tvm.tir.if_then_else(
            tvm.tir.all(h >= 1, w >= 1), A[n, c, h - 1, w - 1], tvm.tir.const(0.0, "float16")),
            name="Pad")
        rc, rr, rs = (te.reduce_axis([0, e], name=n) for e, n in ((8, "rc"), (3, "rr"), (3, "rs")))
        Conv = te.compute([1, 8, 6, 6], lambda n, k, p, q: te.sum(
            (Pad[n, rc, p + rr, q + rs] * W[k, rc, rr, rs]).astype("float32"), axis=[rc, rr, rs]),
            name="Conv")
        _desc([A, W, Conv])


def test_malformed_dag_text(built_lib):
    with pytest.raises(_lib.AmosbError) as e:
        _lib.recognize("garbage\n")
    assert e.value.code == _lib.AMOSB_ERR_ARG


def test_at_flow_plan_only(built_lib, tmp_path):
    """The caller sequence of the reference's README works without a device when trials=0."""
    A, B, Conv = ops.conv2d(1, 64, 56, 56, 64, 3, 3, 1, 1, 1)
    target_dag = at.compute_dag_from_tensors([Conv])
    measure_opt = at.MeasureOptions(target="cuda", timeout=100, number=200, min_repeat_ms=500)
    log = str(tmp_path / "conv.log")
    result = at.auto_tensorize(target_dag, "cuda", log, measure_opt, trials=0)
    assert result.defined()
    schedule_app = result.sch_app
    target_dag2 = schedule_app.target_dag
    inputs = target_dag2.get_inputs()
    args = inputs + list(target_dag2.tensors)
    sch = tvm.te.create_schedule([x.op for x in target_dag2.tensors])
    sch = schedule_app.apply(sch, result.params)
    text = tvm.lower(sch, args, simple_mode=True)
    assert "umma_" in text and "im2col" in text
    sch2, args2 = at.get_schedule(result.sch_app, result.params)
    assert args2 == args
    func = tvm.build(sch2, args2, "cuda")
    assert func.entry_name == "__tvm_main__"
    assert "tcgen05" in func.imported_modules[0].get_source()
    with pytest.raises(_lib.AmosbError):
        tvm.build(sch2, args2, "llvm")
    with pytest.raises(_lib.AmosbError):
        tvm.build(tvm.te.create_schedule([Conv.op]), args2, "cuda")


def test_logs_of_the_reference_tuner_are_read_not_used(built_lib, tmp_path, capsys):
    """A tuning log written by the reference (records of CUDAParamsV2: python/tvm/auto_tensorize/
    tensorization_phases/schedulers/cuda_v2.py:23-76; per-mapping files "mapping_<bits>_<name>" of
    auto_tensorize_v4, auto_tensorize.py:827-829) loads; its values are shown, its records do not
    pick a kernel."""
    A, B, Conv = ops.conv2d(1, 128, 28, 28, 128, 3, 3, 1, 1, 1)
    dag = at.compute_dag_from_tensors([Conv])
    name = "conv2d-nchw-float16-float16-layer-(1,128,28,28,128,3,3,1,1,1).log"
    rec = {"inline": [1, 1], "vectorize": [4, 1],
           "spatial_factors": [[[1, 2, 1, 2], [0, 0, -1]], [[2, 7, 1, 2], [1, -1, -1]]],
           "reduce_factors": [[[4, 2, 1], [-1, 1]]], "last_factors": [[[4, 784, 1], [1, -1]]],
           "output_unroll_step": [512, 1], "last_unroll_step": [512, -1]}
    for bits, value in (("(0,0,0,0,0,1,0)", 326.31), ("(0,0,0,0,1,1,0)", 512.0)):
        with open(tmp_path / f"mapping_{bits}_{name}", "w") as f:
            print(json.dumps({"record": rec, "value": value}), file=f)
            print(json.dumps({"record": rec, "value": value / 2}), file=f)
    mo = at.MeasureOptions(target="cuda")
    r = at.auto_tensorize_v4(dag, "cuda", name, mo, schedule_log_dir=str(tmp_path), trials=0)
    assert r.defined()
    assert r.sch_gen.num_entries() == 4 and r.sch_gen.num_foreign_entries() == 4
    assert abs(r.perf - 1 / 512.0) < 1e-12          # best value the old logs hold
    assert (r.params.tile_n, r.params.cta_pair) == (0, 0) and r.params.foreign
    assert "records of the reference's tuner" in capsys.readouterr().out
    # an own measurement outranks any number of foreign records
    r.sch_gen.feedback(at.TileParams(128, 3), 100.0, log_to_file=False)
    best = r.sch_gen.get_best_entry()
    assert (best.record.tile_n, best.record.cta_pair, best.value) == (128, 3, 100.0)
    # nothing was written next to the old files
    assert sorted(p.name for p in tmp_path.iterdir()) == sorted(
        f"mapping_{b}_{name}" for b in ("(0,0,0,0,0,1,0)", "(0,0,0,0,1,1,0)"))


class _Subgraph:
    """What the reference's dispatcher hands over: `root_ops` and a tag."""

    def __init__(self, tensors, tag):
        self.root_ops = [t.op for t in tensors]
        self.tag = tag


def test_network_level_dispatcher_plan_only(built_lib, tmp_path, capsys):
    """`tg.autoschedule.auto_tensorize_cuda` and `AutoTensorizeContext`
    (python/tvm/tensor_graph/core/auto_schedule/auto_schedule.py:92-105, 351-433) route a matched
    sub-graph to the kernels and tell the caller when a sub-graph does not match."""
    from amos_b200.tvm.tensor_graph.core.auto_schedule.auto_schedule import (
        AutoTensorizeContext, auto_tensorize_cuda)
    A, B, C = ops.batch_gemm(12, 512, 512, 64)
    placeholder_sch = tvm.te.create_schedule([C.op])
    out = auto_tensorize_cuda(placeholder_sch, [C], str(tmp_path / "bg.log"), 0)
    (sch, args), = out.items()
    assert args == [A, B, C] and sch.plan.kind == _lib.OP_BATCHED_GEMM
    # a sub-graph with no tensor-core mapping comes back with empty args
    X = te.placeholder([8, 8], dtype="float16", name="X")
    Y = te.compute([8, 8], lambda i, j: X[i, j] + X[j, i], name="Y")
    keep = tvm.te.create_schedule([Y.op])
    assert auto_tensorize_cuda(keep, [Y], str(tmp_path / "ew.log"), 0) == {keep: []}
    assert "no matched intrinsic" in capsys.readouterr().out

    mo = at.MeasureOptions(target="cuda", dev_id=0)
    sub = _Subgraph([C], "batch_gemm")
    assert AutoTensorizeContext.can_use("bg", str(tmp_path), sub, mo)
    assert not AutoTensorizeContext.can_use("ew", str(tmp_path), _Subgraph([Y], "ew"), mo)
    ctx = AutoTensorizeContext("bg", str(tmp_path), sub, mo)
    assert ctx.get_best_schedule() == (None, None, at.MAX_FLOAT)  # nothing measured yet
    # an existing per-task log (name "at:<task>.log") is picked up
    with open(ctx.log_name, "w") as f:
        print(json.dumps({"record": {"tile_n": [128, 0], "cta_pair": [1, 0]}, "value": 4000.0}),
              file=f)
    ctx2 = AutoTensorizeContext("bg", str(tmp_path), sub, mo)
    sch2, args2 = ctx2.auto_schedule(0)
    assert args2 == [A, B, C] and sch2.plan.tile_n == 128 and sch2.plan.cta_pair == 1
    assert abs(ctx2.get_best_schedule()[2] - 0.25) < 1e-9  # 1/4000 s in milliseconds
    assert ctx2.get_measure_opt() is mo
    # the names the default context reaches for below the public API exist
    for name in ("get_match_results", "auto_tensorize_compute", "CUDAScheduleGeneratorV2",
                 "CUDAScheduleApplierV2", "CUDAProgramChecker", "get_cuda_compute_version",
                 "pebble_local_builder_build", "pebble_local_runner_run",
                 "find_optimized_parameters", "find_optimized_parameters_v2", "MAX_FLOAT"):
        assert hasattr(at, name), name


def test_log_round_trip(built_lib, tmp_path):
    A, B, C = ops.gemm(512, 512, 512)
    dag = at.compute_dag_from_tensors([C])
    log = tmp_path / "gemm.log"
    with open(log, "w") as f:
        print(json.dumps({"record": {"tile_n": [128, 0]}, "value": 2000.0}), file=f)
        print(json.dumps({"record": {"tile_n": [256, 0]}, "value": 5000.0}), file=f)
    mo = at.MeasureOptions(target="cuda")
    r = at.auto_tensorize_v4(dag, "cuda", str(log), mo, schedule_log_dir=str(tmp_path), trials=0)
    assert r.defined() and r.params.tile_n == 256
    assert abs(r.perf - 1 / 5000.0) < 1e-12
    assert r.sch_gen.get_best_entry().value == 5000.0
    assert r.params.to_json() == {"tile_n": [256, 0], "cta_pair": [0, 0]}
    sch, _ = at.get_schedule(r.sch_app, r.params)
    assert sch.plan.tile_n == 256
    r.sch_gen.load_from_file(str(log), clear=True)
    assert r.sch_gen.num_entries() == 2


def test_tuning_without_device_fails_loudly(built_lib, tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    A, B, C = ops.gemm(256, 256, 256)
    with pytest.raises(_lib.AmosbError):
        at.auto_tensorize(at.compute_dag_from_tensors([C]), "cuda", str(tmp_path / "x.log"),
                          at.MeasureOptions(target="cuda"), trials=4)

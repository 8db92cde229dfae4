"""CPU: the oracle against the golden vectors, and its two restatements against each other."""
import os

import numpy as np
import pytest


def test_c_matches_numpy_gemm(oracle):
    rng = np.random.default_rng(11)
    a = rng.uniform(-1, 1, (23, 47)).astype(np.float16)
    b = rng.uniform(-1, 1, (47, 31)).astype(np.float16)
    for mode in ("te_llvm", "exact"):
        ref = oracle.np_gemm(a, b, mode)
        for order in (0, 1):
            assert np.array_equal(oracle.c_gemm(a, b, mode, order=order), ref)
        bt = np.ascontiguousarray(b.T)
        assert np.array_equal(oracle.c_gemm(a, bt, mode, trans_b=True), ref)
    out16 = oracle.c_gemm(a, b, "te_llvm", out_dtype="float16")
    assert out16.dtype == np.float16
    assert np.array_equal(out16, oracle.np_gemm(a, b, "te_llvm", out_dtype="float16"))


def test_c_matches_numpy_batched(oracle):
    rng = np.random.default_rng(12)
    a = rng.normal(0, 1, (3, 9, 20)).astype(np.float16)
    b = rng.normal(0, 1, (3, 20, 13)).astype(np.float16)
    for mode in ("te_llvm", "exact"):
        assert np.array_equal(oracle.c_gemm(a, b, mode), oracle.np_gemm(a, b, mode))


def test_c_matches_numpy_int8(oracle):
    rng = np.random.default_rng(13)
    a = rng.integers(-128, 128, (17, 64), dtype=np.int8)
    b = rng.integers(-128, 128, (64, 29), dtype=np.int8)
    for mode in ("te_llvm", "exact"):
        for order in (0, 1):
            assert np.array_equal(oracle.c_gemm(a, b, mode, order=order), oracle.np_gemm(a, b, mode))
    # exact products are what int32 matmul gives
    assert np.array_equal(oracle.c_gemm(a, b, "exact"), a.astype(np.int32) @ b.astype(np.int32))
    # the llvm narrow multiply really is a different function of the same inputs
    assert not np.array_equal(oracle.c_gemm(a, b, "exact"), oracle.c_gemm(a, b, "te_llvm"))


def test_int8_extremes(oracle):
    a = np.full((4, 32), -128, dtype=np.int8)
    b = np.full((32, 16), -128, dtype=np.int8)
    assert (oracle.c_gemm(a, b, "exact") == 32 * 16384).all()
    assert (oracle.c_gemm(a, b, "te_llvm") == 0).all()  # (-128*-128) wraps to 0 in 8 bits


@pytest.mark.parametrize("geom", [(1, 1, 1), (2, 1, 1), (1, 2, 2), (1, 0, 1), (2, 0, 1)])
def test_c_matches_numpy_conv(oracle, geom):
    stride, pad, dil = geom
    rng = np.random.default_rng(14)
    x = rng.uniform(-1, 1, (2, 5, 9, 8)).astype(np.float16)
    w = rng.normal(0, 0.05, (6, 5, 3, 3)).astype(np.float16)
    for mode in ("te_llvm", "exact"):
        ref = oracle.np_conv2d_nchw(x, w, stride, pad, dil, mode)
        for order in (0, 1):
            got = oracle.c_conv2d_nchw(x, w, stride, pad, dil, mode, order=order)
            assert got.shape == ref.shape
            assert np.array_equal(got, ref)


@pytest.mark.parametrize("geom", [(1, 1, 1), (2, 1, 1), (1, 2, 2), (1, 0, 1)])
def test_nhwc_conv_is_the_nchw_conv_in_another_layout(oracle, geom):
    """The NHWC / RSCK operator: both restatements agree bit for bit, and in `exact` mode (float64
    sums, one rounding) it equals the NCHW operator on transposed operands up to the last bit of the
    different summation order."""
    stride, pad, dil = geom
    rng = np.random.default_rng(16)
    x = rng.uniform(-1, 1, (2, 9, 8, 5)).astype(np.float16)     # N H W C
    w = rng.normal(0, 0.05, (3, 3, 5, 6)).astype(np.float16)    # R S C K
    for mode in ("te_llvm", "exact"):
        ref = oracle.np_conv2d_nhwc(x, w, stride, pad, dil, mode)
        got = oracle.c_conv2d_nhwc(x, w, stride, pad, dil, mode)
        assert got.shape == ref.shape
        assert np.array_equal(got, ref)
    nchw = oracle.c_conv2d_nchw(np.ascontiguousarray(x.transpose(0, 3, 1, 2)),
                                np.ascontiguousarray(w.transpose(3, 2, 0, 1)), stride, pad, dil,
                                "exact")
    np.testing.assert_allclose(oracle.c_conv2d_nhwc(x, w, stride, pad, dil, "exact"),
                               nchw.transpose(0, 2, 3, 1), rtol=1e-6, atol=1e-7)
    out16 = oracle.c_conv2d_nhwc(x, w, stride, pad, dil, "te_llvm", out_dtype="float16")
    assert np.array_equal(out16, oracle.np_conv2d_nhwc(x, w, stride, pad, dil, "te_llvm",
                                                       out_dtype="float16"))


def test_nhwc_against_reference_conv2d_nchw_python(oracle, golden_dir):
    """The NHWC oracle on transposed golden inputs reproduces the reference helper's outputs."""
    g = np.load(os.path.join(golden_dir, "ref_topi_conv2d_nchw.npz"))
    for i in range(int(g["num_cases"])):
        a, w = g[f"case{i}_a"], g[f"case{i}_w"]
        stride, pad, dil = (int(v) for v in g[f"case{i}_geom"])
        ref = g[f"case{i}_out"]
        got = oracle.c_conv2d_nhwc(np.ascontiguousarray(a.transpose(0, 2, 3, 1)),
                                   np.ascontiguousarray(w.transpose(2, 3, 1, 0)), stride, pad, dil,
                                   "exact")
        np.testing.assert_allclose(got.transpose(0, 3, 1, 2), ref, rtol=2e-6, atol=1e-6)


def test_against_reference_conv2d_nhwc_python(oracle, golden_dir):
    """Outputs of the reference's own NHWC helper (python/tvm/topi/testing/conv2d_nhwc_python.py)
    on float16, int8 and tf32-representable float32 inputs pin the NHWC, HWNC, int8 and float32
    conv restatements: int8 bit for bit, the others to float32 rounding of the sums."""
    g = np.load(os.path.join(golden_dir, "ref_topi_conv2d_nhwc.npz"))
    seen = set()
    for i in range(int(g["num_cases"])):
        a, w = g[f"case{i}_a"], g[f"case{i}_w"]
        stride, pad, dil = (int(v) for v in g[f"case{i}_geom"])
        ref = g[f"case{i}_out"]
        hw = np.ascontiguousarray(a.transpose(1, 2, 0, 3))        # the same images as [H,W,N,C]
        seen.add(str(a.dtype))
        if a.dtype == np.int8:
            got = oracle.np_conv2d_nhwc(a, w, stride, pad, dil, "exact")
            assert got.dtype == np.int32 and np.array_equal(got, ref.astype(np.int64))
        elif a.dtype == np.float32:
            # exact tf32 values: every mode multiplies exactly, only the float32 sums round
            for mode in ("tf32", "tf32_rne", "tf32_trunc", "te_llvm"):
                got = oracle.np_conv2d_nhwc_f32(a, w, stride, pad, dil, mode)
                np.testing.assert_allclose(got, ref, rtol=2e-6, atol=2e-6)
            got = oracle.np_conv2d_nhwc_f32(hw, w, stride, pad, dil, "tf32", hwnc=True)
            np.testing.assert_allclose(got.transpose(2, 0, 1, 3), ref, rtol=2e-6, atol=2e-6)
        else:
            for got in (oracle.c_conv2d_nhwc(a, w, stride, pad, dil, "exact"),
                        oracle.np_conv2d_nhwc(a, w, stride, pad, dil, "exact"),
                        oracle.c_conv2d_hwnc(hw, w, stride, pad, dil, "exact").transpose(2, 0, 1, 3),
                        oracle.np_conv2d_hwnc(hw, w, stride, pad, dil, "exact").transpose(2, 0, 1, 3)):
                np.testing.assert_allclose(got, ref, rtol=2e-6, atol=1e-6)
    assert seen == {"float16", "int8", "float32"}


def test_against_reference_dilation_and_hwcn_helpers(oracle, golden_dir):
    """Dilated layers (the reference's tests dilate the filter with `dilate_python` and call the
    undilated helper) and the HWNC layout (the reference's `conv2d_hwcn_python` with the last two
    axes exchanged) pin the oracle's dilation arithmetic and its HWNC restatements: int8 bit for
    bit, float16 to float32 rounding of the sums."""
    g = np.load(os.path.join(golden_dir, "ref_topi_dilated_and_hwnc.npz"))
    kinds = set()
    for i in range(int(g["num_dil"])):
        a, w, ref = g[f"dil{i}_a"], g[f"dil{i}_w"], g[f"dil{i}_out"]
        stride, pad, dil = (int(v) for v in g[f"dil{i}_geom"])
        assert dil > 1
        layout = str(g[f"dil{i}_layout"])
        kinds.add((layout, str(a.dtype)))
        if layout == "nchw":
            gots = [oracle.np_conv2d_nchw(a, w, stride, pad, dil, "exact")]
            if a.dtype == np.float16:
                gots.append(oracle.c_conv2d_nchw(a, w, stride, pad, dil, "exact"))
        else:
            gots = [oracle.np_conv2d_nhwc(a, w, stride, pad, dil, "exact")]
            if a.dtype == np.float16:
                gots.append(oracle.c_conv2d_nhwc(a, w, stride, pad, dil, "exact"))
        for got in gots:
            assert got.shape == ref.shape
            if a.dtype == np.int8:
                assert np.array_equal(got, ref.astype(np.int64))
            else:
                np.testing.assert_allclose(got, ref, rtol=2e-6, atol=1e-6)
    assert kinds == {("nchw", "float16"), ("nchw", "int8"), ("nhwc", "float16"), ("nhwc", "int8")}
    for i in range(int(g["num_hwnc"])):
        a, w, ref = g[f"hwnc{i}_a"], g[f"hwnc{i}_w"], g[f"hwnc{i}_out"]
        stride, pad, dil = (int(v) for v in g[f"hwnc{i}_geom"])
        if a.dtype == np.int8:
            got = oracle.np_conv2d_nhwc(np.ascontiguousarray(a.transpose(2, 0, 1, 3)), w, stride, pad,
                                        dil, "exact").transpose(1, 2, 0, 3)
            assert np.array_equal(got, ref.astype(np.int64))
        else:
            for got in (oracle.c_conv2d_hwnc(a, w, stride, pad, dil, "exact"),
                        oracle.np_conv2d_hwnc(a, w, stride, pad, dil, "exact")):
                np.testing.assert_allclose(got, ref, rtol=2e-6, atol=1e-6)


def test_fp16_modes_are_close(oracle):
    """Rounding every product to fp16 moves the result by about 2^-11/sqrt(3) relative."""
    rng = np.random.default_rng(15)
    a = rng.uniform(-1, 1, (64, 512)).astype(np.float16)
    b = rng.uniform(-1, 1, (512, 64)).astype(np.float16)
    err = oracle.rel_l2(oracle.c_gemm(a, b, "te_llvm"), oracle.c_gemm(a, b, "exact"))
    assert 5e-5 < err < 1e-3


def test_against_reference_conv2d_nchw_python(oracle, golden_dir):
    """`exact` mode reproduces the outputs of the reference's conv2d_nchw_python helper."""
    g = np.load(os.path.join(golden_dir, "ref_topi_conv2d_nchw.npz"))
    for i in range(int(g["num_cases"])):
        a, w = g[f"case{i}_a"], g[f"case{i}_w"]
        stride, pad, dil = (int(v) for v in g[f"case{i}_geom"])
        ref = g[f"case{i}_out"]
        got = oracle.c_conv2d_nchw(a, w, stride, pad, dil, "exact")
        assert got.shape == ref.shape
        # float64 sums in a different order, then one rounding to float32
        np.testing.assert_allclose(got, ref, rtol=2e-6, atol=1e-6)
        got_np = oracle.np_conv2d_nchw(a, w, stride, pad, dil, "exact")
        np.testing.assert_allclose(got_np, ref, rtol=2e-6, atol=1e-6)
        assert oracle.rel_l2(oracle.c_conv2d_nchw(a, w, stride, pad, dil, "te_llvm"), ref) < 1e-3


def test_against_reference_batch_matmul(oracle, golden_dir):
    """`exact` mode reproduces the reference's batch_matmul helper (y is [batch, N, K])."""
    g = np.load(os.path.join(golden_dir, "ref_topi_batch_matmul.npz"))
    for i in range(int(g["num_cases"])):
        x, y, ref = g[f"case{i}_x"], g[f"case{i}_y"], g[f"case{i}_out"]
        got = oracle.c_gemm(x, y, "exact", trans_b=True)
        np.testing.assert_allclose(got, ref, rtol=2e-6, atol=1e-5)
        got2 = oracle.c_gemm(x, np.ascontiguousarray(np.swapaxes(y, 1, 2)), "exact")
        assert np.array_equal(got, got2)
        xi, yi, refi = g[f"case{i}_xi"], g[f"case{i}_yi"], g[f"case{i}_outi"]
        assert np.array_equal(oracle.c_gemm(xi, yi, "exact", trans_b=True), refi.astype(np.int32))


def test_known_answers(oracle, golden_dir):
    k = np.load(os.path.join(golden_dir, "kat_oracle.npz"))
    assert np.array_equal(oracle.c_gemm(k["gemm_a"], k["gemm_b"], "te_llvm"), k["gemm_te_llvm"])
    assert np.array_equal(oracle.c_gemm(k["gemm_a"], k["gemm_b"], "exact"), k["gemm_exact"])
    assert np.array_equal(oracle.c_gemm(k["gemm_a"], k["gemm_b"], "te_llvm", out_dtype="float16"),
                          k["gemm_te_llvm_f16out"])
    assert np.array_equal(oracle.np_gemm(k["gemm_a"], k["gemm_b"], "te_llvm"), k["gemm_te_llvm"])
    assert np.array_equal(oracle.c_gemm(k["gemm8_a"], k["gemm8_b"], "exact"), k["gemm8_exact"])
    assert np.array_equal(oracle.c_gemm(k["gemm8_a"], k["gemm8_b"], "te_llvm"), k["gemm8_te_llvm"])
    assert np.array_equal(oracle.c_gemm(k["bgemm_a"], k["bgemm_b"], "exact"), k["bgemm_exact"])
    assert np.array_equal(oracle.c_gemm(k["bgemm_a"], k["bgemm_b"], "te_llvm",
                                        out_dtype="float16"), k["bgemm_te_llvm_f16out"])
    assert np.array_equal(oracle.c_conv2d_nchw(k["conv_a"], k["conv_w"], 1, 1, 1, "te_llvm"),
                          k["conv_te_llvm"])
    assert np.array_equal(oracle.c_conv2d_nchw(k["conv_a"], k["conv_w"], 1, 1, 1, "exact"),
                          k["conv_exact"])
    assert np.array_equal(oracle.c_conv2d_nchw(k["conv_a"], k["conv_w"], 2, 1, 1, "te_llvm"),
                          k["conv_s2_te_llvm"])
    assert np.array_equal(oracle.c_conv2d_nchw(k["conv_a"], k["conv_w"], 1, 2, 2, "te_llvm"),
                          k["conv_d2_te_llvm"])


def test_threads_do_not_change_results(oracle):
    rng = np.random.default_rng(16)
    a = rng.uniform(-1, 1, (40, 96)).astype(np.float16)
    b = rng.uniform(-1, 1, (96, 48)).astype(np.float16)
    assert np.array_equal(oracle.c_gemm(a, b, "te_llvm", threads=1),
                          oracle.c_gemm(a, b, "te_llvm", threads=4))


def test_bfloat16_carrier_and_semantics(oracle):
    """bfloat16 operands travel as float32 arrays of representable values.  Rounding is to
    nearest-even like torch's; the `te_llvm` mode multiplies exactly (the reference's legalisation
    promotes to float32 and the cast back is eliminated, src/tir/transforms/bf16_legalize.cc:80-94,
    131-152), so it differs from `exact` only by float32 accumulation."""
    import torch
    rng = np.random.default_rng(21)
    x = np.concatenate([rng.normal(0, 1, 4096), rng.normal(0, 1e-3, 512), [0.0, -0.0, 1.0, 65504.0],
                        # ties: exactly half way between two bfloat16 values
                        np.array([0x3F808000, 0x3F818000, 0xBF808000], dtype=np.uint32)
                        .view(np.float32)]).astype(np.float32)
    mine = oracle.to_bf16(x)
    theirs = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(mine.view(np.uint32), theirs.view(np.uint32))
    assert np.array_equal(oracle.to_bf16(mine), mine)  # idempotent
    a = oracle.to_bf16(rng.uniform(-1, 1, (33, 70)))
    b = oracle.to_bf16(rng.uniform(-1, 1, (70, 21)))
    te = oracle.np_gemm(a, b, "te_llvm")
    ex = oracle.np_gemm(a, b, "exact")
    assert ex.dtype == np.float32 and np.allclose(ex, a.astype(np.float64) @ b.astype(np.float64))
    assert 0 < oracle.rel_l2(te, ex) < 1e-6        # exact products, only the accumulator differs
    with pytest.raises(AssertionError):
        oracle.np_gemm(a + np.float32(1e-4), b, "te_llvm")  # not bfloat16-representable
    xh = oracle.to_bf16(rng.uniform(-1, 1, (2, 6, 5, 8)))
    wh = oracle.to_bf16(rng.normal(0, 0.1, (3, 3, 8, 4)))
    nhwc = oracle.np_conv2d_nhwc(xh, wh, 1, 1, 1, "exact")
    nchw = oracle.np_conv2d_nchw(np.ascontiguousarray(xh.transpose(0, 3, 1, 2)),
                                 np.ascontiguousarray(wh.transpose(3, 2, 0, 1)), 1, 1, 1, "exact")
    np.testing.assert_allclose(nhwc, nchw.transpose(0, 2, 3, 1), rtol=1e-6, atol=1e-7)


def test_tf32_conversion_and_semantics(oracle):
    """float32 operands of the reference's tf32 intrinsic: `__float_to_tf32` keeps 10 mantissa bits,
    rounding to nearest with ties away from zero (reference:
    python/tvm/auto_tensorize/hw_abstraction/cuda/wmma_tf32.py:124-133).  Known answers by hand:
    one tf32 step at 1.0 is 2**-10."""
    u = np.float32(2.0 ** -10)
    x = np.array([1.0, 1 + u / 2, 1 + u / 2 - 2.0 ** -23, 1 + u / 4, 1 + 3 * u / 2, -(1 + u / 2),
                  -(1 + u / 4), 0.0, 3.0e38 * 0 + 65504.0], np.float32)
    want_rna = np.array([1.0, 1 + u, 1.0, 1.0, 1 + 2 * u, -(1 + u), -1.0, 0.0, 65504.0], np.float32)
    want_trunc = np.array([1.0, 1.0, 1.0, 1.0, 1 + u, -1.0, -1.0, 0.0, 65504.0], np.float32)
    assert np.array_equal(oracle.to_tf32(x), want_rna)
    assert np.array_equal(oracle.to_tf32(x, "trunc"), want_trunc)
    # ties to even: what a TMA copy of type TFLOAT32 does; differs from rna on the exact ties only
    want_rne = np.array([1.0, 1.0, 1.0, 1.0, 1 + 2 * u, -1.0, -1.0, 0.0, 65504.0], np.float32)
    assert np.array_equal(oracle.to_tf32(x, "rne"), want_rne)
    rng = np.random.default_rng(41)
    y = rng.normal(0, 3, 4096).astype(np.float32)
    r = oracle.to_tf32(y)
    assert np.array_equal(oracle.to_tf32(r), r) and np.array_equal(oracle.to_tf32(r, "trunc"), r)
    differ = oracle.to_tf32(y, "rne") != r                  # only where y is an exact tie
    assert differ.sum() <= 8 and np.all(y.view(np.uint32)[differ] & np.uint32(0x1FFF) == 0x1000)
    assert not (r.view(np.uint32) & np.uint32(0x1FFF)).any()
    assert np.all(np.abs(r - y) <= np.abs(y) * 2.0 ** -11)
    assert np.all(np.abs(oracle.to_tf32(y, "trunc")) <= np.abs(y))
    # the three arithmetic modes on one GEMM: the llvm build (plain float32) is the exact answer to
    # float32 rounding; converting the operands costs ~3e-4 (rna) / ~8e-4 (truncation, biased)
    a = rng.uniform(-1, 1, (40, 96)).astype(np.float32)
    b = rng.uniform(-1, 1, (96, 24)).astype(np.float32)
    exact = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    assert oracle.rel_l2(oracle.np_gemm_f32(a, b, "te_llvm"), exact) <= 1e-6
    e_rna = oracle.rel_l2(oracle.np_gemm_f32(a, b, "tf32"), exact)
    e_tr = oracle.rel_l2(oracle.np_gemm_f32(a, b, "tf32_trunc"), exact)
    assert 5e-5 < e_rna < 6e-4 and e_rna < e_tr < 1e-3
    # the C restatement of the float32 text equals the numpy one bit for bit, in both loop orders
    for order in (0, 1):
        assert np.array_equal(oracle.c_gemm(a, b, order=order), oracle.np_gemm_f32(a, b, "te_llvm"))
    assert np.array_equal(oracle.c_gemm(oracle.to_tf32(a), np.ascontiguousarray(oracle.to_tf32(b).T),
                                        trans_b=True), oracle.np_gemm_f32(a, b, "tf32"))
    # sequential float32 sums and the float64 shortcut agree to float32 rounding; layouts
    assert oracle.rel_l2(oracle.np_gemm_f32(a, b, "tf32", sequential=False),
                         oracle.np_gemm_f32(a, b, "tf32")) <= 1e-6
    assert np.array_equal(oracle.np_gemm_f32(np.ascontiguousarray(a.T), np.ascontiguousarray(b.T),
                                             "tf32", trans_a=True, trans_b=True),
                          oracle.np_gemm_f32(a, b, "tf32"))


def test_int8_conv_modes(oracle):
    """int8 NHWC conv: `exact` is the plain integer convolution (checked against a float64 einsum
    over the padded tensor, exact at these magnitudes); `te_llvm` wraps every product to 8 bits
    first, like the int8 GEMM's `te_llvm` mode, and therefore differs."""
    rng = np.random.default_rng(51)
    x = rng.integers(-128, 128, (2, 6, 5, 16), dtype=np.int8)
    w = rng.integers(-128, 128, (3, 3, 16, 8), dtype=np.int8)
    got = oracle.np_conv2d_nhwc(x, w, 1, 1, 1, "exact")
    assert got.dtype == np.int32
    pad = np.zeros((2, 8, 7, 16), np.float64)
    pad[:, 1:7, 1:6] = x
    want = np.zeros((2, 6, 5, 8), np.float64)
    for rr in range(3):
        for rs in range(3):
            want += np.einsum("nhwc,ck->nhwk", pad[:, rr:rr + 6, rs:rs + 5], w[rr, rs].astype(np.float64))
    assert np.array_equal(got, want.astype(np.int32))
    wrapped = oracle.np_conv2d_nhwc(x, w, 1, 1, 1, "te_llvm")
    assert wrapped.dtype == np.int32 and not np.array_equal(wrapped, got)
    # products that fit 8 bits are not changed by the wrap
    xs, ws = (x % 8).astype(np.int8), (w % 8).astype(np.int8)
    assert np.array_equal(oracle.np_conv2d_nhwc(xs, ws, 1, 1, 1, "te_llvm"),
                          oracle.np_conv2d_nhwc(xs, ws, 1, 1, 1, "exact"))


def test_hwnc_conv_restatements_agree(oracle):
    """HWNC (reference: benchmark/amos/mapping_conv2d_tensorcore.py:74-104): the numpy restatement
    written directly on [H,W,N,C] equals, bit for bit, the C oracle of the NHWC operator between
    two transpositions (same products, same accumulation order rr, rs, rc)."""
    rng = np.random.default_rng(31)
    x = rng.uniform(-1, 1, (9, 8, 3, 5)).astype(np.float16)      # H W N C
    w = rng.normal(0, 0.05, (3, 3, 5, 6)).astype(np.float16)     # R S C K
    for stride, pad, dil in ((1, 1, 1), (2, 1, 1), (1, 2, 2), (1, 0, 1)):
        for mode in ("te_llvm", "exact"):
            ref = oracle.np_conv2d_hwnc(x, w, stride, pad, dil, mode)
            got = oracle.c_conv2d_hwnc(x, w, stride, pad, dil, mode)
            assert got.shape == ref.shape and np.array_equal(got, ref)

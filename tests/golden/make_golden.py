"""Generate the committed golden fixtures of tests/golden/.

Run once, in an environment that has the reference checkout (by default a directory `reference`
beside this repository; AMOS_REFERENCE overrides it):  ``python tests/golden/make_golden.py``

Two families of fixtures are written:

1. ``ref_topi_*.npz`` -- outputs of the REFERENCE's own numpy/scipy test helpers on seeded inputs:
   ``conv2d_nchw_python`` (reference: python/tvm/topi/testing/conv2d_nchw_python.py:24-110),
   ``conv2d_nhwc_python`` (python/tvm/topi/testing/conv2d_nhwc_python.py:24-110) and
   ``batch_matmul`` (reference: python/tvm/topi/testing/batch_matmul.py:22-44).  The helper modules
   are loaded from the reference checkout file by file; the one symbol they import from the rest
   of TVM, ``get_pad_tuple`` (reference: python/tvm/topi/nn/util.py:118-165), is taken from the
   reference source too (its function definition is compiled on its own, because importing the
   ``tvm`` package needs a built libtvm).  These pin the oracle's ``exact`` mode.
2. ``kat_*.npz`` -- known-answer vectors produced by the oracle itself (C restatement, both
   modes) for small seeded cases of every operator, so that a later change of the oracle or of the
   kernels is caught against fixed numbers.

The fixtures are small (a few hundred KB in total); this script is the only thing that reads the
reference checkout, and nothing reads it at test time.
"""
from __future__ import annotations

import ast
import importlib.util
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("AMOS_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))


def _load_reference_helpers():
    util_path = os.path.join(REF, "python/tvm/topi/nn/util.py")
    src = open(util_path).read()
    tree = ast.parse(src)
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "get_pad_tuple"]
    assert fn, "get_pad_tuple not found in the reference"
    mod = ast.Module(body=fn, type_ignores=[])
    ns: dict = {}
    exec(compile(mod, util_path, "exec"), ns)
    # Minimal package skeleton so that `from tvm.topi.nn.util import get_pad_tuple` resolves.
    for name in ("tvm", "tvm.topi", "tvm.topi.nn", "tvm.topi.nn.util"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["tvm.topi.nn.util"].get_pad_tuple = ns["get_pad_tuple"]

    def load(rel, name):
        spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel))
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        return m

    conv = load("python/tvm/topi/testing/conv2d_nchw_python.py", "_ref_conv2d_nchw_python")
    bmm = load("python/tvm/topi/testing/batch_matmul.py", "_ref_batch_matmul")
    nhwc = load("python/tvm/topi/testing/conv2d_nhwc_python.py", "_ref_conv2d_nhwc_python")
    global _dilate_python, _conv2d_hwcn_python
    _dilate_python = load("python/tvm/topi/testing/dilate_python.py", "_ref_dilate_python").dilate_python
    _conv2d_hwcn_python = load("python/tvm/topi/testing/conv2d_hwcn_python.py",
                               "_ref_conv2d_hwcn_python").conv2d_hwcn_python
    return conv.conv2d_nchw_python, bmm.batch_matmul, nhwc.conv2d_nhwc_python


_dilate_python = None
_conv2d_hwcn_python = None


def write_dilated_and_hwnc(conv2d_nchw_python, conv2d_nhwc_python):
    """``ref_topi_dilated_and_hwnc.npz``: what the reference's helpers give for the two things the
    files above do not reach.

    * Dilation: the reference's tests dilate the FILTER with ``dilate_python`` (reference:
      python/tvm/topi/testing/dilate_python.py:22-52) and run the undilated helper on it; the same
      is done here for NCHW / KCRS and NHWC / RSCK, float16 and int8.
    * HWNC: the reference has a helper for ``[H, W, C, N]`` activations and ``[P, Q, K, N]`` outputs
      (``conv2d_hwcn_python``, python/tvm/topi/testing/conv2d_hwcn_python.py:24-78); an HWNC
      problem is that one with the last two axes of activation and output exchanged.
    """
    rng = np.random.default_rng(20260007)
    out = {}
    dil_cases = [
        # (layout, N, C, H, W, K, R, S, stride, pad, dil, kind)
        ("nchw", 2, 16, 11, 9, 24, 3, 3, 1, 2, 2, "f16"),
        ("nchw", 1, 8, 15, 15, 16, 3, 3, 2, 3, 3, "f16"),
        ("nchw", 1, 16, 12, 12, 8, 3, 3, 1, 2, 2, "s8"),
        ("nhwc", 2, 16, 11, 9, 24, 3, 3, 1, 2, 2, "f16"),
        ("nhwc", 1, 32, 13, 13, 16, 3, 3, 1, 2, 2, "s8"),
    ]
    for i, (layout, n, c, h, w, k, r, s, st, pd, dl, kind) in enumerate(dil_cases):
        if kind == "s8":
            a = rng.integers(-128, 128, (n, c, h, w), dtype=np.int8)
            wt = rng.integers(-128, 128, (k, c, r, s), dtype=np.int8)
        else:
            a = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float16)
            wt = rng.normal(0, 0.05, (k, c, r, s)).astype(np.float16)
        if layout == "nchw":
            dw = _dilate_python(wt.astype(np.float64), (1, 1, dl, dl))
            ref = conv2d_nchw_python(a.astype(np.float64), dw, st, pd)
        else:
            a = np.ascontiguousarray(a.transpose(0, 2, 3, 1))    # [N, H, W, C]
            wt = np.ascontiguousarray(wt.transpose(2, 3, 1, 0))  # [R, S, C, K]
            dw = _dilate_python(wt.astype(np.float64), (dl, dl, 1, 1))
            ref = conv2d_nhwc_python(a.astype(np.float64), dw, st, pd)
        out[f"dil{i}_layout"] = np.array(layout)
        out[f"dil{i}_a"], out[f"dil{i}_w"] = a, wt
        out[f"dil{i}_geom"] = np.array([st, pd, dl], dtype=np.int64)
        out[f"dil{i}_out"] = ref
    out["num_dil"] = np.array(len(dil_cases))
    hwnc_cases = [
        # (H, W, N, C, K, R, S, stride, pad, kind)
        (7, 6, 5, 16, 24, 3, 3, 1, 1, "f16"),
        (9, 9, 3, 8, 16, 3, 3, 2, 1, "f16"),
        (6, 6, 4, 16, 16, 1, 1, 1, 0, "s8"),
        (8, 7, 2, 32, 16, 3, 3, 1, 1, "s8"),
    ]
    for i, (h, w, n, c, k, r, s, st, pd, kind) in enumerate(hwnc_cases):
        if kind == "s8":
            a = rng.integers(-128, 128, (h, w, n, c), dtype=np.int8)
            wt = rng.integers(-128, 128, (r, s, c, k), dtype=np.int8)
        else:
            a = rng.uniform(-1, 1, (h, w, n, c)).astype(np.float16)
            wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float16)
        ref = _conv2d_hwcn_python(a.astype(np.float64).transpose(0, 1, 3, 2), wt.astype(np.float64),
                                  st, pd)                      # [P, Q, K, N]
        out[f"hwnc{i}_a"], out[f"hwnc{i}_w"] = a, wt
        out[f"hwnc{i}_geom"] = np.array([st, pd, 1], dtype=np.int64)
        out[f"hwnc{i}_out"] = np.ascontiguousarray(ref.transpose(0, 1, 3, 2))  # [P, Q, N, K]
    out["num_hwnc"] = np.array(len(hwnc_cases))
    np.savez_compressed(os.path.join(HERE, "ref_topi_dilated_and_hwnc.npz"), **out)


def main():
    from oracle import oracle as o

    conv2d_nchw_python, batch_matmul, conv2d_nhwc_python = _load_reference_helpers()
    rng = np.random.default_rng(20260001)

    # ---- 1. reference helpers -------------------------------------------------------------
    conv_cases = [
        # (N, C, H, W, K, R, S, stride, pad)
        (1, 64, 8, 8, 64, 3, 3, 1, 1),     # the README layer shape, spatially reduced
        (2, 16, 9, 7, 24, 3, 3, 1, 1),     # ragged extents
        (2, 64, 14, 14, 32, 1, 1, 1, 0),   # 1x1
        (1, 8, 15, 15, 16, 3, 3, 2, 1),    # stride 2
        (1, 8, 12, 12, 8, 5, 5, 1, 2),     # 5x5
    ]
    out = {}
    for i, (n, c, h, w, k, r, s, st, pd) in enumerate(conv_cases):
        a = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float16)
        wt = rng.normal(0, 0.05, (k, c, r, s)).astype(np.float16)
        ref = conv2d_nchw_python(a.astype(np.float64), wt.astype(np.float64), st, pd)
        out[f"case{i}_a"] = a
        out[f"case{i}_w"] = wt
        out[f"case{i}_geom"] = np.array([st, pd, 1], dtype=np.int64)
        out[f"case{i}_out"] = ref  # float64
    out["num_cases"] = np.array(len(conv_cases))
    np.savez_compressed(os.path.join(HERE, "ref_topi_conv2d_nchw.npz"), **out)

    out = {}
    bmm_cases = [(4, 32, 48, 16), (3, 33, 17, 40), (2, 64, 64, 64)]  # (batch, M, N, K)
    for i, (b, m, n, k) in enumerate(bmm_cases):
        x = rng.normal(0, 1, (b, m, k)).astype(np.float16)
        y = rng.normal(0, 1, (b, n, k)).astype(np.float16)  # the helper takes y as [batch, N, K]
        ref = batch_matmul(x.astype(np.float64), y.astype(np.float64))
        out[f"case{i}_x"] = x
        out[f"case{i}_y"] = y
        out[f"case{i}_out"] = ref
        xi = rng.integers(-128, 128, (b, m, k), dtype=np.int8)
        yi = rng.integers(-128, 128, (b, n, k), dtype=np.int8)
        out[f"case{i}_xi"] = xi
        out[f"case{i}_yi"] = yi
        out[f"case{i}_outi"] = batch_matmul(xi.astype(np.int64), yi.astype(np.int64))
    out["num_cases"] = np.array(len(bmm_cases))
    np.savez_compressed(os.path.join(HERE, "ref_topi_batch_matmul.npz"), **out)

    # NHWC / RSCK helper (reference: python/tvm/topi/testing/conv2d_nhwc_python.py:24-110) on
    # float16, int8 and tf32-representable float32 inputs; own generator, so that the two files
    # above keep their contents
    rng = np.random.default_rng(20260005)
    out = {}
    nhwc_cases = [
        # (N, H, W, C, K, R, S, stride, pad, kind)
        (2, 9, 7, 16, 24, 3, 3, 1, 1, "f16"),
        (1, 15, 15, 8, 16, 3, 3, 2, 1, "f16"),
        (2, 10, 10, 40, 8, 1, 1, 1, 0, "f16"),
        (2, 9, 7, 16, 24, 3, 3, 1, 1, "s8"),
        (1, 12, 12, 32, 16, 5, 5, 1, 2, "s8"),
        (2, 9, 7, 12, 24, 3, 3, 1, 1, "tf32"),
        (1, 15, 15, 8, 16, 3, 3, 2, 1, "tf32"),
    ]
    for i, (n, h, w, c, k, r, s, st, pd, kind) in enumerate(nhwc_cases):
        if kind == "s8":
            a = rng.integers(-128, 128, (n, h, w, c), dtype=np.int8)
            wt = rng.integers(-128, 128, (r, s, c, k), dtype=np.int8)
        elif kind == "tf32":  # float32 values that are exact tf32 numbers (10 mantissa bits)
            a = o.to_tf32(rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32))
            wt = o.to_tf32(rng.normal(0, 0.05, (r, s, c, k)).astype(np.float32))
        else:
            a = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float16)
            wt = rng.normal(0, 0.05, (r, s, c, k)).astype(np.float16)
        ref = conv2d_nhwc_python(a.astype(np.float64), wt.astype(np.float64), st, pd)
        out[f"case{i}_a"] = a
        out[f"case{i}_w"] = wt
        out[f"case{i}_geom"] = np.array([st, pd, 1], dtype=np.int64)
        out[f"case{i}_out"] = ref  # float64; exact for the int8 cases
    out["num_cases"] = np.array(len(nhwc_cases))
    np.savez_compressed(os.path.join(HERE, "ref_topi_conv2d_nhwc.npz"), **out)

    write_dilated_and_hwnc(conv2d_nchw_python, conv2d_nhwc_python)

    # ---- 2. known-answer vectors of the oracle --------------------------------------------
    rng = np.random.default_rng(20260002)
    kat = {}
    a = rng.uniform(-1, 1, (150, 72)).astype(np.float16)
    b = rng.uniform(-1, 1, (72, 136)).astype(np.float16)
    kat["gemm_a"], kat["gemm_b"] = a, b
    kat["gemm_te_llvm"] = o.c_gemm(a, b, "te_llvm")
    kat["gemm_exact"] = o.c_gemm(a, b, "exact")
    kat["gemm_te_llvm_f16out"] = o.c_gemm(a, b, "te_llvm", out_dtype="float16")
    ai = rng.integers(-128, 128, (130, 96), dtype=np.int8)
    bi = rng.integers(-128, 128, (96, 144), dtype=np.int8)
    kat["gemm8_a"], kat["gemm8_b"] = ai, bi
    kat["gemm8_exact"] = o.c_gemm(ai, bi, "exact")
    kat["gemm8_te_llvm"] = o.c_gemm(ai, bi, "te_llvm")
    q = rng.normal(0, 1, (3, 40, 24)).astype(np.float16)
    kt = rng.normal(0, 1, (3, 24, 56)).astype(np.float16)
    kat["bgemm_a"], kat["bgemm_b"] = q, kt
    kat["bgemm_te_llvm_f16out"] = o.c_gemm(q, kt, "te_llvm", out_dtype="float16")
    kat["bgemm_exact"] = o.c_gemm(q, kt, "exact")
    x = rng.uniform(-1, 1, (2, 24, 10, 9)).astype(np.float16)
    w = rng.normal(0, 0.05, (40, 24, 3, 3)).astype(np.float16)
    kat["conv_a"], kat["conv_w"] = x, w
    kat["conv_te_llvm"] = o.c_conv2d_nchw(x, w, 1, 1, 1, "te_llvm")
    kat["conv_exact"] = o.c_conv2d_nchw(x, w, 1, 1, 1, "exact")
    kat["conv_s2_te_llvm"] = o.c_conv2d_nchw(x, w, 2, 1, 1, "te_llvm")
    kat["conv_d2_te_llvm"] = o.c_conv2d_nchw(x, w, 1, 2, 2, "te_llvm")
    np.savez_compressed(os.path.join(HERE, "kat_oracle.npz"), **kat)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()

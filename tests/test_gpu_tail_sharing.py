"""GPU: the shared-out tail of a schedule (k-blocks of the last, short round of tiles cut into
equal shares; partial sums exchanged through scratch memory and flags).

By default only large problems take that path; AMOSB_TAIL_SHARING=1 forces it whenever a round is
short, which is how every kernel family is put through it here on shapes the oracle finishes
quickly.  Integers must come out bit for bit; floats may differ from the whole-tile schedule by the
order of the fp32 additions only."""
import os
from contextlib import contextmanager

import numpy as np
import pytest
import torch

from amos_b200 import _lib, device

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_TE_LLVM = 1e-3
TOL_REORDER = 1e-5


@contextmanager
def _env(**kw):
    old = {k: os.environ.get(k) for k in kw}
    os.environ.update({k: v for k, v in kw.items()})
    try:
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def _run(desc, ins, shape, shared):
    """Run with a guard band; `shared` forces the tail to be shared out, else forbids it."""
    tdt = device.CODE_TO_TORCH[desc.out_dtype]
    numel = int(np.prod(shape))
    buf = torch.full((numel + 2048,), 77, dtype=tdt, device=DEV)
    out = buf[1024:1024 + numel].view(shape)
    with _env(**({"AMOSB_TAIL_SHARING": "1"} if shared else {"AMOSB_NO_TAIL_SHARING": "1"})):
        extra = _lib.workspace_bytes(desc) - _lib.workspace_bytes_min(desc)
        assert (extra > 0) == shared, "the plan does not share the tail as the test expects"
        ws = torch.empty(_lib.workspace_bytes(desc) + 1024, dtype=torch.uint8, device=DEV)
        device.run(desc, ins, [out], workspace=ws)
    assert device.status_peek(0) == 0
    assert (buf[:1024] == 77).all() and (buf[1024 + numel:] == 77).all(), "wrote outside the output"
    return out.cpu().numpy()


FAMILIES = [(256, 1), (128, 1), (64, 1), (128, 3), (256, 2), (128, 2)]


@pytest.mark.parametrize("tile_n,cta_pair", FAMILIES)
@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_fp16_every_family(oracle, tile_n, cta_pair, trans_b):
    m, n, k = 1100, 520, 1032  # 17 k-blocks; a tile is cut into up to ~15 shares
    rng = np.random.default_rng(tile_n + cta_pair)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (n, k) if trans_b else (k, n)).astype(np.float16)
    d = _lib.gemm_desc(m, n, k, trans_b=trans_b, tile_n=tile_n, cta_pair=cta_pair)
    ins = [_t(a), _t(b)]
    got = _run(d, ins, (m, n), True)
    whole = _run(d, ins, (m, n), False)
    assert oracle.rel_l2(got, oracle.c_gemm(a, b, "te_llvm", trans_b=trans_b)) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, whole) <= TOL_REORDER
    # the same shares every time: the result is reproducible bit for bit
    assert np.array_equal(got, _run(d, ins, (m, n), True))


@pytest.mark.parametrize("tile_n,cta_pair", [(256, 1), (128, 1), (256, 2)])
def test_gemm_int8_is_bit_exact(oracle, tile_n, cta_pair):
    m, n, k = 700, 528, 2192  # 18 k-blocks of 128, the last one ragged
    rng = np.random.default_rng(9 + tile_n)
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    d = _lib.gemm_desc(m, n, k, in_dtype=_lib.AMOSB_S8, tile_n=tile_n, cta_pair=cta_pair)
    got = _run(d, [_t(a), _t(b)], (m, n), True)
    assert np.array_equal(got, oracle.c_gemm(a, b, "exact"))


@pytest.mark.parametrize("tile_n,cta_pair", [(256, 1), (128, 1), (256, 2), (128, 2)])
def test_gemm_tf32_single_cta_and_pairs(oracle, tile_n, cta_pair):
    m, n, k = 1100, 520, 520  # 17 k-blocks of 32, the last one ragged
    rng = np.random.default_rng(31 + tile_n + cta_pair)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    d = _lib.gemm_desc(m, n, k, in_dtype=_lib.AMOSB_F32, tile_n=tile_n, cta_pair=cta_pair)
    ins = [_t(a), _t(b)]
    got = _run(d, ins, (m, n), True)
    whole = _run(d, ins, (m, n), False)
    assert oracle.rel_l2(got, oracle.np_gemm_f32(a, b, "tf32_rne")) <= 2e-5
    assert oracle.rel_l2(got, whole) <= TOL_REORDER
    assert np.array_equal(got, _run(d, ins, (m, n), True))


def test_round_of_whole_tiles_after_the_shares(oracle):
    """More tiles than CTAs: shares first, then whole tiles on the same accumulators."""
    m, n, k = 128 * 20, 2048, 2048  # 160 tiles of 128 x 256, 32 k-blocks: 12 tiles shared out
    rng = np.random.default_rng(4)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    d = _lib.gemm_desc(m, n, k, out_dtype=_lib.AMOSB_F16, tile_n=256, cta_pair=1)
    ins = [_t(a), _t(b)]
    got = _run(d, ins, (m, n), True)
    whole = _run(d, ins, (m, n), False)
    rows = [0, 1, 127, 128, 1300, 2559]
    ref = oracle.c_gemm(a[rows], b, "te_llvm").astype(np.float16)
    assert oracle.rel_l2(got[rows].astype(np.float32), ref.astype(np.float32)) <= TOL_TE_LLVM
    assert oracle.rel_l2(got.astype(np.float32), whole.astype(np.float32)) <= 1e-3  # fp16 outputs


def test_batched_gemm_with_bias_and_relu(oracle):
    batch, m, n, k = 5, 264, 200, 640
    rng = np.random.default_rng(5)
    a = rng.normal(0, 1, (batch, m, k)).astype(np.float16)
    b = rng.normal(0, 1, (batch, k, n)).astype(np.float16)
    bias = rng.uniform(-1, 1, (n,)).astype(np.float32)
    d = _lib.gemm_desc(m, n, k, batch=batch, batched=True, tile_n=128, cta_pair=1)
    d.epilogue, d.arg_c, d.addend_dtype = _lib.EPI_ADD_VECTOR | _lib.EPI_RELU, 2, _lib.AMOSB_F32
    got = _run(d, [_t(a), _t(b), _t(bias)], (batch, m, n), True)
    ref = np.maximum(oracle.c_gemm(a, b, "te_llvm") + bias, 0)
    assert oracle.rel_l2(got, ref) <= TOL_TE_LLVM


CONVS = [
    # layout, N, C, H, W, K, R, pad, tile_n, cta_pair
    ("nchw", 9, 136, 14, 14, 264, 3, 1, 256, 2),
    ("nchw", 9, 136, 14, 14, 264, 3, 1, 128, 3),
    ("nchw", 9, 136, 14, 14, 264, 3, 1, 128, 1),
    ("nchw", 12, 1024, 14, 14, 256, 1, 0, 0, 0),   # in place: activation copied by cp.async
    ("nchw", 6, 2048, 8, 8, 264, 1, 0, 256, 2),    # 1x1 as batched GEMM
    ("nhwc", 9, 136, 14, 14, 264, 3, 1, 256, 2),
    ("nhwc", 9, 136, 14, 14, 264, 3, 1, 128, 3),
    ("hwnc", 128, 72, 6, 6, 136, 3, 1, 128, 3),
    ("hwnc", 128, 72, 6, 6, 136, 3, 1, 64, 1),
    ("hwnc", 24, 72, 9, 10, 136, 3, 1, 128, 1),    # few images: pixels packed into a tile
    ("hwnc", 16, 136, 12, 14, 264, 3, 1, 256, 2),  # the same on CTA pairs
]


@pytest.mark.parametrize("cfg", CONVS)
def test_conv2d_every_layout(oracle, cfg):
    layout, n, c, h, w, k, r, pad, tile_n, cta_pair = cfg
    rng = np.random.default_rng(n + c)
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float16)
    f = rng.normal(0, 0.05, (k, c, r, r)).astype(np.float16)
    ref = oracle.c_conv2d_nchw(x, f, 1, pad, 1, "te_llvm")  # [N, K, P, Q]
    if layout == "nchw":
        d = _lib.conv2d_desc(n, c, h, w, k, r, r, 1, pad, 1, tile_n=tile_n, cta_pair=cta_pair)
        ins, shape = [_t(x), _t(f)], ref.shape
    elif layout == "nhwc":
        d = _lib.conv2d_nhwc_desc(n, h, w, c, k, r, r, 1, pad, 1, tile_n=tile_n, cta_pair=cta_pair)
        ins = [_t(x.transpose(0, 2, 3, 1)), _t(f.transpose(2, 3, 1, 0))]
        ref = ref.transpose(0, 2, 3, 1)
        shape = ref.shape
    else:
        d = _lib.conv2d_hwnc_desc(h, w, n, c, k, r, r, 1, pad, 1, tile_n=tile_n, cta_pair=cta_pair)
        ins = [_t(x.transpose(2, 3, 0, 1)), _t(f.transpose(2, 3, 1, 0))]
        ref = ref.transpose(2, 3, 0, 1)
        shape = ref.shape
    got = _run(d, ins, shape, True)
    assert oracle.rel_l2(got, ref) <= TOL_TE_LLVM
    assert oracle.rel_l2(got, _run(d, ins, shape, False)) <= TOL_REORDER


def test_without_scratch_the_tiles_stay_whole(oracle):
    """The optional scratch is optional: a call that brings none computes the same numbers."""
    m, n, k = 1100, 520, 1032
    rng = np.random.default_rng(6)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    d = _lib.gemm_desc(m, n, k, tile_n=256, cta_pair=1)
    ta, tb = _t(a), _t(b)
    out = torch.empty((m, n), dtype=torch.float32, device=DEV)
    lib = _lib.load()
    import ctypes
    ia, ka = device.tensor_arg(ta)
    ib, kb = device.tensor_arg(tb)
    io, ko = device.tensor_arg(out)
    ins = (_lib.AmosbTensor * 2)(ia, ib)
    outs = (_lib.AmosbTensor * 1)(io)
    with _env(AMOSB_TAIL_SHARING="1"):
        assert _lib.workspace_bytes(d) > 0 and _lib.workspace_bytes_min(d) == 0
        rc = lib.amosb_run(ctypes.byref(d), ins, 2, outs, 1, None, 0, None)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), _run(d, [ta, tb], (m, n), False))

"""GPU: the host-buffer entry point (amosb_run_host: numpy arrays in, numpy array out).  It cuts
the operator along its independent axis (rows of M, batches, images) and overlaps the copy-in of
one slice with the kernels of the previous one and the copy-out of the one before; the slices
must give exactly what the device-buffer entry point gives for the whole operator."""
import os

import numpy as np
import pytest
import torch

from amos_b200 import _lib, device, runtime

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def _device_result(desc, ins, out_shape):
    out = torch.empty(out_shape, dtype=device.CODE_TO_TORCH[desc.out_dtype], device=DEV)
    ws = device.get_workspace(_lib.workspace_bytes(desc), 0)
    device.run(desc, [_t(x) for x in ins], [out], workspace=ws)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def _host_result(desc, ins, out_shape, chunks):
    out = np.full(out_shape, 77, dtype=_lib.DTYPE_NAMES[desc.out_dtype])
    mod = runtime.Module(desc)
    old = os.environ.get("AMOSB_HOST_CHUNKS")
    os.environ["AMOSB_HOST_CHUNKS"] = str(chunks)
    try:
        mod(*ins, out)
    finally:
        if old is None:
            del os.environ["AMOSB_HOST_CHUNKS"]
        else:
            os.environ["AMOSB_HOST_CHUNKS"] = old
    assert device.status_peek(0) == 0
    return out, mod.launches_per_call


@pytest.mark.parametrize("chunks", [1, 3, 8])
def test_gemm_slices(chunks):
    rng = np.random.default_rng(chunks)
    a = rng.uniform(-1, 1, (1100, 264)).astype(np.float16)   # 5 row blocks of 256, the last ragged
    b = rng.uniform(-1, 1, (264, 392)).astype(np.float16)
    d = _lib.gemm_desc(1100, 392, 264)
    want = _device_result(d, [a, b], (1100, 392))
    got, launches = _host_result(d, [a, b], (1100, 392), chunks)
    assert np.array_equal(got, want)
    assert launches == {1: 1, 3: 3, 8: 5}[chunks]   # slices are whole 256-row blocks


def test_int8_and_batched_slices(oracle):
    rng = np.random.default_rng(4)
    a = rng.integers(-128, 128, (700, 256), dtype=np.int8)
    b = rng.integers(-128, 128, (256, 272), dtype=np.int8)
    d = _lib.gemm_desc(700, 272, 256, in_dtype=_lib.AMOSB_S8)
    got, _ = _host_result(d, [a, b], (700, 272), 2)
    assert np.array_equal(got, oracle.c_gemm(a, b, "exact"))
    # batched: both operands are cut per batch
    a3 = rng.uniform(-1, 1, (7, 136, 72)).astype(np.float16)
    b3 = rng.uniform(-1, 1, (7, 72, 200)).astype(np.float16)
    d3 = _lib.gemm_desc(136, 200, 72, batch=7, batched=True)
    want = _device_result(d3, [a3, b3], (7, 136, 200))
    got, launches = _host_result(d3, [a3, b3], (7, 136, 200), 4)
    assert np.array_equal(got, want) and launches == 4
    # A stored [K, M]: rows of M are not contiguous, the operator goes through whole
    at_ = np.ascontiguousarray(a3[0].T)
    dt = _lib.gemm_desc(136, 200, 72, trans_a=True)
    got, launches = _host_result(dt, [at_, b3[0]], (136, 200), 4)
    assert np.array_equal(got, want[0]) and launches == 1


@pytest.mark.parametrize("layout", ["nchw", "nhwc", "hwnc"])
def test_conv_slices(layout):
    rng = np.random.default_rng(6)
    n, c, h, w, k = 128 if layout == "hwnc" else 10, 64, 12, 12, 72
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float16)
    f = rng.normal(0, 0.05, (k, c, 3, 3)).astype(np.float16)
    if layout == "nchw":
        d, ins, shape = _lib.conv2d_desc(n, c, h, w, k, 3, 3, pad=1), [x, f], (n, k, h, w)
    elif layout == "nhwc":
        d = _lib.conv2d_nhwc_desc(n, h, w, c, k, 3, 3, pad=1)
        ins = [np.ascontiguousarray(x.transpose(0, 2, 3, 1)),
               np.ascontiguousarray(f.transpose(2, 3, 1, 0))]
        shape = (n, h, w, k)
    else:
        d = _lib.conv2d_hwnc_desc(h, w, n, c, k, 3, 3, pad=1)
        ins = [np.ascontiguousarray(x.transpose(2, 3, 0, 1)),
               np.ascontiguousarray(f.transpose(2, 3, 1, 0))]
        shape = (h, w, n, k)
    want = _device_result(d, ins, shape)
    got, launches = _host_result(d, ins, shape, 4)
    assert np.array_equal(got, want)
    per_slice = 2 if layout == "nchw" else 1          # NCHW: re-layout pass + main loop
    assert launches == (1 if layout == "hwnc" else 4) * per_slice


def test_full_shape_addend_is_cut_with_the_output_and_vectors_are_not():
    rng = np.random.default_rng(12)
    a = rng.uniform(-1, 1, (768, 64)).astype(np.float16)
    b = rng.uniform(-1, 1, (64, 136)).astype(np.float16)
    for flag, addend in ((_lib.EPI_ADD_FULL, rng.uniform(-1, 1, (768, 136)).astype(np.float32)),
                         (_lib.EPI_ADD_VECTOR, rng.uniform(-1, 1, (136,)).astype(np.float32))):
        d = _lib.gemm_desc(768, 136, 64)
        d.epilogue = flag | _lib.EPI_RELU
        d.addend_dtype, d.arg_c = _lib.AMOSB_F32, 2
        want = _device_result(d, [a, b, addend], (768, 136))
        got, launches = _host_result(d, [a, b, addend], (768, 136), 3)
        assert np.array_equal(got, want) and launches == 3


def test_slices_that_would_start_unaligned_fall_back_to_one():
    """Images of 3 x 5 x 5 float16 values are 150 bytes: a cut between images would hand the
    kernels an address that is not a multiple of 16 bytes, so the operator goes through whole."""
    rng = np.random.default_rng(2)
    x = rng.uniform(-1, 1, (6, 3, 5, 5)).astype(np.float16)
    f = rng.normal(0, 0.1, (8, 3, 3, 3)).astype(np.float16)
    d = _lib.conv2d_desc(6, 3, 5, 5, 8, 3, 3, pad=1)
    want = _device_result(d, [x, f], (6, 8, 5, 5))
    got, launches = _host_result(d, [x, f], (6, 8, 5, 5), 3)
    assert np.array_equal(got, want) and launches == 2


def test_pinned_and_pageable_host_memory_give_the_same_result():
    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, (2048, 512)).astype(np.float16)
    b = rng.uniform(-1, 1, (512, 1024)).astype(np.float16)
    d = _lib.gemm_desc(2048, 1024, 512, out_dtype=_lib.AMOSB_F16)
    want, _ = _host_result(d, [a, b], (2048, 1024), 4)
    pa, pb = torch.from_numpy(a).pin_memory(), torch.from_numpy(b).pin_memory()
    pc = torch.empty(2048, 1024, dtype=torch.float16).pin_memory()
    os.environ["AMOSB_HOST_CHUNKS"] = "4"
    try:
        runtime.Module(d)(pa.numpy(), pb.numpy(), pc.numpy())
    finally:
        del os.environ["AMOSB_HOST_CHUNKS"]
    assert np.array_equal(pc.numpy(), want)


def test_host_sharded_call_as_one_rank_and_as_two_on_one_gpu(tmp_path):
    """shard.HostShardedCall on pinned host operands: as a single rank (no exchange) and as the
    two ranks of a one-process group taken in turn on this one GPU with the exchange replaced by
    its result (each rank's slice of B copied into place by hand) -- the slicing, the buffer
    views and the copies are what is under test; the collective itself runs in the two-rank CPU
    test and in the multi-GPU benchmark."""
    from amos_b200 import shard
    rng = np.random.default_rng(12)
    m, n, k = 300, 520, 264
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    full = _lib.gemm_desc(m, n, k)
    want = _device_result(full, [a, b], (m, n))
    # one rank
    out = torch.zeros((m, n), dtype=torch.float32).pin_memory()
    call = shard.HostShardedCall(full, [torch.from_numpy(a).pin_memory(), torch.from_numpy(b).pin_memory()],
                                 out, 1, 0, DEV)
    assert call.gathered is None and call.h2d_bytes == a.nbytes + b.nbytes
    call.run()
    assert np.array_equal(out.numpy(), want)
    # two ranks, one after the other: B arrives as two byte slices
    got = np.zeros((m, n), np.float32)
    for rank in range(2):
        ld, ins, _ = shard.shard_arrays(full, [a, b], [], 2, rank)
        start, count = shard.partition(m, 2, rank)
        o = torch.zeros((count, n), dtype=torch.float32).pin_memory()

        class _NoExchange(shard.HostShardedCall):
            def run(self):  # what run() does, with the all-gather replaced by both slices copied in
                flat = self.flat_host
                self.gathered[:flat.numel()].copy_(flat, non_blocking=True)
                for i, (h, d) in enumerate(zip(self.host_inputs, self.dev_inputs)):
                    if i != self.rep:
                        d.copy_(h, non_blocking=True)
                self.call.run()
                self.host_output.copy_(self.dev_output, non_blocking=True)
                torch.cuda.current_stream().synchronize()

        c2 = _NoExchange(ld, [torch.from_numpy(np.ascontiguousarray(x)).pin_memory() for x in ins], o,
                         2, rank, DEV, min_gather_bytes=1024)
        assert c2.gathered is not None and c2.part_bytes * 2 >= b.nbytes
        assert c2.my_hi - c2.my_lo == min(c2.part_bytes, b.nbytes - rank * c2.part_bytes)
        c2.run()
        got[start:start + count] = o.numpy()
    assert np.array_equal(got, want)

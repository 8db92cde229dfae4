"""CPU: the sharding logic, single process and as two gloo ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from amos_b200 import _lib, shard


def test_partition_covers_everything_once():
    for total in (0, 1, 7, 96, 256, 4096):
        for world in (1, 2, 3, 4, 8):
            spans = [shard.partition(total, world, r) for r in range(world)]
            assert sum(c for _, c in spans) == total
            pos = 0
            for start, count in spans:
                assert start == pos and count >= 0
                pos += count
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        shard.partition(8, 2, 2)


def test_local_desc_and_views():
    d = _lib.gemm_desc(4096, 4096, 4096, out_dtype=_lib.AMOSB_F16)
    ld, start, count = shard.local_desc(d, 8, 3)
    assert (ld.m, ld.n, ld.k, start, count) == (512, 4096, 4096, 1536, 512)
    a = np.zeros((4096, 8), np.float16)
    b = np.zeros((8, 16), np.float16)
    c = np.zeros((4096, 16), np.float16)
    d2 = _lib.gemm_desc(4096, 16, 8)
    ld, ins, outs = shard.shard_arrays(d2, [a, b], [c], 4, 1)
    assert ins[0].shape == (1024, 8) and ins[1].shape == (8, 16) and outs[0].shape == (1024, 16)
    assert np.shares_memory(ins[0], a) and np.shares_memory(outs[0], c)
    bd = _lib.gemm_desc(512, 512, 64, batch=96)
    ld, start, count = shard.local_desc(bd, 8, 7)
    assert (ld.batch, start, count) == (12, 84, 12)
    cd = _lib.conv2d_desc(256, 128, 28, 28, 128, 3, 3, pad=1)
    ld, start, count = shard.local_desc(cd, 3, 0)
    assert (ld.conv_n, start, count) == (86, 0, 86)
    assert shard.local_desc(cd, 3, 2)[0].conv_n == 85
    # NHWC: images are still the outermost axis of activation and output
    hd = _lib.conv2d_nhwc_desc(10, 14, 14, 64, 32, 3, 3, pad=1)
    xh = np.zeros((10, 14, 14, 64), np.float16)
    fh = np.zeros((3, 3, 64, 32), np.float16)
    yh = np.zeros((10, 14, 14, 32), np.float32)
    ld, ins, outs = shard.shard_arrays(hd, [xh, fh], [yh], 4, 3)
    assert ld.kind == _lib.OP_CONV2D_NHWC and ld.conv_n == 2
    assert ins[0].shape == (2, 14, 14, 64) and ins[1].shape == (3, 3, 64, 32)
    assert outs[0].shape == (2, 14, 14, 32) and np.shares_memory(outs[0], yh)
    # HWNC: images are the third axis -- a rank's share is a strided slice, handed over compact
    wd = _lib.conv2d_hwnc_desc(14, 14, 256, 64, 32, 3, 3, pad=1)
    ld, start, count = shard.local_desc(wd, 1, 0)
    assert (ld.kind, ld.conv_n, start, count) == (_lib.OP_CONV2D_HWNC, 256, 0, 256)
    ld, start, count = shard.local_desc(wd, 2, 1)
    assert (ld.kind, ld.conv_n, start, count) == (_lib.OP_CONV2D_HWNC, 128, 128, 128)
    xw = np.arange(4 * 4 * 6 * 8, dtype=np.float16).reshape(4, 4, 6, 8)
    fw = np.zeros((3, 3, 8, 16), np.float16)
    yw = np.zeros((4, 4, 6, 16), np.float32)
    sd = _lib.conv2d_hwnc_desc(4, 4, 6, 8, 16, 3, 3, pad=1)
    ld, ins, outs = shard.shard_arrays(sd, [xw, fw], [yw], 3, 2)
    assert ld.conv_n == 2 and ins[0].shape == (4, 4, 2, 8) and ins[0].flags["C_CONTIGUOUS"]
    assert np.array_equal(ins[0], xw[:, :, 4:6]) and outs[0].shape == (4, 4, 2, 16)
    # fused addends: a vector over N stays whole, a tensor of the output's shape is cut with it
    gd = _lib.gemm_desc(64, 16, 8)
    gd.epilogue, gd.arg_c, gd.addend_dtype = _lib.EPI_ADD_VECTOR, 2, _lib.AMOSB_F32
    bias = np.zeros((16,), np.float32)
    ld, ins, _ = shard.shard_arrays(gd, [np.zeros((64, 8), np.float16), np.zeros((8, 16), np.float16),
                                         bias], [], 4, 1)
    assert ins[0].shape == (16, 8) and ins[1].shape == (8, 16) and ins[2].shape == (16,)
    gd.epilogue = _lib.EPI_ADD_FULL
    full = np.zeros((64, 16), np.float32)
    ld, ins, _ = shard.shard_arrays(gd, [np.zeros((64, 8), np.float16), np.zeros((8, 16), np.float16),
                                         full], [], 4, 1)
    assert ins[2].shape == (16, 16) and np.shares_memory(ins[2], full)
    bgd = _lib.gemm_desc(32, 16, 8, batch=6)
    bgd.epilogue, bgd.arg_c, bgd.addend_dtype = _lib.EPI_ADD_VECTOR, 2, _lib.AMOSB_F32
    ld, ins, _ = shard.shard_arrays(bgd, [np.zeros((6, 32, 8), np.float16),
                                          np.zeros((6, 8, 16), np.float16), bias], [], 3, 0)
    assert ins[0].shape == (2, 32, 8) and ins[1].shape == (2, 8, 16) and ins[2].shape == (16,)
    # more ranks than units
    small = _lib.conv2d_desc(1, 64, 56, 56, 64, 3, 3, pad=1)
    assert shard.local_desc(small, 2, 1)[2] == 0
    # operand order follows the descriptor
    swapped = _lib.gemm_desc(4096, 16, 8)
    swapped.arg_a, swapped.arg_b = 1, 0
    ld, ins, outs = shard.shard_arrays(swapped, [b, a], [c], 4, 2)
    assert ins[0].shape == (8, 16) and ins[1].shape == (1024, 8)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as o
        rng = np.random.default_rng(5)
        # uneven split: 37 rows over 2 ranks
        a = rng.uniform(-1, 1, (37, 24)).astype(np.float16)
        b = rng.uniform(-1, 1, (24, 16)).astype(np.float16)
        full = _lib.gemm_desc(37, 16, 24)
        out = np.zeros((37, 16), np.float32)
        ld, ins, outs = shard.shard_arrays(full, [a, b], [out], world, rank)
        # the CPU stand-in for the device call: each rank computes only its rows
        local = o.c_gemm(np.ascontiguousarray(ins[0]), ins[1], "te_llvm")
        assert local.shape == (ld.m, 16)
        gathered = shard.gather_output(torch.from_numpy(local), full)
        ref = o.c_gemm(a, b, "te_llvm")
        assert np.array_equal(gathered.numpy(), ref)
        # conv: 3 images over 2 ranks
        x = rng.uniform(-1, 1, (3, 4, 6, 6)).astype(np.float16)
        w = rng.normal(0, 0.05, (5, 4, 3, 3)).astype(np.float16)
        cd = _lib.conv2d_desc(3, 4, 6, 6, 5, 3, 3, pad=1)
        ld, ins, _ = shard.shard_arrays(cd, [x, w], [], world, rank)
        local = o.c_conv2d_nchw(np.ascontiguousarray(ins[0]), ins[1], 1, 1, 1, "te_llvm")
        gathered = shard.gather_output(torch.from_numpy(local), cd)
        assert np.array_equal(gathered.numpy(), o.c_conv2d_nchw(x, w, 1, 1, 1, "te_llvm"))
        # a GEMM with a bias vector and one with a full-shape addend, 37 rows over 2 ranks
        bias = rng.uniform(-1, 1, (16,)).astype(np.float32)
        resid = rng.uniform(-1, 1, (37, 16)).astype(np.float32)
        for bits, addend in ((_lib.EPI_ADD_VECTOR, bias), (_lib.EPI_ADD_FULL, resid)):
            fd = _lib.gemm_desc(37, 16, 24)
            fd.epilogue, fd.arg_c, fd.addend_dtype = bits | _lib.EPI_RELU, 2, _lib.AMOSB_F32
            ld, ins, _ = shard.shard_arrays(fd, [a, b, addend], [], world, rank)
            local = np.maximum(o.c_gemm(np.ascontiguousarray(ins[0]), ins[1], "te_llvm") + ins[2], 0)
            gathered = shard.gather_output(torch.from_numpy(local.astype(np.float32)), fd)
            assert np.array_equal(gathered.numpy(),
                                  np.maximum(ref + addend, 0).astype(np.float32))
        # HWNC: the image axis is the third one; the gather puts the shards back in place
        xw = rng.uniform(-1, 1, (5, 5, 3, 8)).astype(np.float16)
        ww = rng.normal(0, 0.05, (3, 3, 8, 8)).astype(np.float16)
        wd = _lib.conv2d_hwnc_desc(5, 5, 3, 8, 8, 3, 3, pad=1)
        ld, ins, _ = shard.shard_arrays(wd, [xw, ww], [], world, rank)
        local = o.c_conv2d_hwnc(ins[0], ins[1], 1, 1, 1, "te_llvm")
        gathered = shard.gather_output(torch.from_numpy(local), wd)
        assert np.array_equal(gathered.numpy(), o.c_conv2d_hwnc(xw, ww, 1, 1, 1, "te_llvm"))
        # operands in host memory: each rank copies its own rows of A and ONE slice of B, the
        # slices are all-gathered, the (stand-in) kernel sees the whole B and the rank's rows
        class _Fake:
            def __init__(self, desc, ins, outs):
                self.desc, self.ins, self.outs = desc, ins, outs

            def run(self):
                a_l, b_l = self.ins[0].numpy(), self.ins[1].numpy()
                self.outs[0].copy_(torch.from_numpy(o.c_gemm(np.ascontiguousarray(a_l), b_l, "te_llvm")))
                return 1

        a2 = rng.uniform(-1, 1, (37, 24)).astype(np.float16)
        b2 = rng.uniform(-1, 1, (24, 1000)).astype(np.float16)   # 48000 bytes: not a multiple of 2 x 16
        full2 = _lib.gemm_desc(37, 1000, 24)
        ld, ins, _ = shard.shard_arrays(full2, [a2, b2], [], world, rank)
        host_out = torch.zeros((ld.m, 1000), dtype=torch.float32)
        call = shard.HostShardedCall(ld, [torch.from_numpy(np.ascontiguousarray(x)) for x in ins],
                                     host_out, world, rank, "cpu", min_gather_bytes=1024,
                                     prepare=_Fake)
        assert call.gathered is not None and call.h2d_bytes < a2.nbytes + b2.nbytes
        for _ in range(2):
            call.run()
        gathered = shard.gather_output(host_out, full2)
        assert np.array_equal(gathered.numpy(), o.c_gemm(a2, b2, "te_llvm"))
        # a small replicated operand is copied whole, without the exchange
        small = shard.HostShardedCall(ld, [torch.from_numpy(np.ascontiguousarray(x)) for x in ins],
                                      host_out, world, rank, "cpu", prepare=_Fake)
        assert small.gathered is None
        small.run()
        assert np.array_equal(shard.gather_output(host_out, full2).numpy(), o.c_gemm(a2, b2, "te_llvm"))
        # max-over-ranks reduction used for timing
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == world
        open(os.path.join(tmpdir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks(oracle, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()

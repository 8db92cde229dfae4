"""Data-parallel sharding of one operator over the GPUs of one box: one process per GPU
(`torch.distributed`), independent work per rank, no collective on the compute path.

* GEMM / int8 GEMM: rows of A and C are split (B is replicated);
* batched GEMM: the batch is split;
* conv2d: the images (N) are split (the filter is replicated).  In the HWNC layout the images are
  the third axis of the activation and of the output: a rank's share is a strided slice, which is
  copied into a compact tensor once, outside any timed path (the library takes compact tensors only).

The reference has no multi-device path at all (its "remote" measurement is TVM RPC to a single
device, reference: python/tvm/auto_tensorize/search/measure.py:793-981); this module is the one
parallelism strategy added here.  An optional `gather_output` all-gathers the output shards over
NCCL (NVLink) -- or gloo on CPU, which is how the host logic is tested without GPUs.
"""
from __future__ import annotations

from typing import Sequence

from . import _lib


def partition(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous split of `total` units over `world` ranks: (start, count) of `rank`.  The first
    `total % world` ranks get one extra unit; ranks beyond `total` get (total, 0)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def shard_axis_extent(desc: _lib.AmosbOpDesc) -> int:
    """Number of independent units along the sharded axis of `desc`."""
    if desc.kind == _lib.OP_GEMM:
        return int(desc.m)
    if desc.kind == _lib.OP_BATCHED_GEMM:
        return int(desc.batch)
    if desc.kind in _lib.CONV_KINDS:
        return int(desc.conv_n)
    raise _lib.AmosbError(_lib.AMOSB_ERR_ARG, f"descriptor has no operator kind ({desc.kind})")


def local_desc(desc: _lib.AmosbOpDesc, world: int, rank: int) -> tuple[_lib.AmosbOpDesc, int, int]:
    """Descriptor of the part of `desc` that `rank` computes, with (start, count) along the sharded
    axis.  count may be 0 (more ranks than units): the caller then skips the launch."""
    start, count = partition(shard_axis_extent(desc), world, rank)
    d = desc.copy()
    if desc.kind == _lib.OP_GEMM:
        d.m = count
    elif desc.kind == _lib.OP_BATCHED_GEMM:
        d.batch = count
    else:
        d.conv_n = count
    return d, start, count


def shard_arrays(desc: _lib.AmosbOpDesc, inputs: Sequence, outputs: Sequence, world: int,
                 rank: int):
    """Views of full-size `inputs`/`outputs` (numpy arrays or torch tensors, in the callable's
    argument order) restricted to what `rank` reads and writes.  The operand that is not split
    along the sharded axis (B of a GEMM, the conv filter) is returned whole."""
    d, start, count = local_desc(desc, world, rank)
    ins = list(inputs)
    sl = slice(start, start + count)
    has_addend = bool(desc.epilogue & (_lib.EPI_ADD_VECTOR | _lib.EPI_ADD_FULL))
    if has_addend and desc.epilogue & _lib.EPI_ADD_FULL:
        # an addend of the output's shape is cut like the output; a vector over N stays whole
        ins[desc.arg_c] = ins[desc.arg_c][sl]
    if desc.kind == _lib.OP_BATCHED_GEMM:
        ins[desc.arg_a] = ins[desc.arg_a][sl]
        ins[desc.arg_b] = ins[desc.arg_b][sl]
    elif desc.kind == _lib.OP_GEMM and desc.trans_a:
        # A is stored [K, M]: a rank's rows of M are columns of it, which the library (compact
        # strides only) cannot take as a view -- the slice is copied once, outside any timed path
        ins[desc.arg_a] = _compact(ins[desc.arg_a][:, sl])
    elif desc.kind == _lib.OP_CONV2D_HWNC:
        ins[desc.arg_a] = _compact(ins[desc.arg_a][:, :, sl])
    else:
        ins[desc.arg_a] = ins[desc.arg_a][sl]
    if desc.kind == _lib.OP_CONV2D_HWNC:
        outs = [o[:, :, sl] for o in outputs]  # strided views: gather_output concatenates along N
    else:
        outs = [o[sl] for o in outputs]
    return d, ins, outs


def _compact(x):
    return x.contiguous() if hasattr(x, "contiguous") else \
        __import__("numpy").ascontiguousarray(x)


def gather_output(local_out, desc: _lib.AmosbOpDesc, group=None):
    """All-gather the output shards (a torch tensor per rank, possibly of unequal length along
    the sharded axis: axis 0, or the image axis 2 of an HWNC output) into the full output on every
    rank.  Outside the timed compute path."""
    import torch
    import torch.distributed as dist

    if desc.kind == _lib.OP_CONV2D_HWNC:
        moved = gather_output(local_out.permute(2, 0, 1, 3).contiguous(), _as_nhwc(desc), group)
        return moved.permute(1, 2, 0, 3).contiguous()
    world = dist.get_world_size(group)
    total = shard_axis_extent(desc)
    counts = [partition(total, world, r)[1] for r in range(world)]
    biggest = max(counts)
    tail = tuple(local_out.shape[1:])
    padded = torch.zeros((biggest,) + tail, dtype=local_out.dtype, device=local_out.device)
    padded[: local_out.shape[0]] = local_out
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:c] for p, c in zip(parts, counts)], dim=0)


def _as_nhwc(desc: _lib.AmosbOpDesc) -> _lib.AmosbOpDesc:
    d = desc.copy()
    d.kind = _lib.OP_CONV2D_NHWC
    return d

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

`HostShardedCall` is the same split for operands that start in HOST memory every call.  There the
replicated operand is the expensive part: eight ranks each copying all of B from their own host
buffer push eight copies of it through one host's memory and PCIe.  Instead each rank copies the
1/world slice of it that it is given over its own link and the ranks exchange the slices over
NVLink (one all-gather): every byte of the operand crosses the host bus once per call, as on one
GPU, and the all-gather is the one collective of the path.
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


def replicated_arg(desc: _lib.AmosbOpDesc):
    """Index of the input every rank needs whole (B of a GEMM, the filter of a convolution), or
    None (a batched GEMM splits both operands)."""
    return None if desc.kind == _lib.OP_BATCHED_GEMM else desc.arg_b


class HostShardedCall:
    """One rank's part of a sharded call whose operands and result live in pinned host memory.

    `host_inputs` are this rank's inputs as `shard_arrays` cuts them (its own rows / images, the
    replicated operand whole); `host_output` receives this rank's rows.  Each `run()`:
    copies the rank's own operand (and addend) to the GPU; copies ONE 1/world slice of the
    replicated operand and all-gathers the slices over the process group when that operand is
    large enough for it to matter (`min_gather_bytes`), else copies it whole; runs the kernels;
    copies the rank's rows of the result back and waits for them.  Everything is queued on the
    current stream, the copies from and to pinned memory asynchronously."""

    def __init__(self, desc: _lib.AmosbOpDesc, host_inputs: Sequence, host_output, world: int,
                 rank: int, device, group=None, min_gather_bytes: int = 1 << 20, prepare=None):
        """`prepare(desc, inputs, outputs)` returns the object whose `run()` launches the kernels
        on those device tensors (default: `device.PreparedCall`; tests without a GPU pass a
        stand-in and `device="cpu"`)."""
        import torch

        if prepare is None:
            from . import device as _device
            prepare = _device.PreparedCall
        self.world, self.rank, self.group = world, rank, group
        self.desc = desc  # already the rank's local descriptor
        self.host_inputs = list(host_inputs)
        self.host_output = host_output
        self.dev_inputs = [torch.empty(t.shape, dtype=t.dtype, device=device)
                           for t in self.host_inputs]
        self.dev_output = torch.empty(host_output.shape, dtype=host_output.dtype, device=device)
        self.rep = replicated_arg(desc)
        self.gathered = None
        if self.rep is not None and world > 1:
            full = self.host_inputs[self.rep]
            nbytes = full.numel() * full.element_size()
            if nbytes >= min_gather_bytes:
                # byte slices of equal length (the last one padded): what this rank copies in
                self.part_bytes = -(-nbytes // (world * 16)) * 16
                self.flat_host = full.reshape(-1).view(torch.uint8)
                self.gathered = torch.empty(self.part_bytes * world, dtype=torch.uint8,
                                            device=device)
                self.part = torch.zeros(self.part_bytes, dtype=torch.uint8, device=device)
                self.dev_inputs[self.rep] = self.gathered[:nbytes].view(full.dtype).view(full.shape)
                lo = min(rank * self.part_bytes, nbytes)
                hi = min(lo + self.part_bytes, nbytes)
                self.my_lo, self.my_hi = lo, hi
        self.call = prepare(desc, self.dev_inputs, [self.dev_output])
        self.launches_per_call = None
        self.h2d_bytes = sum(t.numel() * t.element_size() for i, t in enumerate(self.host_inputs)
                             if not (self.gathered is not None and i == self.rep))
        if self.gathered is not None:
            self.h2d_bytes += self.my_hi - self.my_lo
        self.d2h_bytes = host_output.numel() * host_output.element_size()

    def run(self) -> None:
        import torch
        import torch.distributed as dist
        # the slice of the replicated operand first, so that its exchange over NVLink runs while the
        # rank's own operand is still coming over PCIe
        pending = None
        if self.gathered is not None:
            n = self.my_hi - self.my_lo
            if n > 0:
                self.part[:n].copy_(self.flat_host[self.my_lo:self.my_hi], non_blocking=True)
            if dist.get_backend(self.group) == "nccl":
                pending = dist.all_gather_into_tensor(self.gathered, self.part, group=self.group,
                                                      async_op=True)
            else:
                dist.all_gather(list(self.gathered.chunk(self.world)), self.part, group=self.group)
        for i, (h, d) in enumerate(zip(self.host_inputs, self.dev_inputs)):
            if self.gathered is not None and i == self.rep:
                continue
            d.copy_(h, non_blocking=True)
        if pending is not None:
            pending.wait()  # the current stream waits for the exchange; the host does not
        self.launches_per_call = self.call.run()
        self.host_output.copy_(self.dev_output, non_blocking=True)
        if self.dev_output.is_cuda:
            torch.cuda.current_stream(self.dev_output.device).synchronize()

#!/usr/bin/env python
"""Benchmark of the tensor-core mapped operators on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One JSON line on stdout (rank 0).  A "step" is one pass of the operator over one set of seeded
synthetic operands.  Headline workload: the fp16 GEMM M=N=K=4096 with fp32 accumulation and fp16
output; the other configurations are measured briefly and reported under "configs".

N > 1: launched by torchrun, one rank per GPU.  By default the NAMED configuration is split across
the ranks -- rows of M (GEMM), batches (batched GEMM), images (conv); B / the filter replicated; no
collective on the timed path ("scaling": "strong") -- `value` = work of all ranks divided by the
slowest rank's device time; every rank checks its output shard against the same rows of an
unsharded run on its own GPU ("shard_parity"), and the optional NCCL all-gather of the output is
timed separately ("gather").  `--scaling weak` gives every rank the named configuration instead;
under the default that figure is reported as the extra "weak_scaling".
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL_INT8_OVER_F16 = 2.0  # dense int8 tensor rate is twice the fp16 rate on this part
NOMINAL_TF32_OVER_F16 = 0.5  # dense tf32 tensor rate is half the fp16 rate


# --------------------------------------------------------------------------------------------
# Workloads (shapes, value distributions and seeds of the named configurations)
# --------------------------------------------------------------------------------------------
def _conv(n, c, h, w, k, r, s, stride, pad, layout="nchw"):
    return dict(kind="conv", n=n, c=c, h=h, w=w, k=k, r=r, s=s, stride=stride, pad=pad, dil=1,
                layout=layout)


WORKLOADS = {
    "conv_c1_n1_c64_56x56_k64_3x3": dict(_conv(1, 64, 56, 56, 64, 3, 3, 1, 1), seed=20260000,
                                          wdist="uniform", shard=False),
    "gemm_f16_4096": dict(kind="gemm", m=4096, n=4096, k=4096, dtype="f16", out="float16",
                          seed=20260001, dist="uniform", shard=True),
    "conv_c3a_n256_c64_56x56_k256_1x1": dict(_conv(256, 64, 56, 56, 256, 1, 1, 1, 0),
                                              seed=20260002, wdist="normal", shard=True),
    "conv_c3b_n256_c128_28x28_k128_3x3": dict(_conv(256, 128, 28, 28, 128, 3, 3, 1, 1),
                                               seed=20260002, wdist="normal", shard=True),
    "conv_c3c_n256_c256_14x14_k256_3x3": dict(_conv(256, 256, 14, 14, 256, 3, 3, 1, 1),
                                               seed=20260002, wdist="normal", shard=True),
    "conv_c3d_n256_c1024_14x14_k256_1x1": dict(_conv(256, 1024, 14, 14, 256, 1, 1, 1, 0),
                                                seed=20260002, wdist="normal", shard=True),
    "conv_c3e_n256_c512_7x7_k512_3x3": dict(_conv(256, 512, 7, 7, 512, 3, 3, 1, 1),
                                             seed=20260002, wdist="normal", shard=True),
    "gemm_s8_8192": dict(kind="gemm", m=8192, n=8192, k=8192, dtype="s8", out="int32",
                         seed=20260003, dist="int", shard=True),
    "bgemm_f16_96x512x512x64": dict(kind="bgemm", batch=96, m=512, n=512, k=64, dtype="f16",
                                    out="float16", seed=20260004, dist="normal", shard=True),
    "bgemm_f16_96x512x64x512": dict(kind="bgemm", batch=96, m=512, n=64, k=512, dtype="f16",
                                    out="float16", seed=20260005, dist="normal", shard=True),
    # the same batch-256 layers in the reference's NHWC / RSCK layout
    # (benchmark/amos/mapping_conv2d_tensorcore.py:43-72): operands consumed in place, one kernel
    "conv_nhwc_c3b_n256_28x28_c128_k128_3x3": dict(
        _conv(256, 128, 28, 28, 128, 3, 3, 1, 1, "nhwc"), seed=20260002, wdist="normal", shard=True),
    "conv_nhwc_c3c_n256_14x14_c256_k256_3x3": dict(
        _conv(256, 256, 14, 14, 256, 3, 3, 1, 1, "nhwc"), seed=20260002, wdist="normal", shard=True),
    "conv_nhwc_c3d_n256_14x14_c1024_k256_1x1": dict(
        _conv(256, 1024, 14, 14, 256, 1, 1, 1, 0, "nhwc"), seed=20260002, wdist="normal",
        shard=True),
    "conv_nhwc_c3e_n256_7x7_c512_k512_3x3": dict(
        _conv(256, 512, 7, 7, 512, 3, 3, 1, 1, "nhwc"), seed=20260002, wdist="normal", shard=True),
    # float32 operands on the tf32 path (the reference's wmma_tf32_fp32 family), the headline shape
    "gemm_tf32_4096": dict(kind="gemm", m=4096, n=4096, k=4096, dtype="f32", out="float32",
                           seed=20260001, dist="uniform", shard=True),
    # ... and in its HWNC / RSCK layout (same file, :74-104); images are not the outermost axis, so
    # these run on one GPU only
    "conv_hwnc_c3b_28x28_n256_c128_k128_3x3": dict(
        _conv(256, 128, 28, 28, 128, 3, 3, 1, 1, "hwnc"), seed=20260002, wdist="normal", shard=True),
    "conv_hwnc_c3c_14x14_n256_c256_k256_3x3": dict(
        _conv(256, 256, 14, 14, 256, 3, 3, 1, 1, "hwnc"), seed=20260002, wdist="normal", shard=True),
}
HEADLINE = "gemm_f16_4096"


def make_desc(w):
    from amos_b200 import _lib
    if w["kind"] == "conv" and w.get("layout") == "hwnc":
        return _lib.conv2d_hwnc_desc(w["h"], w["w"], w["n"], w["c"], w["k"], w["r"], w["s"],
                                     w["stride"], w["pad"], w["dil"], out_dtype=_lib.AMOSB_F32)
    if w["kind"] == "conv" and w.get("layout") == "nhwc":
        return _lib.conv2d_nhwc_desc(w["n"], w["h"], w["w"], w["c"], w["k"], w["r"], w["s"],
                                     w["stride"], w["pad"], w["dil"], out_dtype=_lib.AMOSB_F32)
    if w["kind"] == "conv":
        return _lib.conv2d_desc(w["n"], w["c"], w["h"], w["w"], w["k"], w["r"], w["s"], w["stride"],
                                w["pad"], w["dil"], out_dtype=_lib.AMOSB_F32)
    in_dtype = {"s8": _lib.AMOSB_S8, "f32": _lib.AMOSB_F32}.get(w["dtype"], _lib.AMOSB_F16)
    return _lib.gemm_desc(w["m"], w["n"], w["k"], in_dtype=in_dtype,
                          out_dtype=_lib.DTYPE_CODES[w["out"]], batch=w.get("batch", 1),
                          batched=w["kind"] == "bgemm")


def make_inputs(w, variant=0):
    """Seeded host operands (numpy), identical for every GPU count."""
    rng = np.random.default_rng(w["seed"] + 7919 * variant)
    if w["kind"] == "conv":
        a = rng.uniform(-1, 1, (w["n"], w["c"], w["h"], w["w"])).astype(np.float16)
        if w["wdist"] == "normal":
            f = rng.normal(0, 0.05, (w["k"], w["c"], w["r"], w["s"])).astype(np.float16)
        else:
            f = rng.uniform(-1, 1, (w["k"], w["c"], w["r"], w["s"])).astype(np.float16)
        if w.get("layout") == "hwnc":  # the same values, laid out [H,W,N,C] and [R,S,C,K]
            return [np.ascontiguousarray(a.transpose(2, 3, 0, 1)),
                    np.ascontiguousarray(f.transpose(2, 3, 1, 0))]
        if w.get("layout") == "nhwc":  # the same values, laid out [N,H,W,C] and [R,S,C,K]
            return [np.ascontiguousarray(a.transpose(0, 2, 3, 1)),
                    np.ascontiguousarray(f.transpose(2, 3, 1, 0))]
        return [a, f]
    lead = (w["batch"],) if w["kind"] == "bgemm" else ()
    sa, sb = lead + (w["m"], w["k"]), lead + (w["k"], w["n"])
    if w["dist"] == "int":
        return [rng.integers(-128, 128, sa, dtype=np.int8), rng.integers(-128, 128, sb, dtype=np.int8)]
    if w["dist"] == "normal":
        return [rng.normal(0, 1, sa).astype(np.float16), rng.normal(0, 1, sb).astype(np.float16)]
    fdt = np.float32 if w["dtype"] == "f32" else np.float16
    return [rng.uniform(-1, 1, sa).astype(fdt), rng.uniform(-1, 1, sb).astype(fdt)]


def out_shape(desc):
    from amos_b200 import _lib
    if desc.kind == _lib.OP_CONV2D_NCHW:
        return (desc.conv_n, desc.conv_k, desc.conv_p, desc.conv_q)
    if desc.kind == _lib.OP_CONV2D_NHWC:
        return (desc.conv_n, desc.conv_p, desc.conv_q, desc.conv_k)
    if desc.kind == _lib.OP_CONV2D_HWNC:
        return (desc.conv_p, desc.conv_q, desc.conv_n, desc.conv_k)
    if desc.kind == _lib.OP_BATCHED_GEMM:
        return (desc.batch, desc.m, desc.n)
    return (desc.m, desc.n)


def work_and_bytes(desc):
    """(operations, algorithmic bytes): every input read once, the output written once."""
    from amos_b200 import _lib
    eb = _lib.DTYPE_BYTES
    if desc.kind in _lib.CONV_KINDS:
        ops = 2.0 * desc.conv_n * desc.conv_k * desc.conv_p * desc.conv_q * desc.conv_c \
            * desc.conv_r * desc.conv_s
        byt = (desc.conv_n * desc.conv_c * desc.conv_h * desc.conv_w
               + desc.conv_k * desc.conv_c * desc.conv_r * desc.conv_s) * eb[desc.in_dtype] \
            + desc.conv_n * desc.conv_k * desc.conv_p * desc.conv_q * eb[desc.out_dtype]
        return ops, float(byt)
    ops = 2.0 * desc.batch * desc.m * desc.n * desc.k
    byt = desc.batch * (desc.m * desc.k + desc.k * desc.n) * eb[desc.in_dtype] \
        + desc.batch * desc.m * desc.n * eb[desc.out_dtype]
    return ops, float(byt)


def ncu_traffic(name):
    """DRAM bytes (read + write) per launch of the workload's kernels, from the ncu captures that
    profiles/ncu_traffic.json records; (None, reason) where no capture exists."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            table = json.load(f)["workloads"]
    except (OSError, ValueError, KeyError):
        return None, "profiles/ncu_traffic.json is missing"
    rec = table.get(name)
    if rec is None:
        return None, "no entry for this workload"
    if rec.get("dram_bytes") is None:
        return None, rec.get("reason", "not captured")
    return float(rec["dram_bytes"]), rec.get("source")


def measure_int8_library_peak(dev, seconds=1.0):
    """int8 tensor-core peak of this GPU as the vendor library reaches it: torch._int_mm (cuBLASLt)
    on 8192^3, best single call (burst) and a back-to-back loop of `seconds` (sustained)."""
    import torch
    n = 8192
    tdev = f"cuda:{dev}"
    a = torch.randint(-128, 128, (n, n), dtype=torch.int8, device=tdev)
    b = torch.randint(-128, 128, (n, n), dtype=torch.int8, device=tdev)
    ops = 2.0 * n ** 3
    best = None
    for rhs, label in ((b, "B row-major"), (b.t().contiguous().t(), "B column-major")):
        try:
            for _ in range(3):
                torch._int_mm(a, rhs)
            torch.cuda.synchronize(dev)
            burst = float("inf")
            for _ in range(10):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                torch._int_mm(a, rhs)
                e1.record()
                e1.synchronize()
                burst = min(burst, e0.elapsed_time(e1))
            reps = max(10, int(seconds * 1e3 / burst))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                torch._int_mm(a, rhs)
            e1.record()
            e1.synchronize()
            sustained = e0.elapsed_time(e1) / reps
        except Exception as exc:  # the library refused this layout
            sys.stderr.write(f"torch._int_mm ({label}) failed: {exc}\n")
            continue
        rec = {"int8_tops": ops / burst / 1e9, "int8_tops_sustained": ops / sustained / 1e9,
               "how": f"torch._int_mm (cuBLASLt) 8192^3, {label}: best of 10 (burst) and {reps} "
                      f"calls back to back (sustained), CUDA events, measured in this run"}
        if best is None or rec["int8_tops"] > best["int8_tops"]:
            best = rec
    del a, b
    torch.cuda.empty_cache()
    return best


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# --------------------------------------------------------------------------------------------
# Clock sampling during the timed region
# --------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap",
               0x8: "hw_slowdown", 0x10: "sync_boost", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
               0x100: "display_clock_setting"}

    def __init__(self, index):
        self.samples, self.mask, self.max_mhz = [], 0, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = None
            try:  # NVML numbering ignores CUDA_VISIBLE_DEVICES: find the device by UUID
                import torch
                uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self._h = None
            if self._h is None:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _once(self):
        nv = self._nv
        try:
            self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
            self.mask |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
        except Exception:
            try:
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
            except Exception:
                pass

    def _loop(self):
        while not self._stop.is_set():
            self._once()
            time.sleep(0.01)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
            self._once()

    def summary(self):
        reasons = [n for bit, n in self.REASONS.items() if self.mask & bit and n != "gpu_idle"]
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(self.samples)}


# --------------------------------------------------------------------------------------------
# Our arm
# --------------------------------------------------------------------------------------------
def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def _barrier(world, dev):
    import torch
    torch.cuda.synchronize(dev)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        torch.cuda.synchronize(dev)


def measure_workload(name, steps, warmup, world, rank, dev, sampler=None, e2e_steps=0,
                     use_graph=True, scaling="strong", min_region_s=0.0, check_shard=False,
                     time_gather=False):
    """Device-resident timing (and optionally the host-buffer end-to-end timing) of one workload
    on this rank's shard.  Returns a dict of per-rank figures; the caller reduces over ranks.

    The K steps are captured once into a CUDA graph.  One replay is the short ("burst") region;
    with `min_region_s` the graph is then replayed until the timed region lasts at least that long
    (the "sustained" region: power-capped clocks, the reference's min_repeat_ms = 500 discipline,
    reference benchmark/amos/mapping_gemm_tensorcore.py:38)."""
    import torch
    from amos_b200 import _lib, device, runtime, shard

    w = WORKLOADS[name]
    if world > 1 and not w["shard"]:
        return None
    weak = scaling == "weak" and world > 1
    if weak:
        # the job is `world` times the named configuration along its independent axis (rows of M,
        # batches, images); every rank's share is exactly the named configuration
        axis = {"gemm": "m", "bgemm": "batch", "conv": "n"}[w["kind"]]
        full = make_desc(dict(w, **{axis: w[axis] * world}))
    else:
        full = make_desc(w)
    desc, start, count = shard.local_desc(full, world, rank)
    ops_local, bytes_local = work_and_bytes(desc) if count > 0 else (0.0, 0.0)
    res = {"ops_local": ops_local, "bytes_local": bytes_local, "ms": 0.0, "burst_ms": 0.0,
           "passes": 1, "launches": 0, "e2e_ms": None, "h2d": 0, "d2h": 0, "shard_ok": 1.0,
           "shard_bit_exact": 1.0, "shard_rel_l2": 0.0, "gather_ms": 0.0}
    if count == 0:
        raise SystemExit(f"{name}: more ranks ({world}) than rows / batches / images to split")
    torch.cuda.nvtx.range_push(f"bench:{name}:setup")
    tdev = f"cuda:{dev}"
    host = make_inputs(w)
    if weak:
        # the rank's own rows / batches / images (seeded by rank); B and the filter are replicated
        own = make_inputs(w, variant=rank) if rank else host
        host_local = list(own) if w["kind"] == "bgemm" else [own[0], host[1]]
    else:
        _, host_local, _ = shard.shard_arrays(full, host, [], world, rank)
    set_bytes = bytes_local
    nsets = max(2, int(math.ceil(1.5 * L2_BYTES / max(set_bytes, 1.0))) + 1)
    nsets = min(nsets, 64)
    out_dtype = device.CODE_TO_TORCH[desc.out_dtype]
    sets = []
    for v in range(nsets):
        if v == 0:
            ins = [torch.from_numpy(np.ascontiguousarray(x)).to(tdev) for x in host_local]
        else:
            # further sets: the same values rolled along the reduction-free axis (cheap, distinct
            # addresses); set 0 is the one whose result is checked
            ins = [torch.roll(t, shifts=v, dims=0).contiguous() for t in sets[0][0]]
        out = torch.empty(out_shape(desc), dtype=out_dtype, device=tdev)
        sets.append((ins, [out]))
    ws = device.get_workspace(_lib.workspace_bytes(desc), dev)
    stream = torch.cuda.current_stream(dev)
    calls = [device.PreparedCall(desc, ins, outs, stream, ws) for ins, outs in sets]
    torch.cuda.nvtx.range_pop()
    for i in range(max(warmup, 3)):
        res["launches_per_step"] = calls[i % nsets].run()
    _barrier(world, dev)
    graph = None
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                cap = torch.cuda.current_stream(dev)
                for i in range(steps):
                    calls[i % nsets].run(cap)
            graph.replay()  # one untimed replay: uploads the graph
        except Exception as exc:  # pragma: no cover - depends on the driver
            sys.stderr.write(f"graph capture failed ({exc}); timing plain launches\n")
            graph = None
        _barrier(world, dev)

    def one_pass():
        if graph is not None:
            graph.replay()
        else:
            for i in range(steps):
                calls[i % nsets].run()

    def timed(passes, ctx):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        with ctx:
            e0.record(stream)
            for _ in range(passes):
                one_pass()
            e1.record(stream)
            torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1)

    torch.cuda.nvtx.range_push(f"bench:{name}:timed")
    res["burst_ms"] = timed(1, _Null())
    passes = 1
    if min_region_s > 0:
        passes = int(min(50000, max(1, math.ceil(min_region_s * 1e3 / max(res["burst_ms"], 1e-3)))))
        if world > 1:  # every rank must replay the same number of times
            import torch.distributed as dist
            t = torch.tensor([passes], dtype=torch.int64, device=tdev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            passes = int(t.item())
        _barrier(world, dev)
        res["ms"] = timed(passes, sampler if sampler is not None else _Null())
    else:
        res["ms"] = res["burst_ms"]
    torch.cuda.nvtx.range_pop()
    res["passes"] = passes
    res["launch"] = "cuda_graph" if graph is not None else "stream"
    res["launches"] = passes * steps * res["launches_per_step"]
    res["nsets"] = nsets
    device.sync_check(dev)  # raises if a kernel gave up a bounded wait: the numbers would be void
    local_out = sets[0][1][0]

    if check_shard and world > 1 and not weak:
        # The rank runs the unsharded operator once on its own GPU (same seed, hence the same
        # operands) and compares its shard with the same rows / batches / images: no collective.
        full_ins = [torch.from_numpy(np.ascontiguousarray(x)).to(tdev) for x in host]
        full_out = torch.empty(out_shape(full), dtype=out_dtype, device=tdev)
        device.PreparedCall(full, full_ins, [full_out], stream,
                            device.get_workspace(_lib.workspace_bytes(full), dev)).run()
        calls[0].run()  # the shard again, after the workspace may have been replaced
        torch.cuda.synchronize(dev)
        if full.kind == _lib.OP_CONV2D_HWNC:  # images are the third axis of [P, Q, N, K]
            want = full_out[:, :, start:start + count]
        else:
            want = full_out[start:start + count]
        exact = bool(torch.equal(local_out, want))
        rel = 0.0
        if not exact:
            diff = (local_out.double() - want.double()).norm()
            rel = float(diff / want.double().norm().clamp_min(1e-300))
        integer = desc.out_dtype == _lib.AMOSB_S32
        res["shard_bit_exact"] = 1.0 if exact else 0.0
        res["shard_rel_l2"] = rel
        # integers must match bit for bit; floats may differ by the order of the fp32 additions
        # when the shard picks a tile family that splits the reduction
        res["shard_ok"] = 1.0 if (exact or (not integer and rel <= 1e-5)) else 0.0
        del full_ins, full_out

    if time_gather and world > 1 and not weak:
        shard.gather_output(local_out, full)  # warm-up: communicator set-up, allocations
        _barrier(world, dev)
        g0 = torch.cuda.Event(enable_timing=True)
        g1 = torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        gathered = shard.gather_output(local_out, full)
        g1.record(stream)
        torch.cuda.synchronize(dev)
        res["gather_ms"] = g0.elapsed_time(g1)
        res["gather_bytes"] = int(gathered.numel() * gathered.element_size())
        del gathered

    if e2e_steps > 0:
        torch.cuda.nvtx.range_push(f"bench:{name}:e2e")
        pin_in = [torch.from_numpy(np.ascontiguousarray(x)).pin_memory() for x in host_local]
        pin_out = torch.empty(out_shape(desc), dtype=out_dtype).pin_memory()
        hs = None
        if world > 1 and not weak and os.environ.get("AMOSB_BENCH_E2E_NO_EXCHANGE") is None:
            # several ranks, one host: each rank copies in its own rows and ONE slice of the operand
            # every rank needs whole; the slices are exchanged over NVLink (shard.HostShardedCall)
            try:
                hs = shard.HostShardedCall(desc, pin_in, pin_out, world, rank, tdev)
                hs.run()
            except Exception as exc:  # pragma: no cover - depends on the collective library
                sys.stderr.write(f"host-sharded call unavailable ({exc}); every rank copies the "
                                 f"replicated operand whole\n")
                hs = None
        if hs is not None:
            step = hs.run
            res["e2e_via"] = "shard.HostShardedCall"
        else:
            mod = runtime.Module(desc)
            np_args = [t.numpy() for t in pin_in] + [pin_out.numpy()]

            def step():
                mod(*np_args)  # H2D of both operands, kernels, D2H of the result, synchronises
            res["e2e_via"] = "Module(*numpy) -> amosb_run_host"
        for _ in range(2):
            step()
        # what came back is what the device-resident run of the same shard produced
        res["e2e_ok"] = 1.0 if torch.equal(pin_out, sets[0][1][0].cpu()) else 0.0
        _barrier(world, dev)
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(e2e_steps):
            step()
        t1.record()
        torch.cuda.synchronize(dev)
        res["e2e_ms"] = t0.elapsed_time(t1)
        res["e2e_steps"] = e2e_steps
        if hs is not None:
            res["h2d"], res["d2h"] = int(hs.h2d_bytes), int(hs.d2h_bytes)
            res["e2e_launches"] = e2e_steps * int(hs.launches_per_call or 0)
        else:
            res["h2d"] = int(sum(t.numel() * t.element_size() for t in pin_in))
            res["d2h"] = int(pin_out.numel() * pin_out.element_size())
            res["e2e_launches"] = e2e_steps * mod.launches_per_call
        torch.cuda.nvtx.range_pop()
    del sets, calls
    torch.cuda.empty_cache()
    return res


def bind_to_gpu_cpus(dev):
    """Restrict this rank to the host cores next to its GPU (the PCI device's `local_cpulist`), so
    that the pinned host buffers it allocates afterwards land in that socket's memory and its
    copies do not cross the socket link.  Returns the cpu list used, or None if the topology
    cannot be read (then nothing changes)."""
    import torch
    try:
        pr = torch.cuda.get_device_properties(dev)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/local_cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return text
    except Exception:  # no sysfs entry, no such attribute, not permitted: leave the affinity alone
        return None


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def reduce_over_ranks(res, world, dev):
    """max of the times, sum of the work, min of the parity flags, over ranks; plus every rank's
    own end-to-end time (the ranks share the host's bus, so the aggregate alone hides who waits)."""
    keys_max = ["ms", "burst_ms", "gather_ms", "shard_rel_l2"]
    keys_sum = ["ops_local", "bytes_local", "launches", "h2d", "d2h"]
    keys_min = ["shard_ok", "shard_bit_exact", "e2e_ok"]
    out = {k: float(res.get(k) or 0.0) for k in keys_max + keys_sum + keys_min}
    out["e2e_via"] = res.get("e2e_via")
    out["e2e_ms"] = res["e2e_ms"]
    out["e2e_ms_per_rank"] = [res["e2e_ms"]] if res["e2e_ms"] else None
    if world == 1:
        return out
    import torch
    import torch.distributed as dist
    tdev = f"cuda:{dev}"
    t = torch.tensor([out[k] for k in keys_max] + [res["e2e_ms"] or 0.0], dtype=torch.float64,
                     device=tdev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    for i, k in enumerate(keys_max):
        out[k] = float(t[i])
    out["e2e_ms"] = float(t[-1]) or None
    u = torch.tensor([out[k] for k in keys_sum], dtype=torch.float64, device=tdev)
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    for i, k in enumerate(keys_sum):
        out[k] = float(u[i])
    v = torch.tensor([out[k] for k in keys_min], dtype=torch.float64, device=tdev)
    dist.all_reduce(v, op=dist.ReduceOp.MIN)
    for i, k in enumerate(keys_min):
        out[k] = float(v[i])
    mine = torch.tensor([res["e2e_ms"] or 0.0], dtype=torch.float64, device=tdev)
    every = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    out["e2e_ms_per_rank"] = [float(x) for x in every] if out["e2e_ms"] else None
    return out


def roofline_for(desc_full, ops, byts, ms_per_step, n_gpus, peaks, peaks_kind, long_region,
                 int8_peak=None):
    """Roofline record of one timing.  Denominators: the measured bf16 tensor rate (fp16 runs at the
    same rate; tf32 at half of it, stated), the int8 rate measured in this run with the vendor
    library when available (else twice the bf16 rate, stated), the measured copy bandwidth; the
    burst figures for short regions, the sustained ones for regions of half a second and more."""
    from amos_b200 import _lib
    i8 = desc_full.in_dtype == _lib.AMOSB_S8
    tf32 = desc_full.in_dtype == _lib.AMOSB_F32
    tc_key = "bf16_tflops_sustained" if long_region else "bf16_tflops"
    if i8 and int8_peak:
        per_gpu = int8_peak["int8_tops_sustained" if long_region else "int8_tops"]
        note = ("int8_tops_sustained" if long_region else "int8_tops") + \
            " of measured (torch._int_mm 8192^3 in this run)"
    else:
        per_gpu = peaks[tc_key] * (NOMINAL_INT8_OVER_F16 if i8 else NOMINAL_TF32_OVER_F16 if tf32
                                   else 1.0)
        note = (f"{tc_key} of {peaks_kind}" + (" x2 (int8 rate assumed twice the measured bf16 "
                                               "rate)" if i8 else "") +
                (" x0.5 (tf32 rate assumed half the measured bf16 rate)" if tf32 else ""))
    tc_peak = per_gpu * n_gpus
    hbm_peak = peaks["hbm_gbs"] * n_gpus
    ai = ops / byts
    ridge = tc_peak * 1e12 / (hbm_peak * 1e9)
    sec = ms_per_step / 1e3
    if ai >= ridge:
        achieved = ops / sec / 1e12
        return {"bound": "tensor", "achieved": achieved, "peak": tc_peak,
                "unit": "TOP/s" if i8 else "TFLOP/s", "frac": achieved / tc_peak,
                "traffic": None, "peak_source": note}
    achieved = byts / sec / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
            "frac": achieved / hbm_peak, "traffic": None,
            "peak_source": f"hbm_gbs of {peaks_kind}"}


def same_size_copy_us(total_bytes, dev, reps=20):
    """Time of a plain device-to-device copy that moves `total_bytes` (half read, half written), on
    four buffer pairs in rotation so that L2 serves nothing: what this box's memory system gives a
    kernel of that size.  Small transfers stay far below the large-copy rate that is the roofline
    denominator (a 64 MB copy runs at about half of it), so HBM-bound configurations carry this
    figure beside their fraction.  None if the buffers would not be small beside the GPU's memory."""
    import torch
    half = int(total_bytes // 2) // 16 * 16
    if half <= 0 or half * 8 > (8 << 30):
        return None
    src = [torch.empty(half, dtype=torch.uint8, device=dev) for _ in range(4)]
    dst = [torch.empty(half, dtype=torch.uint8, device=dev) for _ in range(4)]
    for i in range(4):
        dst[i].copy_(src[i])
    torch.cuda.synchronize(dev)
    beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    beg.record()
    for i in range(reps):
        dst[i % 4].copy_(src[i % 4])
    end.record()
    end.synchronize()
    return beg.elapsed_time(end) / reps * 1e3


def config_for(name, world, scaling):
    """The `config` object of the JSON line; both arms print the same one."""
    w = WORKLOADS[name]
    if world == 1:
        sharding = "none"
    elif scaling == "weak":
        sharding = (f"{world} x the named configuration along rows of M / batch / images, one "
                    f"named configuration per rank, no collective")
    else:
        sharding = (f"rows of M / batch / images of the named configuration split over {world} "
                    f"ranks, B / filter replicated, no collective")
    return {"workload": name, "shape": {k: v for k, v in w.items() if k not in ("seed", "shard")},
            "sharding": sharding}


def cpu_baseline(name, budget_s=12.0, threads=1, order=0):
    """Time the CPU restatement of the reference's llvm build (oracle, te_llvm arithmetic, the
    default schedule's loop nest) on a bounded slice of the workload."""
    from oracle import oracle as o
    w = WORKLOADS[name]
    host = make_inputs(w)
    if w["kind"] == "conv":
        a, f = host
        d = make_desc(w)
        per_img = 2.0 * w["k"] * w["c"] * w["r"] * w["s"] * d.conv_p * d.conv_q
        probe_n = 1

        def run(nimg):
            t = time.perf_counter()
            if w.get("layout") == "hwnc":
                o.c_conv2d_hwnc(a[:, :, :nimg], f, w["stride"], w["pad"], w["dil"], "te_llvm",
                                threads=threads)
            elif w.get("layout") == "nhwc":
                o.c_conv2d_nhwc(a[:nimg], f, w["stride"], w["pad"], w["dil"], "te_llvm",
                                threads=threads)
            else:
                o.c_conv2d_nchw(a[:nimg], f, w["stride"], w["pad"], w["dil"], "te_llvm",
                                order=order, threads=threads)
            return time.perf_counter() - t
        t1 = run(probe_n)
        nimg = int(max(1, min(w["n"], budget_s / max(t1, 1e-6))))
        t = run(nimg) if nimg > 1 else t1
        ops = per_img * nimg
        whole = nimg == w["n"]
        sample = f"{nimg} of {w['n']} images"
    else:
        a, b = host
        lead = w.get("batch", 1)
        a2 = a.reshape(-1, a.shape[-1]) if w["kind"] == "gemm" else a
        rows_total = w["m"] if w["kind"] == "gemm" else lead

        def run(rows):
            t = time.perf_counter()
            o.c_gemm(a2[:rows], b if w["kind"] == "gemm" else b[:rows], "te_llvm", order=order,
                     threads=threads)
            return time.perf_counter() - t
        probe = 4 if w["kind"] == "gemm" else 1
        t1 = run(probe)
        rows = int(max(probe, min(rows_total, probe * budget_s / max(t1, 1e-6))))
        t = run(rows) if rows > probe else t1
        unit_ops = 2.0 * w["n"] * w["k"] * (1 if w["kind"] == "gemm" else w["m"])
        ops = unit_ops * rows
        whole = rows == rows_total
        sample = f"{rows} of {rows_total} " + ("rows of M" if w["kind"] == "gemm" else "batches")
    i8 = w.get("dtype") == "s8"
    how = "the whole workload" if whole else f"extrapolated from a slice: {sample}"
    return {"value": ops / t / 1e12, "unit": "TOP/s" if i8 else "TFLOP/s", "cores": threads,
            "kind": "port", "sample": how + f", {t:.1f} s, te_llvm arithmetic, loop order "
            + ("i,j,k as scheduled by default" if order == 0 else "interchanged")}


def _line_for(name, args, world, res, red, peaks, peaks_kind, int8_peak):
    """value / roofline / burst records of one measured workload (rank 0)."""
    w = WORKLOADS[name]
    full = make_desc(w)
    i8 = w.get("dtype") == "s8"
    steps_total = args.steps * res["passes"]
    ms_per_step = red["ms"] / steps_total
    burst_ms_per_step = red["burst_ms"] / args.steps
    ops, byts = red["ops_local"], red["bytes_local"]
    long_region = red["ms"] >= 500.0
    roof = roofline_for(full, ops, byts, ms_per_step, world, peaks, peaks_kind, long_region,
                        int8_peak)
    traffic, source = ncu_traffic(name)
    roof["traffic"] = traffic
    roof["traffic_source"] = source
    burst = roofline_for(full, ops, byts, burst_ms_per_step, world, peaks, peaks_kind, False,
                         int8_peak)
    burst_rec = {"value": ops / (burst_ms_per_step / 1e3) / 1e12, "ms_per_step": burst_ms_per_step,
                 "timed_region_s": red["burst_ms"] / 1e3, "frac": burst["frac"],
                 "peak": burst["peak"], "peak_source": burst["peak_source"]}
    return ms_per_step, ops / (ms_per_step / 1e3) / 1e12, roof, burst_rec, i8


def run_ours(args):
    import torch
    from amos_b200 import _lib
    _lib.load()
    rank, world, local = _dist_env()
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    dev = local
    torch.cuda.set_device(dev)
    numa = bind_to_gpu_cpus(dev) if world > 1 else None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{dev}"))
    peaks, peaks_kind = load_peaks()
    name = args.workload
    w = WORKLOADS[name]
    sampler = ClockSampler(dev) if rank == 0 else None
    need_i8 = (w.get("dtype") == "s8" or not args.no_others) and not args.no_int8_peak
    int8_peak = measure_int8_library_peak(dev) if need_i8 else None
    if world > 1 and need_i8:
        # every rank measured its own GPU; the slowest one is the job's denominator
        import torch.distributed as dist
        vals = torch.tensor([int8_peak["int8_tops"] if int8_peak else 0.0,
                             int8_peak["int8_tops_sustained"] if int8_peak else 0.0],
                            dtype=torch.float64, device=f"cuda:{dev}")
        dist.all_reduce(vals, op=dist.ReduceOp.MIN)
        if float(vals[0]) > 0 and int8_peak:
            int8_peak["int8_tops"], int8_peak["int8_tops_sustained"] = float(vals[0]), float(vals[1])
        else:
            int8_peak = None
    res = measure_workload(name, args.steps, args.warmup, world, rank, dev, sampler,
                           e2e_steps=max(3, min(args.steps, 20)), scaling=args.scaling,
                           min_region_s=args.min_region_s, check_shard=True, time_gather=True)
    red = reduce_over_ranks(res, world, dev)
    ms_per_step, value, roof, burst_rec, i8 = _line_for(name, args, world, res, red, peaks,
                                                        peaks_kind, int8_peak)
    unit = "TOP/s" if i8 else "TFLOP/s"
    ops = red["ops_local"]
    e2e_steps = res.get("e2e_steps", 1)
    e2e_val = ops / ((red["e2e_ms"] / e2e_steps) / 1e3) / 1e12 if red["e2e_ms"] else None

    weak_rec = None
    if world > 1 and args.scaling == "strong" and w["shard"]:
        wres = measure_workload(name, args.steps, 3, world, rank, dev, scaling="weak")
        wred = reduce_over_ranks(wres, world, dev)
        wms = wred["ms"] / args.steps
        weak_rec = {"value": wred["ops_local"] / (wms / 1e3) / 1e12, "unit": unit,
                    "ms_per_step": wms,
                    "note": "every rank runs the named configuration on its own rows / batches / "
                            "images (the job is n_gpus times the configuration); short region"}

    # the other named configurations, briefly (short regions: burst denominators)
    others = {}
    if not args.no_others:
        steps_o = max(5, min(args.steps, 30))
        for other in WORKLOADS:
            if other == name:
                continue
            r = measure_workload(other, steps_o, 3, world, rank, dev, scaling=args.scaling,
                                 check_shard=True)
            if r is None:
                continue
            o_red = reduce_over_ranks(r, world, dev)
            d_o = make_desc(WORKLOADS[other])
            per = o_red["ms"] / steps_o
            rf = roofline_for(d_o, o_red["ops_local"], o_red["bytes_local"], per, world, peaks,
                              peaks_kind, False, int8_peak)
            others[other] = {"value": o_red["ops_local"] / (per / 1e3) / 1e12,
                             "unit": "TOP/s" if WORKLOADS[other].get("dtype") == "s8" else "TFLOP/s",
                             "us_per_step": per * 1e3, "roofline_bound": rf["bound"],
                             "roofline_frac": rf["frac"], "kernels_per_step": r["launches_per_step"]}
            if world > 1:
                others[other]["shard_parity"] = bool(o_red["shard_ok"])
            elif rf["bound"] == "hbm":
                cp_us = same_size_copy_us(o_red["bytes_local"], dev)
                if cp_us:
                    others[other]["copy_of_same_bytes_us"] = cp_us
                    others[other]["frac_of_same_size_copy"] = cp_us / (per * 1e3)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(name)
    if rank == 0:
        clocks = sampler.summary() if sampler else None
        if clocks and clocks.get("sm_mhz"):
            clocks["ms_per_step_x_mhz"] = ms_per_step * clocks["sm_mhz"]
        line = {
            "metric": "TFLOP/s (int8: TOPS) per conv/GEMM config",
            "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": args.scaling if world > 1 else "strong", "vs_baseline": None,
            "dtype": "s8" if i8 else ("tf32" if w.get("dtype") == "f32" else "f16"),
            "data": "synthetic",
            "config": config_for(name, world, args.scaling),
            "run": {"launch": res.get("launch"), "rank0_cpus": numa,
                    "passes": res["passes"], "timed_region_s": red["ms"] / 1e3,
                    "l2": f"rotating {res.get('nsets', 1)} operand sets "
                          f"({res.get('nsets', 1) * res['bytes_local'] / 1e6:.0f} MB per rank) "
                          "larger than the 126 MB L2"},
            "burst": burst_rec,
            "e2e": {"value": e2e_val, "unit": unit, "h2d_bytes_per_step": int(red["h2d"]),
                    "d2h_bytes_per_step": int(red["d2h"]),
                    "ms_per_step_per_rank": ([x / e2e_steps for x in red["e2e_ms_per_rank"]]
                                             if red["e2e_ms_per_rank"] else None),
                    "result_matches_device_run": bool(red["e2e_ok"]),
                    "note": ("shard.HostShardedCall, every step: each rank copies its own rows and "
                             "1/n_gpus of the replicated operand from pinned host memory, the "
                             "slices are all-gathered over NVLink (NCCL), kernels, the rank's rows "
                             "of the result are copied back; h2d/d2h bytes are summed over ranks"
                             if red.get("e2e_via") == "shard.HostShardedCall" else
                             "Module(*numpy) -> amosb_run_host: pinned host operands copied in, "
                             "kernels, full output copied back, every step; all ranks share one "
                             "host's PCIe and memory bus")},
            "gpu_launches": int(red["launches"]),
            "roofline": roof,
            "int8_peak": int8_peak,
            "cpu_baseline": cpu,
            "clocks": clocks,
            "configs": others,
        }
        if world > 1 and args.scaling == "strong":
            line["shard_parity"] = bool(red["shard_ok"])
            line["shard_parity_detail"] = {
                "bit_exact": bool(red["shard_bit_exact"]), "max_rel_l2": red["shard_rel_l2"],
                "how": "every rank runs the unsharded operator on its own GPU from the same seed "
                       "and compares its shard with the same rows / batches / images"}
            gbytes = res.get("gather_bytes", 0)
            line["gather"] = {"ms": red["gather_ms"], "bytes": gbytes,
                              "gbs": (gbytes / (red["gather_ms"] / 1e3) / 1e9
                                      if red["gather_ms"] else None),
                              "note": "shard.gather_output: NCCL all-gather of the output shards "
                                      "to every rank, outside the timed compute path"}
            line["weak_scaling"] = weak_rec
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# Reference arm: the CPU restatement of the reference's llvm build, all host threads
# --------------------------------------------------------------------------------------------
def run_reference(args):
    rank, world, _ = _dist_env()
    if rank != 0:
        return
    from oracle import oracle as o
    o.build()
    name = args.workload
    w = WORKLOADS[name]
    threads = len(os.sched_getaffinity(0))
    host = make_inputs(w)
    total_steps = args.steps + max(args.warmup, 0)
    budget_per_step = max(0.3, 90.0 / max(total_steps, 1))
    i8 = w.get("dtype") == "s8"
    if w["kind"] == "conv":
        a, f = host
        d = make_desc(w)
        per_unit = 2.0 * w["k"] * w["c"] * w["r"] * w["s"] * d.conv_p * d.conv_q
        total_units, unit_name = w["n"], "images"

        def run(units):
            if w.get("layout") == "hwnc":
                o.c_conv2d_hwnc(a[:, :, :units], f, w["stride"], w["pad"], w["dil"], "te_llvm",
                                threads=threads)
            elif w.get("layout") == "nhwc":
                o.c_conv2d_nhwc(a[:units], f, w["stride"], w["pad"], w["dil"], "te_llvm",
                                threads=threads)
            else:
                o.c_conv2d_nchw(a[:units], f, w["stride"], w["pad"], w["dil"], "te_llvm", order=0,
                                threads=threads)
    else:
        a, b = host
        gem = w["kind"] == "gemm"
        per_unit = 2.0 * w["n"] * w["k"] * (1 if gem else w["m"])
        total_units, unit_name = (w["m"], "rows of M") if gem else (w["batch"], "batches")

        def run(units):
            o.c_gemm(a[:units], b if gem else b[:units], "te_llvm", order=0, threads=threads)
    probe = min(total_units, threads if w["kind"] != "conv" else 1)
    t = time.perf_counter()
    run(probe)
    t_probe = time.perf_counter() - t
    units = int(max(probe, min(total_units, probe * budget_per_step / max(t_probe, 1e-6))))
    for _ in range(max(args.warmup, 0)):
        run(units)
    t = time.perf_counter()
    for _ in range(args.steps):
        run(units)
    dt = time.perf_counter() - t
    value = per_unit * units * args.steps / dt / 1e12
    unit = "TOP/s" if i8 else "TFLOP/s"
    how = "the whole workload" if units == total_units else \
        f"extrapolated from a slice: {units} of {total_units} {unit_name} per step"
    sample = (f"{how}; C restatement of the te default schedule (loops i,j,k), te_llvm "
              f"arithmetic, OpenMP over the outer axis")
    print(json.dumps({
        "impl": "reference",
        "metric": "TFLOP/s (int8: TOPS) per conv/GEMM config",
        "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": args.scaling if args.gpus > 1 else "strong", "vs_baseline": None,
        "dtype": "s8" if i8 else ("tf32" if w.get("dtype") == "f32" else "f16"),
        "data": "synthetic",
        "config": config_for(name, args.gpus, args.scaling),
        "note": "the reference (TVM llvm build) cannot be built here; this is its CPU restatement "
                "(oracle port) on the host cores of rank 0; the figure does not depend on n_gpus",
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: strong = the named configuration is split over the ranks (rows of "
                         "M / batches / images); weak = every rank runs the named configuration on "
                         "its own rows / batches / images (the job is N times the configuration)")
    ap.add_argument("--min-region-s", type=float, default=0.5,
                    help="replay the captured steps until the timed region of the headline "
                         "workload lasts at least this long (0: one pass)")
    ap.add_argument("--no-others", action="store_true", help="skip the non-headline configs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-int8-peak", action="store_true",
                    help="skip measuring the int8 library peak (int8 rows then use 2 x the bf16 peak, "
                         "stated); for runs under a profiler")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

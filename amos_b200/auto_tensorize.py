"""The `tvm.auto_tensorize` (``at``) surface on top of the fixed-mapping sm_100a kernels.

Kept from the reference: the entry points and result objects callers use
(reference: python/tvm/auto_tensorize/auto_tensorize.py:37-51, 242-301, 661-685;
python/tvm/auto_tensorize/search/measure.py:26-61, 319-338; the JSON-lines tuning log of
python/tvm/auto_tensorize/search/parameter.py:269-316).

Replaced: intrinsic matching, mapping enumeration and schedule search.  The native recogniser
classifies the `te` DAG; the "search space" that remains is the tile width of the tcgen05 kernel
(64 / 128 / 256 output columns per CTA tile), explored by timing each variant on the device.
Search knobs of the reference that no longer mean anything are accepted and ignored.
"""
from __future__ import annotations

import json
import os
import time

from . import _lib, te

MAX_FLOAT = 1e10

_NO_MATCH = "This workload has no matched intrinsic for target: %s"


# ------------------------------------------------------------------------------------------------
# DAG view
# ------------------------------------------------------------------------------------------------
class ComputeDAG:
    """`at.compute_dag_from_tensors([out])` (reference: python/tvm/auto_tensorize/hw_abstraction/
    hw_abs_base.py:8-25, src/auto_tensorize/hw_abstraction.cc:77-94)."""

    def __init__(self, tensors):
        self.tensors = list(tensors)
        ops = te.topo_ops(self.tensors)
        self.op_lst = [op for op in ops if not isinstance(op, te.PlaceholderOp)]
        self.read_graph = {op: list(op.input_tensors) for op in self.op_lst}
        self.feed_graph: dict = {}
        for op in self.op_lst:
            for inp in op.input_tensors:
                self.feed_graph.setdefault(inp.op, []).append(op)

    def get_inputs(self):
        inputs = []
        for op in self.op_lst:
            for inp in op.input_tensors:
                if isinstance(inp.op, te.PlaceholderOp) and all(inp is not x for x in inputs):
                    inputs.append(inp)
        return inputs

    def serialise(self) -> str:
        return te.serialise_dag(self.tensors)


def compute_dag_from_tensors(tensors) -> ComputeDAG:
    return ComputeDAG(tensors)


# ------------------------------------------------------------------------------------------------
# Measurement options / params / log entries
# ------------------------------------------------------------------------------------------------
class MeasureOptions:
    """Same fields as the reference (python/tvm/auto_tensorize/search/measure.py:26-61)."""

    def __init__(self, target="llvm", build_func="default", target_host="llvm", timeout=10,
                 verbose=1, number=100, repeat=1, min_repeat_ms=150, cooldown_interval=0,
                 enable_cpu_cache_flush=1, dev_id=0, use_rpc=False, key=None, host=None,
                 port=None, priority=1):
        self.target = target
        self.build_func = build_func
        self.target_host = target_host
        self.timeout = timeout
        self.verbose = verbose
        self.number = number
        self.repeat = repeat
        self.min_repeat_ms = min_repeat_ms
        self.cooldown_interval = cooldown_interval
        self.enable_cpu_cache_flush = enable_cpu_cache_flush
        self.dev_id = dev_id
        self.use_rpc = use_rpc
        self.key = key
        self.host = host
        self.port = port
        self.priority = priority


class TileParams:
    """Schedule parameters: the one free choice left, stored like the reference's params as
    ``[value, direction]`` pairs (reference: python/tvm/auto_tensorize/tensorization_phases/
    schedulers/cuda_v2.py:23-76)."""

    def __init__(self, tile_n: int = 0, cta_pair: int = 0):
        self.foreign = False           # True for a record read from a log of the reference's tuner
        self.tile_n = int(tile_n)      # 0 = launcher's choice, else 64 / 128 / 256
        self.cta_pair = int(cta_pair)  # 0 = launcher's choice, 1 = one CTA per tile, 2 = CTA pairs, 3 = tall tiles

    def to_json(self) -> dict:
        return {"tile_n": [self.tile_n, 0], "cta_pair": [self.cta_pair, 0]}

    @classmethod
    def from_json(cls, obj: dict) -> "TileParams":
        """Records written by this library carry `tile_n` / `cta_pair`.  A record of the reference's
        own tuner (`inline`, `vectorize`, `spatial_factors`, ...: schedulers/cuda_v2.py:23-76)
        describes a kernel that does not exist here: it is read as "launcher's choice" and marked
        `foreign`, so that old logs load and their values can be shown, without steering anything."""
        def val(key):
            v = obj.get(key, [0, 0])
            return v[0] if isinstance(v, (list, tuple)) else v
        params = cls(val("tile_n"), val("cta_pair"))
        params.foreign = "tile_n" not in obj and "cta_pair" not in obj
        return params

    def __str__(self):
        return json.dumps(self.to_json())

    __repr__ = __str__


class Entry:
    def __init__(self, record: TileParams, value: float):
        self.record = record
        self.value = value

    def to_json(self) -> dict:
        return {"record": self.record.to_json(), "value": self.value}


class Mapping:
    """The (single) mapping of an operator onto the tcgen05 instruction, printable like the
    reference's IntrinMatchResult / Record."""

    def __init__(self, desc: _lib.AmosbOpDesc):
        kind = _lib.OP_NAMES[desc.kind]
        self.hw_abs_dag = {_lib.AMOSB_S8: "tcgen05_int8_int32",
                           _lib.AMOSB_BF16: "tcgen05_bf16_fp32",
                           _lib.AMOSB_F32: "tcgen05_tf32_fp32"}.get(desc.in_dtype,
                                                                    "tcgen05_fp16_fp32")
        self.compute_key = ("t" if desc.trans_a else "n") + \
            ("t" if (desc.trans_b or kind == "conv2d_nchw") else "n") + "n"
        self.shape_key = "128x{N}x" + {_lib.AMOSB_S8: "32", _lib.AMOSB_F32: "8"}.get(desc.in_dtype,
                                                                                    "16")
        if kind in ("conv2d_nchw", "conv2d_nhwc", "conv2d_hwnc"):
            self.axis_map = {"i": ["n", "p", "q"], "j": ["k"], "rk": ["rr", "rs", "rc"]}
        elif kind == "batched_gemm":
            self.axis_map = {"i": ["i"], "j": ["j"], "rk": ["k"], "time": ["b"]}
        else:
            self.axis_map = {"i": ["i"], "j": ["j"], "rk": ["k"]}

    def to_json(self) -> dict:
        return {"hw_abs_dag": self.hw_abs_dag, "compute_key": self.compute_key,
                "shape_key": self.shape_key, "axis_map": self.axis_map}

    def __str__(self):
        return (f"MatchResult(hw_abs_dag:{self.hw_abs_dag}, compute:{self.compute_key}, "
                f"shape:{self.shape_key}, axis_map:{self.axis_map})")


class ScheduleGenerator:
    """Keeps measured entries, best first, and the JSON-lines log
    (reference: python/tvm/auto_tensorize/search/parameter.py:269-316)."""

    def __init__(self, desc: _lib.AmosbOpDesc, log_file: str | None):
        self.desc = desc
        self.log_file = log_file
        self.entries: list[Entry] = []

    def candidates(self) -> list[TileParams]:
        d = self.desc
        conv = d.kind in _lib.CONV_KINDS
        n = d.conv_k if conv else d.n
        i8_mn = d.in_dtype == _lib.AMOSB_S8 and not conv and not d.trans_b
        rows = d.conv_n * d.conv_p * d.conv_q if conv else d.m
        widths = [256, 128] if i8_mn else [256, 128, 64]
        out = []
        for w in widths:
            smaller = [x for x in widths if x < w]
            if smaller and n <= max(smaller):
                continue  # a narrower tile already covers N
            out.append(TileParams(w, 1))
            if not conv and (d.trans_a or d.in_dtype == _lib.AMOSB_F32):
                continue  # A[k,i] and float32 (tf32) operands: single-CTA 128-row tiles only
            if d.kind == _lib.OP_CONV2D_HWNC:
                if rows > 128 and w == 128:
                    out.append(TileParams(w, 3))
                continue  # HWNC: single-CTA tiles (128 or 256 rows)
            if rows > 128 and (w == 256 or (w == 128 and not i8_mn)):
                out.append(TileParams(w, 2))
            if rows > 128 and w == 128 and d.in_dtype in (_lib.AMOSB_F16, _lib.AMOSB_BF16):
                out.append(TileParams(w, 3))  # one CTA per 256 x 128 tile
        return out or [TileParams(widths[-1], 1)]

    def feedback(self, record: TileParams, value: float, log_to_file: bool = True) -> None:
        self.entries.append(Entry(record, value))
        self.entries.sort(key=lambda e: -e.value)
        if log_to_file and self.log_file:
            with open(self.log_file, "a") as f:
                print(json.dumps(Entry(record, value).to_json()), file=f, flush=True)

    def clear(self, log_file: str | None) -> None:
        self.entries = []
        self.log_file = log_file

    def load_from_file(self, file_name: str, clear: bool = False) -> None:
        if clear:
            self.clear(file_name)
        with open(file_name, "r") as fin:
            for line in fin:
                line = line.strip()
                if not line:
                    continue
                obj = json.loads(line)
                self.feedback(TileParams.from_json(obj["record"]), obj["value"], False)

    def num_entries(self) -> int:
        return len(self.entries)

    def has_entry(self) -> bool:
        return bool(self.entries)

    def topk(self, k: int = 1):
        return self.entries[:k]

    def num_foreign_entries(self) -> int:
        return sum(1 for e in self.entries if e.record.foreign)

    def get_best_entry(self) -> Entry:
        """Best measured entry of this library's own kernels; if the log only holds records of the
        reference's tuner, the best of those (its value is what that log says, nothing more)."""
        assert self.entries
        own = [e for e in self.entries if not e.record.foreign]
        return own[0] if own else self.entries[0]


class ScheduleApplier:
    """`result.sch_app`: carries the DAG and stamps the chosen kernel plan on a schedule."""

    def __init__(self, target_dag: ComputeDAG, desc: _lib.AmosbOpDesc):
        self.target_dag = target_dag
        self.desc = desc

    def apply(self, sch: te.Schedule, params: TileParams, mapping_func=None) -> te.Schedule:
        d = self.desc.copy()
        d.tile_n = int(params.tile_n) if params is not None else 0
        d.cta_pair = int(getattr(params, "cta_pair", 0)) if params is not None else 0
        sch.plan = d
        return sch


class AutoTensorizeResult:
    def __init__(self, sch_gen=None, sch_app=None, params=None, perf=None, mapping=None):
        self.sch_gen = sch_gen
        self.sch_app = sch_app
        self.params = params
        self.perf = perf
        self.mapping = mapping

    def defined(self) -> bool:
        return (self.sch_gen is not None and self.sch_app is not None
                and self.params is not None and self.perf is not None)


# ------------------------------------------------------------------------------------------------
# Build / evaluate
# ------------------------------------------------------------------------------------------------
def get_match_results(target_dag: ComputeDAG, target: str = "cuda"):
    """Recognise the operator; returns a list with one mapping, or [] when nothing matches
    (reference: python/tvm/auto_tensorize/tensorization_phases/intrin_match.py:168-181)."""
    if str(target) != "cuda":
        return []
    try:
        desc = _lib.recognize(target_dag.serialise())
    except _lib.AmosbError as e:
        if e.code == _lib.AMOSB_ERR_UNSUPPORTED:
            return []
        raise
    m = Mapping(desc)
    m.desc = desc
    return [m]


def get_schedule(sch_app: ScheduleApplier, params: TileParams):
    """reference: python/tvm/auto_tensorize/auto_tensorize.py:294-301."""
    target_dag = sch_app.target_dag
    inputs = target_dag.get_inputs()
    sch = te.create_schedule([x.op for x in target_dag.tensors])
    args = inputs + list(target_dag.tensors)
    sch = sch_app.apply(sch, params)
    return sch, args


def _random_args(desc: _lib.AmosbOpDesc, dev_id: int):
    """Random operands for timing, like the reference runner's random_fill
    (python/tvm/auto_tensorize/search/measure.py:697-704)."""
    import torch
    from . import device
    dev = f"cuda:{dev_id}"
    tdt = device.CODE_TO_TORCH
    if desc.kind == _lib.OP_CONV2D_NCHW:
        shapes = [(desc.conv_n, desc.conv_c, desc.conv_h, desc.conv_w),
                  (desc.conv_k, desc.conv_c, desc.conv_r, desc.conv_s)]
        oshape = (desc.conv_n, desc.conv_k, desc.conv_p, desc.conv_q)
    elif desc.kind == _lib.OP_CONV2D_NHWC:
        shapes = [(desc.conv_n, desc.conv_h, desc.conv_w, desc.conv_c),
                  (desc.conv_r, desc.conv_s, desc.conv_c, desc.conv_k)]
        oshape = (desc.conv_n, desc.conv_p, desc.conv_q, desc.conv_k)
    elif desc.kind == _lib.OP_CONV2D_HWNC:
        shapes = [(desc.conv_h, desc.conv_w, desc.conv_n, desc.conv_c),
                  (desc.conv_r, desc.conv_s, desc.conv_c, desc.conv_k)]
        oshape = (desc.conv_p, desc.conv_q, desc.conv_n, desc.conv_k)
    else:
        a = (desc.k, desc.m) if desc.trans_a else (desc.m, desc.k)
        b = (desc.n, desc.k) if desc.trans_b else (desc.k, desc.n)
        oshape = (desc.m, desc.n)
        if desc.kind == _lib.OP_BATCHED_GEMM:
            a, b, oshape = (desc.batch,) + a, (desc.batch,) + b, (desc.batch,) + oshape
        shapes = [a, b]
    ordered = [None] * desc.n_inputs
    ordered[desc.arg_a], ordered[desc.arg_b] = shapes[0], shapes[1]
    ins = []
    for i, s in enumerate(ordered):
        if s is None:  # the fused addend
            n_axis = desc.conv_k if desc.kind in _lib.CONV_KINDS else desc.n
            ashape = (n_axis,) if desc.epilogue & _lib.EPI_ADD_VECTOR else oshape
            ins.append(torch.zeros(ashape, dtype=tdt[desc.addend_dtype], device=dev))
        elif desc.in_dtype == _lib.AMOSB_S8:
            ins.append(torch.randint(-128, 128, s, dtype=torch.int8, device=dev))
        else:
            ins.append((torch.rand(s, device=dev) * 2 - 1).to(tdt[desc.in_dtype]))
    out = torch.empty(oshape, dtype=tdt[desc.out_dtype], device=dev)
    return ins, [out]


def evaluate_params(schedule_app: ScheduleApplier, params: TileParams,
                    measure_opt: MeasureOptions, timeout=100, dump=False) -> float:
    """Mean time of one run in milliseconds, or MAX_FLOAT on failure
    (reference: python/tvm/auto_tensorize/search/measure.py:319-338)."""
    from . import runtime
    try:
        sch, _ = get_schedule(schedule_app, params)
        mod = runtime.Module(sch.plan)
        if dump:
            print(mod.imported_modules[0].get_source()[:2000], flush=True)
        ins, outs = _random_args(sch.plan, measure_opt.dev_id)
        ev = mod.time_evaluator(mod.entry_name, runtime.gpu(measure_opt.dev_id),
                                number=max(1, min(measure_opt.number, 100)),
                                repeat=max(1, measure_opt.repeat),
                                min_repeat_ms=measure_opt.min_repeat_ms)
        return ev(*ins, *outs).mean * 1e3
    except Exception as e:  # measurement failures are data, as in the reference
        if measure_opt.verbose:
            print("Evaluate Fatal Error\n", repr(e), flush=True)
        return MAX_FLOAT


def _device_present(dev_id: int) -> bool:
    try:
        import torch
        return torch.cuda.is_available() and dev_id < torch.cuda.device_count()
    except Exception:
        return False


def _tensorize(target_dag, target, log_file, measure_opt, trials, verbose, tag="auto_tensorize",
               read_only_logs=()):
    measure_opt.target = target
    matches = get_match_results(target_dag, target)
    if not matches:
        print(_NO_MATCH % target, flush=True)
        return AutoTensorizeResult()
    mapping = matches[0]
    desc = mapping.desc
    print("Possible matchings:", flush=True)
    print(0, ":", str(mapping), flush=True)
    sch_gen = ScheduleGenerator(desc, log_file)
    sch_app = ScheduleApplier(target_dag, desc)
    if log_file and os.path.isfile(log_file):
        sch_gen.load_from_file(log_file)
    for extra in read_only_logs:
        sch_gen.load_from_file(extra)
    if sch_gen.num_foreign_entries():
        print(f"[{tag}] read {sch_gen.num_foreign_entries()} records of the reference's tuner; "
              "they are kept for display and do not select a kernel", flush=True)
    if trials:
        if not _device_present(measure_opt.dev_id):
            raise _lib.AmosbError(_lib.AMOSB_ERR_CUDA,
                                  "tuning needs a CUDA device; pass trials=0 to only plan")
        beg = time.time()
        for params in sch_gen.candidates()[: max(1, int(trials))]:
            ms = evaluate_params(sch_app, params, measure_opt)
            ok = ms < MAX_FLOAT
            print(".Y" if ok else ".E", end="", flush=True)
            print("*Y" if ok else "*E", end="", flush=True)
            sch_gen.feedback(params, 1.0 / (ms / 1e3) if ok else 1.0 / MAX_FLOAT)
        print(flush=True)
        if verbose:
            print(f"[{tag}] explored {sch_gen.num_entries()} tile variants in "
                  f"{time.time() - beg:.2f} s", flush=True)
    if sch_gen.entries:
        entry = sch_gen.get_best_entry()
        params, perf = entry.record, 1.0 / entry.value  # the log stores 1/seconds
    else:
        # nothing measured and no log: the launcher's own tile heuristic, cost unknown
        params, perf = TileParams(0), MAX_FLOAT
    return AutoTensorizeResult(sch_gen, sch_app, params, perf, mapping=mapping)


def auto_tensorize(target_dag, target, log_file, measure_opt, trials=200, builder=None,
                   runner=None, verbose=False, transform_dump=False, transform_strict=True,
                   drop_output=False, transform_policy="all_fit", search_group_size=16,
                   enable_split_K=False, build_parallel=1, run_parallel=1):
    """reference: python/tvm/auto_tensorize/auto_tensorize.py:242-291."""
    print("[AMOS] Mapping starts...\nUsing the fixed tcgen05 mapping with tile-width tuning",
          flush=True)
    return _tensorize(target_dag, target, log_file, measure_opt, trials, verbose)


def auto_tensorize_v2(target_dag, target, log_file, measure_opt, trials=200, **kwargs):
    return _tensorize(target_dag, target, log_file, measure_opt, trials,
                      kwargs.get("verbose", False), "auto_tensorize_v2")


def auto_tensorize_v3(target_dag, target, log_file, measure_opt, trials=200, **kwargs):
    return _tensorize(target_dag, target, log_file, measure_opt, trials,
                      kwargs.get("verbose", False), "auto_tensorize_v3")


def auto_tensorize_v4(target_dag, target, schedule_log_file, measure_opt,
                      schedule_log_dir="schedules", trials=200, repeat_rounds=10, builder=None,
                      runner=None, verbose_schedule=False, transform_dump=False,
                      transform_strict=True, search_group_size=5, desired_compute_key=None,
                      desired_shape_key=None, enable_split_K=False, use_shared_store=False,
                      drop_output=False, build_parallel=1, run_parallel=1,
                      explore_full_match=False, enable_perf_model=False, perf_percentage=0.5):
    """reference: python/tvm/auto_tensorize/auto_tensorize.py:661-685.  One mapping exists, so the
    per-mapping log directory holds a single file; `trials=0` is the pure test mode that only
    reads the log (reference: :779-783)."""
    if trials == 0:
        print("Pure testing mode...", flush=True)
    log_file = schedule_log_file
    if schedule_log_dir and schedule_log_file and not os.path.isabs(schedule_log_file) \
            and os.path.dirname(schedule_log_file) == "":
        if trials or os.path.isdir(schedule_log_dir):
            os.makedirs(schedule_log_dir, exist_ok=True)
            log_file = os.path.join(schedule_log_dir, schedule_log_file)
    # per-mapping files of the reference's v4 tuner in the same directory
    # ("mapping_<bits>_<log file>", auto_tensorize.py:827-829): read, never written
    import glob
    old = []
    if schedule_log_dir and schedule_log_file and os.path.isdir(schedule_log_dir):
        pattern = os.path.join(glob.escape(schedule_log_dir),
                               "mapping_*_" + glob.escape(os.path.basename(schedule_log_file)))
        old = sorted(glob.glob(pattern))
    return _tensorize(target_dag, target, log_file, measure_opt, trials, verbose_schedule,
                      "auto_tensorize_v4", read_only_logs=old)


# ------------------------------------------------------------------------------------------------
# Names the network-level dispatcher reaches for below the public entry points
# (reference: python/tvm/tensor_graph/core/auto_schedule/auto_schedule.py:351-433, 719-830)
# ------------------------------------------------------------------------------------------------
class TransformState:
    """What `auto_tensorize_compute` hands on as `new_state`: the DAG and its recognised operator.
    (The reference's state holds the DAG rewritten for the chosen mapping; there is one mapping
    here and no rewrite.)"""

    def __init__(self, target_dag: ComputeDAG, desc: _lib.AmosbOpDesc):
        self.target_dag = target_dag
        self.desc = desc


def auto_tensorize_compute(target_dag, target, log_file, measure_opt, verbose=False,
                           transform_dump=False, transform_strict=True, drop_output=False,
                           transform_policy="all_fit"):
    """-> (match_result, new_state), or (None, None) with the reference's message when nothing
    matches (reference: python/tvm/auto_tensorize/auto_tensorize.py:54-120)."""
    measure_opt.target = target
    matches = get_match_results(target_dag, target)
    if not matches:
        print(_NO_MATCH % target, flush=True)
        return None, None
    print("Possible matchings:", flush=True)
    for i, m in enumerate(matches):
        print(i, ":", str(m), flush=True)
    return matches[0], TransformState(target_dag, matches[0].desc)


class ScheduleComputeInfo:
    def __init__(self, target_dag: ComputeDAG, desc: _lib.AmosbOpDesc):
        self.target_dag = target_dag
        self.desc = desc


class CUDAScheduleGeneratorV2(ScheduleGenerator):
    """reference: python/tvm/auto_tensorize/tensorization_phases/schedulers/cuda_v2.py:90-395."""

    def __init__(self, match_result, new_state, log_file=None, arch=100, verbose_init=True):
        super().__init__(new_state.desc, log_file)
        self.match_result = match_result
        self.target_dag = new_state.target_dag

    def get_schedule_compute_info(self) -> ScheduleComputeInfo:
        return ScheduleComputeInfo(self.target_dag, self.desc)


class CUDAScheduleApplierV2(ScheduleApplier):
    """reference: .../schedulers/cuda_v2.py:398-854."""

    def __init__(self, match_result, schedule_compute_info, arch=100, verbose_init=True):
        super().__init__(schedule_compute_info.target_dag, schedule_compute_info.desc)
        self.match_result = match_result


class CUDAProgramChecker:
    """Accepted for interface compatibility: every compiled tile variant fits the device by
    construction, so there is nothing to reject (reference: search/checker.py:43-82)."""

    def __init__(self, check_scope=3, arch=100, verbose_init=True):
        self.arch = arch

    def check(self, ir_module=None) -> None:
        return None


def get_cuda_compute_version(dev_id: int = 0) -> int:
    if _device_present(dev_id):
        import torch
        major, minor = torch.cuda.get_device_capability(dev_id)
        return major * 10 + minor
    return 100


def pebble_local_builder_build(*args, **kwargs):
    """Builder hook of the reference's search loop; nothing is compiled at tuning time here."""
    return None


def pebble_local_runner_run(*args, **kwargs):
    """Runner hook of the reference's search loop; `find_optimized_parameters` times in-process."""
    return None


tg_parallel_builder_build = pebble_local_builder_build


def find_optimized_parameters(match_results, schedule_gen, schedule_app, measure_opt, checker,
                              trials, search_group_size=16, policy="", builder=None, runner=None,
                              verbose=False, build_parallel=1, run_parallel=1):
    """Time up to `trials` tile variants, feed them to `schedule_gen` (and its log) and return
    (best value = 1/seconds, best params) (reference: search/parameter.py:386-460)."""
    best_value, best_params = 1 / MAX_FLOAT, None
    if schedule_gen.has_entry():
        top1 = schedule_gen.topk(k=1)[0]
        best_value, best_params = top1.value, top1.record
    if trials:
        if not _device_present(measure_opt.dev_id):
            raise _lib.AmosbError(_lib.AMOSB_ERR_CUDA,
                                  "tuning needs a CUDA device; pass trials=0 to only plan")
        for params in schedule_gen.candidates()[: max(1, int(trials))]:
            ms = evaluate_params(schedule_app, params, measure_opt)
            ok = ms < MAX_FLOAT
            print(".Y*Y" if ok else ".E*E", end="", flush=True)
            value = 1.0 / (ms / 1e3) if ok else 1.0 / MAX_FLOAT
            schedule_gen.feedback(params, value)
            if value > best_value:
                best_value, best_params = value, params
        print(flush=True)
    return best_value, best_params


find_optimized_parameters_v2 = find_optimized_parameters
find_optimized_parameters_v3 = find_optimized_parameters

"""Routing of network sub-graphs onto the tensor-core kernels.

A graph-level scheduler (the reference's `tensor_graph` auto-scheduler is one) hands over
sub-graphs: objects with `root_ops` (the `te` operations whose first outputs are the sub-graph's
results) and a printable `tag`.  For each it wants to know whether the tensor-core path applies,
to spend a number of tuning trials on it, and to get back `(schedule, args)` for `tvm.build`
together with the cost in milliseconds.

Contract kept (names, arguments, return values, log location "at:<task>.log"):
reference python/tvm/tensor_graph/core/auto_schedule/auto_schedule.py:92-105 (`auto_tensorize_cuda`)
and :351-433 (`AutoTensorizeContext`).  The reference's own dispatcher also runs unmodified on top
of `amos_b200.auto_tensorize`; tests/test_reference_dispatcher.py executes it that way.  This
module is for callers that have no reference checkout: it is written against the contract, on
this library's own tuning objects.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Any

from . import auto_tensorize as at

_TARGET = "cuda"


def _results_of(subgraph) -> list:
    return [op.output(0) for op in subgraph.root_ops]


def _task_log(top_log_dir: str, task: str) -> str:
    return os.path.join(top_log_dir, f"at:{task}.log")


@dataclasses.dataclass
class _Tuned:
    """One recognised sub-graph with its measured tile variants."""
    dag: at.ComputeDAG
    mapping: Any
    generator: at.ScheduleGenerator
    applier: at.ScheduleApplier

    @classmethod
    def open(cls, dag: at.ComputeDAG, target: str, log_path: str | None) -> "_Tuned | None":
        """Recognise `dag`; None when no tensor-core mapping exists.  An existing log is read."""
        found = at.get_match_results(dag, target)
        if not found:
            return None
        mapping = found[0]
        gen = at.ScheduleGenerator(mapping.desc, log_path)
        if log_path and os.path.isfile(log_path):
            gen.load_from_file(log_path)
        return cls(dag, mapping, gen, at.ScheduleApplier(dag, mapping.desc))

    def measure(self, trials: int, options: at.MeasureOptions) -> None:
        """Time up to `trials` tile variants on the device and record them (log included)."""
        if trials <= 0:
            return
        if not at._device_present(options.dev_id):
            raise at._lib.AmosbError(at._lib.AMOSB_ERR_CUDA,
                                     "tuning needs a CUDA device; pass trials=0 to only plan")
        for params in self.generator.candidates()[:trials]:
            ms = at.evaluate_params(self.applier, params, options)
            self.generator.feedback(params, 1e3 / ms if ms < at.MAX_FLOAT else 1.0 / at.MAX_FLOAT)

    def best(self):
        """(schedule, args, milliseconds) of the fastest measured variant, or (None, None,
        MAX_FLOAT) when nothing has been measured or logged."""
        if not self.generator.entries:
            return None, None, at.MAX_FLOAT
        entry = self.generator.get_best_entry()
        sch, args = at.get_schedule(self.applier, entry.record)
        return sch, args, 1e3 / entry.value  # the log keeps runs per second


def auto_tensorize_cuda(sch, tensors, log_file, trials):
    """{schedule: args} for the sub-graph that ends in `tensors`.  A sub-graph without a
    tensor-core mapping comes back as {sch: []}: the caller's own schedule, no arguments, which
    tells it to schedule the sub-graph some other way."""
    options = at.MeasureOptions(target=_TARGET, timeout=10, number=200, min_repeat_ms=500)
    outcome = at.auto_tensorize(at.compute_dag_from_tensors(tensors), _TARGET, log_file, options,
                                trials=trials, transform_dump=True)
    if not outcome.defined():
        return {sch: []}
    new_sch, args = at.get_schedule(outcome.sch_app, outcome.params)
    return {new_sch: args}


class AutoTensorizeContext:
    """Tuning state of one sub-graph inside a graph-level scheduler."""

    @classmethod
    def can_use(cls, name, top_log_dir, subgraph, measure_option) -> bool:
        dag = at.compute_dag_from_tensors(_results_of(subgraph))
        return bool(at.get_match_results(dag, measure_option.target))

    def __init__(self, name, top_log_dir, subgraph, measure_option):
        if str(measure_option.target) != _TARGET:
            raise RuntimeError(f"the tensor-core path exists for target cuda only, not "
                               f"{measure_option.target}")
        self.name = name
        self.subgraph = subgraph
        self.measure_option = measure_option
        self.log_name = _task_log(top_log_dir, name)
        self.target_dag = at.compute_dag_from_tensors(_results_of(subgraph))
        self._tuned = _Tuned.open(self.target_dag, measure_option.target, self.log_name)
        if self._tuned is None:
            raise ValueError(f"sub-graph {name!r} has no tensor-core mapping; ask can_use() first")
        self.total_trials = 0

    # the objects a scheduler may want to look at
    @property
    def match_result(self):
        return self._tuned.mapping

    @property
    def schedule_gen(self):
        return self._tuned.generator

    @property
    def schedule_app(self):
        return self._tuned.applier

    def auto_schedule(self, trials):
        tag = getattr(self.subgraph, "tag", self.name)
        print(f"[dispatch] {tag}: {trials} trial(s), log {self.log_name}", flush=True)
        self.total_trials += trials
        self._tuned.measure(trials, self.measure_option)
        sch, args, _ = self._tuned.best()
        return sch, args

    def get_best_schedule(self):
        return self._tuned.best()

    def get_measure_opt(self):
        return self.measure_option

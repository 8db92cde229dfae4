"""Runtime boundary: what `tvm.build(sch, args, "cuda")` returns in the reference, re-provided on
top of the C ABI -- a callable module taking NDArray / DLPack / torch CUDA buffers, writing its
outputs in place, asynchronous on the current stream, plus `time_evaluator`.

reference: python/tvm/runtime/module.py:40-45, 108-112, 168-234 (Module, entry_name,
time_evaluator), src/runtime/rpc/rpc_module.cc:341-405 (timing loop), python/tvm/runtime/ndarray.py
(NDArray, array/empty), python/tvm/contrib/dlpack.py:21-65 (to_pytorch_func).
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import numpy as np
import torch

from . import _lib, device, te

_NP_TO_TORCH = {
    "float16": torch.float16,
    "float32": torch.float32,
    "int8": torch.int8,
    "int32": torch.int32,
    "bfloat16": torch.bfloat16,  # for `empty(...)`; numpy itself has no bfloat16 arrays
}


class TVMError(_lib.AmosbError):
    """Alias kept so that `except tvm.TVMError` in caller code keeps working."""


class Context:
    """Device handle (`tvm.gpu(i)` / `tvm.context("cuda", i)`)."""

    def __init__(self, device_type: str, device_id: int):
        if device_type not in ("cuda", "gpu"):
            raise _lib.AmosbError(_lib.AMOSB_ERR_UNSUPPORTED,
                                  f"only CUDA devices exist on this path, got {device_type!r}")
        self.device_type = "cuda"
        self.device_id = int(device_id)

    @property
    def exist(self) -> bool:
        return torch.cuda.is_available() and self.device_id < torch.cuda.device_count()

    def sync(self) -> None:
        torch.cuda.synchronize(self.device_id)

    def __repr__(self):
        return f"gpu({self.device_id})"


def gpu(dev_id: int = 0) -> Context:
    return Context("cuda", dev_id)


def context(dev_type: str, dev_id: int = 0) -> Context:
    return Context(dev_type, dev_id)


class NDArray:
    """Device array: a thin owner of a torch CUDA tensor (memory only)."""

    def __init__(self, tensor: torch.Tensor):
        self._t = tensor

    @property
    def shape(self):
        return tuple(self._t.shape)

    @property
    def dtype(self) -> str:
        return str(self._t.dtype).replace("torch.", "")

    @property
    def ctx(self) -> Context:
        return Context("cuda", self._t.device.index or 0)

    context = ctx

    def asnumpy(self) -> np.ndarray:
        t = self._t.detach().cpu()
        if t.dtype == torch.bfloat16:  # numpy has no bfloat16: hand back the exact values as float32
            t = t.to(torch.float32)
        return t.numpy()

    numpy = asnumpy

    def copyfrom(self, source) -> "NDArray":
        src = source._t if isinstance(source, NDArray) else torch.as_tensor(np.asarray(source))
        if tuple(src.shape) != self.shape:
            raise ValueError(f"array shape do not match the shape of NDArray {src.shape} vs "
                             f"{self.shape}")
        self._t.copy_(src.to(self._t.dtype))
        return self

    def to_dlpack(self):
        return torch.utils.dlpack.to_dlpack(self._t)

    def __dlpack__(self, stream=None):
        return self._t.__dlpack__(stream=stream)

    def __dlpack_device__(self):
        return self._t.__dlpack_device__()

    def torch(self) -> torch.Tensor:
        return self._t

    def __repr__(self):
        return f"NDArray(shape={self.shape}, dtype={self.dtype}, ctx={self.ctx})"


def array(arr, ctx: Context | None = None) -> NDArray:
    """`tvm.nd.array(np_array, ctx)`."""
    ctx = ctx or gpu(0)
    a = np.ascontiguousarray(arr)
    if str(a.dtype) not in _NP_TO_TORCH:
        raise _lib.AmosbError(_lib.AMOSB_ERR_ARG, f"unsupported dtype {a.dtype}")
    t = torch.from_numpy(a).to(f"cuda:{ctx.device_id}")
    return NDArray(t)


def empty(shape, dtype: str = "float32", ctx: Context | None = None) -> NDArray:
    ctx = ctx or gpu(0)
    return NDArray(torch.empty(tuple(shape), dtype=_NP_TO_TORCH[dtype],
                               device=f"cuda:{ctx.device_id}"))


def from_dlpack(capsule_or_obj) -> NDArray:
    return NDArray(torch.utils.dlpack.from_dlpack(capsule_or_obj))


def _as_torch(x) -> torch.Tensor:
    if isinstance(x, NDArray):
        return x._t
    if isinstance(x, torch.Tensor):
        return x
    if hasattr(x, "__dlpack__") or type(x).__name__ == "PyCapsule":
        return torch.utils.dlpack.from_dlpack(x)
    raise TypeError(f"cannot pass {type(x)} to a built module; give NDArray, torch.Tensor, a DLPack "
                    "object, or numpy arrays for every argument (host path)")


class BenchmarkResult:
    """`.mean` (seconds) and `.results` like the reference's time_evaluator result."""

    def __init__(self, results: Sequence[float]):
        self.results = tuple(results)
        self.mean = float(np.mean(self.results))
        self.std = float(np.std(self.results))

    def __repr__(self):
        return f"BenchmarkResult(mean={self.mean}, results={self.results})"


class _DeviceSource:
    """`Module.imported_modules[0]`: the device-side part; `get_source()` returns the CUDA
    source of the kernel the plan uses (the reference returns the generated CUDA C there)."""

    def __init__(self, plan_text: str):
        self._plan = plan_text

    def get_source(self, fmt: str = "") -> str:
        import os
        here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
        parts = [f"// {self._plan}\n"]
        names = ["ptx.cuh", "umma_kernel.cuh"]  # the pair kernel builds on the single-CTA file
        if "umma_pair" in self._plan:
            names.append("umma_pair_kernel.cuh")
        if "conv_prepack" in self._plan:
            names.append("launch.cu")  # the re-layout kernels live beside the launchers
        for name in names:
            path = os.path.join(here, name)
            if os.path.exists(path):
                with open(path) as f:
                    parts.append(f"// ---- {name}\n" + f.read())
        return "\n".join(parts)


class Module:
    """Callable built operator.  `module(*inputs, *outputs)`: inputs in `dag.get_inputs()` order,
    outputs last and written in place; returns None; asynchronous on the current stream."""

    entry_name = "__tvm_main__"
    type_key = "amosb"

    def __init__(self, desc: _lib.AmosbOpDesc, n_inputs: int | None = None, n_outputs: int = 1):
        _lib.load()  # fail loudly now if the native library is missing
        self.desc = desc
        self.n_inputs = desc.n_inputs if n_inputs is None else n_inputs
        self.n_outputs = n_outputs
        self.launches_per_call = 0
        self._calls: dict = {}  # prepared calls by buffer addresses (small cache)
        self.imported_modules = [_DeviceSource(_lib.describe_plan(desc))]

    # -------------------------------------------------------------------------------- calls
    def __call__(self, *args):
        if len(args) != self.n_inputs + self.n_outputs:
            raise TVMError(_lib.AMOSB_ERR_ARG,
                           f"num_args should be {self.n_inputs + self.n_outputs}, got {len(args)}")
        if all(isinstance(a, np.ndarray) for a in args):
            return self._call_host(args)
        tensors = [_as_torch(a) for a in args]
        self.launches_per_call = self._prepared(tensors).run()
        return None

    def _prepared(self, tensors) -> "device.PreparedCall":
        key = tuple((t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype) for t in tensors)
        call = self._calls.get(key)
        if call is None:
            if len(self._calls) >= 16:
                self._calls.clear()
            call = device.PreparedCall(self.desc, tensors[: self.n_inputs],
                                       tensors[self.n_inputs:])
            self._calls[key] = call
        return call

    def _call_host(self, arrays: Sequence[np.ndarray], dev: int | None = None):
        """Host-buffer path: numpy arrays in, result written into the numpy output array; the
        library does the host<->device copies (amosb_run_host) on the current CUDA device."""
        lib = _lib.load()
        if dev is None:
            dev = torch.cuda.current_device()
        keep = []
        structs = []
        for a in arrays:
            if not a.flags["C_CONTIGUOUS"]:
                raise TVMError(_lib.AMOSB_ERR_ARG, "strides: expected to be compact array")
            code = _lib.DTYPE_CODES.get(str(a.dtype))
            if code is None:
                raise TVMError(_lib.AMOSB_ERR_ARG, f"unsupported dtype {a.dtype}")
            t, k = _lib.make_tensor(a.ctypes.data, 0, code, list(a.shape))
            structs.append(t)
            keep.append(k)
        ins = (_lib.AmosbTensor * self.n_inputs)(*structs[: self.n_inputs])
        outs = (_lib.AmosbTensor * self.n_outputs)(*structs[self.n_inputs:])
        rc = lib.amosb_run_host(ctypes.byref(self.desc), ins, self.n_inputs, outs, self.n_outputs,
                                dev)
        _lib.check(rc)
        self.launches_per_call = lib.amosb_last_launch_count()
        return None

    def get_function(self, name: str):
        if name not in (self.entry_name, "main", "default_function"):
            raise AttributeError(f"Module has no function '{name}'")
        return self

    def __getitem__(self, name: str):
        return self.get_function(name)

    # ------------------------------------------------------------------------------- timing
    def time_evaluator(self, func_name: str, ctx: Context, number: int = 10, repeat: int = 1,
                       min_repeat_ms: int = 0, f_preproc: str = ""):
        """Same contract as the reference: each of `repeat` measurements runs the function
        `number` times back to back and reports the mean time of one run in seconds; `number` grows
        until one measurement lasts at least `min_repeat_ms`.  Timed with CUDA events on the
        launching stream instead of the host clock."""
        self.get_function(func_name)

        def evaluator(*args) -> BenchmarkResult:
            tensors = [_as_torch(a) for a in args]
            ins = tensors[: self.n_inputs]
            dev = ins[0].device.index or 0
            stream = torch.cuda.current_stream(dev)
            call = self._prepared(tensors)
            call.run(stream)  # warm-up, like the reference's first call
            stream.synchronize()
            results = []
            n = max(1, int(number))
            for _ in range(max(1, int(repeat))):
                while True:
                    start = torch.cuda.Event(enable_timing=True)
                    end = torch.cuda.Event(enable_timing=True)
                    start.record(stream)
                    for _ in range(n):
                        call.run(stream)
                    end.record(stream)
                    end.synchronize()
                    ms = start.elapsed_time(end)
                    if ms >= min_repeat_ms or ms <= 0:
                        break
                    n = int(max(min_repeat_ms / (ms / n) + 1, n * 1.618))
                results.append(ms / 1e3 / n)
            return BenchmarkResult(results)

        return evaluator


def to_pytorch_func(module: Module):
    """`tvm.contrib.dlpack.to_pytorch_func(f)`: torch tensors in (already accepted natively)."""

    def wrapped(*args):
        return module(*args)

    return wrapped

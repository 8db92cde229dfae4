"""Device plumbing: hand torch CUDA tensors (memory + stream only) to the C ABI.

PyTorch is used here for device allocations and the current stream; all compute happens in
libamosb.so.  There is no fallback: a CPU tensor is rejected.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from . import _lib

_TORCH_TO_CODE = {
    torch.float16: _lib.AMOSB_F16,
    torch.float32: _lib.AMOSB_F32,
    torch.int8: _lib.AMOSB_S8,
    torch.int32: _lib.AMOSB_S32,
    torch.bfloat16: _lib.AMOSB_BF16,
}
CODE_TO_TORCH = {v: k for k, v in _TORCH_TO_CODE.items()}

_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def tensor_arg(t: torch.Tensor):
    """AmosbTensor view of a torch CUDA tensor (no copy)."""
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"expected a torch.Tensor, got {type(t)}")
    if t.device.type != "cuda":
        raise _lib.AmosbError(_lib.AMOSB_ERR_ARG,
                              "Argument device_type is expected to be cuda; this path has no CPU "
                              "implementation")
    if t.dtype not in _TORCH_TO_CODE:
        raise _lib.AmosbError(_lib.AMOSB_ERR_ARG, f"unsupported dtype {t.dtype}")
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    return _lib.make_tensor(t.data_ptr(), dev, _TORCH_TO_CODE[t.dtype], list(t.shape),
                            list(t.stride()))


def get_workspace(nbytes: int, device: int) -> torch.Tensor | None:
    """Cached per-device scratch buffer with at least `nbytes` behind its first 1024-byte boundary.
    One buffer per device serves every Module and PreparedCall that does not bring its own: calls
    that use scratch (NCHW conv2d) must be stream-ordered on a device, or pass `workspace=`."""
    if nbytes <= 0:
        return None
    key = (device, 0)
    buf = _workspaces.get(key)
    # what counts is the length from the first 1024-byte boundary on (the caching allocator hands
    # out 512-byte multiples, and PreparedCall rounds the base up)
    if buf is None or buf.numel() - (-buf.data_ptr() % 1024) < nbytes:
        buf = torch.empty(nbytes + 1024, dtype=torch.uint8, device=f"cuda:{device}")
        _workspaces[key] = buf
    return buf


class PreparedCall:
    """One operator call with its argument structures built once: `run()` is a single C call.

    Building the ctypes views of the tensors costs tens of microseconds in Python, more than some
    of the kernels take; callers that repeat a call on the same buffers (benchmarks, the module's
    call cache, time_evaluator) prepare once and run many times.  The tensors are kept alive."""

    def __init__(self, desc: _lib.AmosbOpDesc, inputs: Sequence[torch.Tensor],
                 outputs: Sequence[torch.Tensor], stream: torch.cuda.Stream | None = None,
                 workspace: torch.Tensor | None = None):
        self._lib = _lib.load()
        self.desc = desc.copy()
        self._keep = [list(inputs), list(outputs)]
        self._ins = (_lib.AmosbTensor * len(inputs))()
        for i, t in enumerate(inputs):
            self._ins[i], k = tensor_arg(t)
            self._keep.append(k)
        self._outs = (_lib.AmosbTensor * len(outputs))()
        for i, t in enumerate(outputs):
            self._outs[i], k = tensor_arg(t)
            self._keep.append(k)
        self._n_in, self._n_out = len(inputs), len(outputs)
        dev = self._ins[0].device_id
        self.device = dev
        ws_bytes = _lib.workspace_bytes(self.desc)
        self._ws_ptr, self._ws_len = None, 0
        if ws_bytes > 0:
            if workspace is None:
                workspace = get_workspace(ws_bytes, dev)
            base = workspace.data_ptr()
            aligned = (base + 1023) // 1024 * 1024
            self._ws_ptr = ctypes.c_void_p(aligned)
            self._ws_len = workspace.numel() * workspace.element_size() - (aligned - base)
            self._keep.append(workspace)
        self._stream = stream
        self._desc_ref = ctypes.byref(self.desc)

    def run(self, stream: torch.cuda.Stream | None = None) -> int:
        st = stream or self._stream or torch.cuda.current_stream(self.device)
        rc = self._lib.amosb_run(self._desc_ref, self._ins, self._n_in, self._outs, self._n_out,
                                 self._ws_ptr, self._ws_len, st.cuda_stream)
        if rc < 0:
            _lib.check(rc)
        return self._lib.amosb_last_launch_count()


def run(desc: _lib.AmosbOpDesc, inputs: Sequence[torch.Tensor], outputs: Sequence[torch.Tensor],
        stream: torch.cuda.Stream | None = None, workspace: torch.Tensor | None = None) -> int:
    """Enqueue the operator on `stream` (default: torch's current stream of the tensors' device).
    Returns the number of kernels launched."""
    return PreparedCall(desc, inputs, outputs, stream, workspace).run()


def sync_check(device: int = 0) -> None:
    """Synchronise `device`; raise AmosbError(-4) if a kernel gave up a bounded wait since the last
    check (its results are then not valid)."""
    _lib.check(_lib.load().amosb_sync_check(device))


def status_peek(device: int = 0, clear: bool = True) -> int:
    """Synchronise `device` and return its device-side status word (0 = no wait ran out)."""
    return _lib.check(_lib.load().amosb_status_peek(device, 1 if clear else 0))

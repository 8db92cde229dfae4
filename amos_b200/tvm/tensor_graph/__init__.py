"""`tvm.tensor_graph`: only the auto-tensorize dispatcher contract
(reference: python/tvm/tensor_graph/core/auto_schedule/auto_schedule.py:92-105, 351-433)."""
from ...dispatch import AutoTensorizeContext, auto_tensorize_cuda  # noqa: F401

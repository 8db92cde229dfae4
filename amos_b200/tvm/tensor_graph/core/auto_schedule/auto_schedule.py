"""Same module path as the reference's dispatcher
(python/tvm/tensor_graph/core/auto_schedule/auto_schedule.py)."""
from .....dispatch import AutoTensorizeContext, auto_tensorize_cuda  # noqa: F401

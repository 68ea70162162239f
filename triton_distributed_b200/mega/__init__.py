"""Decode megakernel: task-graph builder (``ModelBuilder``) and the Qwen3 model on top of it
(the reference's ``mega_triton_kernel`` package)."""
from .model_builder import ModelBuilder, TASK_NAMES  # noqa: F401
from .qwen3 import Qwen3Model  # noqa: F401

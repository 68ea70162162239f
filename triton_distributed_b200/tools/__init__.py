"""Tooling: contextual autotuner, intra-kernel profiler host side."""
from .autotuner import contextual_autotune, current_config, config_space  # noqa: F401
from . import profiler  # noqa: F401

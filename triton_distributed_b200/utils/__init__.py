"""Timing, printing, comparison and profiling helpers (the reference's ``triton_dist.utils`` helper half:
``perf_func`` :274, ``dist_print`` :289, ``assert_allclose`` :870, ``bitwise_equal`` :902, ``group_profile`` :505)."""
from .timing import perf_func, L2Flusher, device_time_ms, ClockSampler  # noqa: F401
from .misc import dist_print, assert_allclose, bitwise_equal, generate_data, MyLogger  # noqa: F401
from .profile import group_profile, get_torch_prof_ctx  # noqa: F401
from .roofline import load_peaks, gemm_roofline, fused_roofline  # noqa: F401

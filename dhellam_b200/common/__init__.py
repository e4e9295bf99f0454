from .common import get_workspace, get_qkv_layout, print_rank0  # noqa: F401
from .benchmark import benchmark, benchmark_ms, benchmark_ms_ops, device_time_ms  # noqa: F401

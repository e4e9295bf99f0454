from .common import get_workspace, get_qkv_layout, print_rank0  # noqa: F401
from .benchmark import (benchmark, benchmark_dhellam, benchmark_ms, benchmark_ms_ops, benchmark_ms_ops_cp,  # noqa: F401
                        device_time_ms)
from .global_variables import GLOBAL_VARIABLES  # noqa: F401
from .template_launch import (launch_on_stream, launch_with_event, template_bwd, template_bwd_new, template_fwd,  # noqa: F401
                              template_fwd_new)

from .megatron import _add_dhellam_args, get_args, initialize_dhellam_megatron  # noqa: F401
from . import parallel_state  # noqa: F401

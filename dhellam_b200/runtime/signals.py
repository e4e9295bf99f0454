"""Device-side bounded waits and the status word.

Every spin in the kernel library (mbarrier polls, flag polls on local or peer memory) has a
clock budget; when it runs out the kernel records ``(code, site, block, expected)`` in a
status word and returns.  ``check_device_status`` turns a non-zero status into a typed
exception between steps.  The reference has no counterpart: it relies on
``--distributed-timeout-minutes`` and NCCL's asynchronous error handling
(script/run.sh:39, 135).
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_uint32, c_void_p

import torch

from .. import kernels as K


class CommTimeout(RuntimeError):
    """A device-side wait on a local or peer signal ran out of budget."""

    def __init__(self, status):
        self.code, self.where, self.block, self.extra = status.code, status.where, status.block, status.extra
        super().__init__(f"device wait gave up: code={self.code} site={self.where} block={self.block} expected={self.extra}")


def check_device_status():
    """Synchronises, reads and clears the status word; raises ``CommTimeout`` if set."""
    st = K.read_status(clear=True)
    if st.code != 0:
        raise CommTimeout(st)


def probe_flag_wait(expect: int = 1, budget_cycles: int = 200000, flag=None):
    """Runs the self-test kernel that waits for ``flag >= expect`` for at most
    ``budget_cycles`` and returns the (cleared) status word."""
    if flag is None:
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = K.proto("dh_probe_flag_wait", [c_void_p, c_uint32, c_longlong, c_void_p])
    K.check(fn(flag.data_ptr(), expect, budget_cycles, K.stream_ptr(None)), "dh_probe_flag_wait")
    return K.read_status(clear=True)

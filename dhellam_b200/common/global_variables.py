"""Process-wide blackboard with the reference's name (dhellam/common/global_variables.py:1-2).

The reference passes the step's inputs, the loss and the optimizer's loss-scale function
between its patched Megatron loop and the folded model through this dict
(megatron.patch:764-770, 786-803; dhellam/core/dsllm.py:86-106).  The engine here passes
them as arguments (``DoubleStrandEngine.run_step``, ``Env``); the dict is kept so that code
written against the reference finds the same keys, and ``Trainer`` mirrors the values
that outside code used to read: ``loss`` after every step and ``loss_scale_func``.
"""


class _Blackboard(dict):
    """A key that was never written reads as an empty dict that is kept under that key
    (what the reference's blackboard does), so ``GLOBAL_VARIABLES["x"]["y"] = 1`` works
    without set-up."""

    def __missing__(self, key):
        value = self[key] = {}
        return value


GLOBAL_VARIABLES = _Blackboard(inputs=None, loss=None, loss_scale_func=None)

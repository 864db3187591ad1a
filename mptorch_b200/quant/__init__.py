"""``mptorch_b200.quant``: drop-in for the reference's ``mptorch.quant`` package on B200 GPUs."""
from .quant_function import *  # noqa: F401,F403
from .quant_function import __all__ as _qf_all

__all__ = list(_qf_all)

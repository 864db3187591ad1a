"""``mptorch_b200.quant``: drop-in for the reference's ``mptorch.quant`` package on B200 GPUs."""
from . import functional  # noqa: F401
from .modules import *  # noqa: F401,F403
from .modules import __all__ as _mod_all
from .quant_format import *  # noqa: F401,F403
from .quant_format import __all__ as _fmt_all
from .quant_function import *  # noqa: F401,F403
from .quant_function import __all__ as _qf_all

__all__ = list(_qf_all) + list(_fmt_all) + list(_mod_all)

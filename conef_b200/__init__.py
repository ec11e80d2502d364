"""conef_b200: compressed-gradient data parallelism with contractive error feedback for B200.

Public surface::

    from conef_b200 import PowerSGDState, powerSGD_hook          # and the other states / hooks
    ddp_model.register_comm_hook(state, hook)
    from conef_b200 import get_comm_hooks                        # --grad_reducer registry
    from conef_b200.compressors import DenseCS, DenseCSHash3     # error compressors

The reference's import names are kept as thin aliases under
``conef_b200.communication`` (and a top-level ``communication`` package).
"""
from .parallel import *  # noqa: F401,F403
from .parallel import __all__ as _parallel_all
from .trainer import DataParallelTrainer

__version__ = "0.1.0"
__all__ = list(_parallel_all) + ["DataParallelTrainer"]

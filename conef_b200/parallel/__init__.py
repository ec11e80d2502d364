"""Data-parallel gradient compression: states, hooks, plans, engines, registry."""
from .hooks import (C2CS_hook_v2, RandomBlock_hook, UnbiasedMtrx_hook, UnbiasedRandomBlock_hook,
                    allreduce_fut, batched_powerSGD_hook, hpowerSGD_hook, powerSGD_hook)
from .registry import REDUCERS, build_state_and_hook, get_comm_hooks
from .states import (PowerSGDState, RandomBlockState, UnbiasedRandomBlockState, hPowerSGDState,
                     unbiasedMtrxState)

__all__ = ["PowerSGDState", "hPowerSGDState", "RandomBlockState", "UnbiasedRandomBlockState",
           "unbiasedMtrxState", "powerSGD_hook", "batched_powerSGD_hook", "C2CS_hook_v2", "hpowerSGD_hook",
           "RandomBlock_hook", "UnbiasedRandomBlock_hook", "UnbiasedMtrx_hook", "allreduce_fut",
           "get_comm_hooks", "build_state_and_hook", "REDUCERS"]

"""Alias module: same names as the reference's ``communication/hPowerSGD_hook.py``."""
from ..ops.reference import topk_keep_ as _topk  # noqa: F401
from ..parallel.hooks import hpowerSGD_hook  # noqa: F401
from ..parallel.states import hPowerSGDState  # noqa: F401

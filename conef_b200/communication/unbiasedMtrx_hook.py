"""Alias module: same names as the reference's ``communication/unbiasedMtrx_hook.py``."""
from ..parallel.hooks import UnbiasedMtrx_hook  # noqa: F401
from ..parallel.states import unbiasedMtrxState  # noqa: F401

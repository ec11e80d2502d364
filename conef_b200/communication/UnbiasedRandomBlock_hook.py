"""Alias module: same names as the reference's ``communication/UnbiasedRandomBlock_hook.py``."""
from ..parallel.hooks import UnbiasedRandomBlock_hook  # noqa: F401
from ..parallel.states import UnbiasedRandomBlockState  # noqa: F401

"""Alias module: same names as the reference's ``communication/RandomBlock_hook.py``."""
from ..parallel.hooks import RandomBlock_hook  # noqa: F401
from ..parallel.states import RandomBlockState  # noqa: F401

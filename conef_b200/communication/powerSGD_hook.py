"""Alias module: same names as the reference's ``communication/powerSGD_hook.py``."""
from ..ops.reference import gram_schmidt_ref as _orthogonalize, should_compress as _should_compress  # noqa: F401
from ..parallel.hooks import (C2CS_hook_v2, _report_compression_stats, batched_powerSGD_hook,  # noqa: F401
                              powerSGD_hook)
from ..parallel.states import PowerSGDState  # noqa: F401

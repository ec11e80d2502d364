"""Top-level ``communication`` package: lets scripts written against the reference
(``import communication.powerSGD_hook as powerSGD``) run unchanged on conef_b200."""
import sys as _sys

from conef_b200 import communication as _impl
from conef_b200.communication import (RandomBlock_hook, UnbiasedRandomBlock_hook, compressors,  # noqa: F401
                                      hPowerSGD_hook, powerSGD_hook, unbiasedMtrx_hook)
from conef_b200.communication.compressors import CountSketch, CountSketchHash3, halfCountSketch  # noqa: F401

for _name in ("powerSGD_hook", "hPowerSGD_hook", "RandomBlock_hook", "UnbiasedRandomBlock_hook",
              "unbiasedMtrx_hook", "compressors"):
    _sys.modules[f"communication.{_name}"] = getattr(_impl, _name)
for _name in ("CountSketch", "CountSketchHash3", "halfCountSketch"):
    _sys.modules[f"communication.compressors.{_name}"] = getattr(_impl.compressors, _name)

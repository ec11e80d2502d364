"""Minimal stand-in for ``pynvrtc`` (not installed in this image): ``pynvrtc.compiler.Program``."""
from . import compiler  # noqa: F401

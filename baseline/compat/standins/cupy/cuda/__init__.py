from . import device, function  # noqa: F401

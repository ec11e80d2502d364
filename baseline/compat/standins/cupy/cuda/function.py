"""``cupy.cuda.function.Module`` / ``Function`` on the CUDA driver API (cuda-python).

``Module().load(ptx_bytes)`` hands the PTX to ``cuModuleLoadData`` (the driver JIT-compiles it for
the current device); ``get_function(name)`` returns a callable with CuPy's launch signature
``f(grid, block, args, shared_mem, stream=obj_with_ptr)``.  As in CuPy, a Python ``int`` argument
is passed as a 64-bit integer and a ``float`` as a double; the driver copies as many bytes as
the kernel's parameter declares, so 32-bit ``int`` parameters read the low word.
"""
import numpy as np
import torch

try:
    from cuda.bindings import driver
except ImportError:  # older cuda-python layout
    from cuda import cuda as driver


def _check(res, what):
    if int(res[0]) != 0:
        raise RuntimeError(f"{what} failed with {res[0]}")
    return res[1] if len(res) > 1 else None


class Function:
    def __init__(self, module, name):
        self.module = module
        self._func = _check(driver.cuModuleGetFunction(module._module, name.encode()), "cuModuleGetFunction")

    def __call__(self, grid, block, args, shared_mem=0, stream=None):
        packed = []
        for a in args:
            if isinstance(a, bool):
                packed.append(np.array([a], dtype=np.bool_))
            elif isinstance(a, int):
                packed.append(np.array([a], dtype=np.int64))
            elif isinstance(a, float):
                packed.append(np.array([a], dtype=np.float64))
            elif isinstance(a, np.generic) or isinstance(a, np.ndarray):
                packed.append(np.asarray(a).reshape(1))
            elif torch.is_tensor(a):
                packed.append(np.array([a.data_ptr()], dtype=np.uint64))
            else:
                raise TypeError(f"unsupported kernel argument {type(a)}")
        ptrs = np.array([p.ctypes.data for p in packed], dtype=np.uint64)
        grid = tuple(grid) + (1,) * (3 - len(grid))
        block = tuple(block) + (1,) * (3 - len(block))
        strm = 0 if stream is None else int(getattr(stream, "ptr", stream))
        _check(driver.cuLaunchKernel(self._func, *grid, *block, int(shared_mem), strm, ptrs.ctypes.data, 0),
               "cuLaunchKernel")


class Module:
    def __init__(self):
        self._module = None
        self._image = None

    def load(self, image: bytes):
        torch.cuda.init()
        torch.zeros(1, device="cuda")          # the primary context must exist and be current
        if not image.endswith(b"\0"):
            image = image + b"\0"               # PTX text is read as a C string
        self._image = np.frombuffer(image, dtype=np.uint8)
        self._module = _check(driver.cuModuleLoadData(self._image.ctypes.data), "cuModuleLoadData")

    def get_function(self, name: str) -> Function:
        return Function(self, name)

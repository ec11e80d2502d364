"""Run-time compilation of a CUDA source string into a launchable kernel.

Same call shape as the reference's ``cupyKernel`` (``communication/compressors/cupy_kernel.py:10-45``,
which needs CuPy and pynvrtc): ``JitKernel(src, "name")(grid, block, args, strm, smem)``.
Here NVRTC and the CUDA driver API are reached through the ``cuda-python`` bindings, the target
is the current device's architecture (``sm_100a`` on B200, real SASS rather than PTX), and the
kernel is launched on the given stream (by default PyTorch's current stream).

The library's own kernels are compiled ahead of time (``csrc/``); this loader is for users who
bring their own error-compressor kernels as source strings, as the reference's sketches do.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np
import torch


def _bindings():
    try:
        from cuda.bindings import driver, nvrtc
    except ImportError:  # older cuda-python layout
        from cuda import cuda as driver, nvrtc
    return driver, nvrtc


def _check(res, what):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"{what} failed with {err}")
    return res[1:] if len(res) > 2 else (res[1] if len(res) == 2 else None)


class JitKernel:
    def __init__(self, kernel_src: str, func_name: str, options: Sequence[str] = ()):
        self.src, self.name, self.options = kernel_src, func_name, tuple(options)
        self._func = None
        self._module = None

    @staticmethod
    def compute_arch(device: Optional[int] = None) -> str:
        major, minor = torch.cuda.get_device_capability(device)
        suffix = "a" if major >= 9 else ""      # architecture-specific features (tcgen05, TMA) need the 'a' target
        return f"sm_{major}{minor}{suffix}"

    def compile(self) -> None:
        driver, nvrtc = _bindings()
        torch.cuda.init()
        torch.zeros(1, device="cuda")            # make sure the primary context exists
        prog = _check(nvrtc.nvrtcCreateProgram(self.src.encode(), f"{self.name}.cu".encode(), 0, [], []), "nvrtcCreateProgram")
        opts = [f"--gpu-architecture={self.compute_arch()}".encode(), b"--std=c++17", *[o.encode() for o in self.options]]
        res = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
        if int(res[0]) != 0:
            size = _check(nvrtc.nvrtcGetProgramLogSize(prog), "nvrtcGetProgramLogSize")
            log = b" " * size
            nvrtc.nvrtcGetProgramLog(prog, log)
            raise RuntimeError("NVRTC compilation failed:\n" + log.decode(errors="replace"))
        size = _check(nvrtc.nvrtcGetCUBINSize(prog), "nvrtcGetCUBINSize")
        image = b" " * size
        _check(nvrtc.nvrtcGetCUBIN(prog, image), "nvrtcGetCUBIN")
        self._module = _check(driver.cuModuleLoadData(np.char.array(image).ctypes.data), "cuModuleLoadData")
        self._func = _check(driver.cuModuleGetFunction(self._module, self.name.encode()), "cuModuleGetFunction")

    def __call__(self, grid, block, args, strm=None, smem: int = 0) -> None:
        """``args``: device pointers (ints or tensors) and Python / NumPy scalars, in kernel order."""
        driver, _ = _bindings()
        if self._func is None:
            self.compile()
        if strm is None:
            strm = torch.cuda.current_stream().cuda_stream
        packed = []
        for a in args:
            if torch.is_tensor(a):
                packed.append(np.array([a.data_ptr()], dtype=np.uint64))
            elif isinstance(a, bool):
                packed.append(np.array([a], dtype=np.int32))
            elif isinstance(a, int):
                # plain ints are device addresses when they look like pointers, else 32-bit integers
                packed.append(np.array([a], dtype=np.uint64 if a > 0xFFFFFFFF else np.int32))
            elif isinstance(a, float):
                packed.append(np.array([a], dtype=np.float32))
            else:
                packed.append(np.asarray(a).reshape(1))
        ptrs = np.array([p.ctypes.data for p in packed], dtype=np.uint64)
        grid = tuple(grid) + (1,) * (3 - len(grid))
        block = tuple(block) + (1,) * (3 - len(block))
        if smem > 48 * 1024:
            _check(driver.cuFuncSetAttribute(
                self._func, driver.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, int(smem)),
                "cuFuncSetAttribute")
        _check(driver.cuLaunchKernel(self._func, *grid, *block, int(smem), int(strm), ptrs.ctypes.data, 0), "cuLaunchKernel")


cupyKernel = JitKernel

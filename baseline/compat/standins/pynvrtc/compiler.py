"""``Program(src, name).compile(options) -> PTX text`` on cuda-python's NVRTC binding: the call
shape used by ``communication/compressors/cupy_kernel.py:20-27`` of the reference."""
try:
    from cuda.bindings import nvrtc
except ImportError:  # older cuda-python layout
    from cuda import nvrtc


class ProgramException(Exception):
    pass


class Program:
    def __init__(self, src, name="default_program", headers=(), include_names=()):
        self._src = src if isinstance(src, bytes) else src.encode()
        self._name = name if isinstance(name, bytes) else name.encode()

    def compile(self, options=()):
        err, prog = nvrtc.nvrtcCreateProgram(self._src, self._name, 0, [], [])
        if int(err) != 0:
            raise ProgramException(f"nvrtcCreateProgram: {err}")
        opts = [o if isinstance(o, bytes) else o.encode() for o in options]
        (err,) = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
        if int(err) != 0:
            _, size = nvrtc.nvrtcGetProgramLogSize(prog)
            log = b" " * size
            nvrtc.nvrtcGetProgramLog(prog, log)
            raise ProgramException(log.decode(errors="replace"))
        _, size = nvrtc.nvrtcGetPTXSize(prog)
        ptx = b" " * size
        (err,) = nvrtc.nvrtcGetPTX(prog, ptx)
        if int(err) != 0:
            raise ProgramException(f"nvrtcGetPTX: {err}")
        nvrtc.nvrtcDestroyProgram(prog)
        return ptx.rstrip(b"\0").decode()

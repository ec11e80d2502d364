"""In-tree build of the native library for sm_100a.

``python -m conef_b200.ops.build`` compiles every ``csrc/*.cu`` with nvcc into
``conef_b200/ops/_conef_native.so`` (one shared object, plain C ABI, bound with
ctypes).  The build is a cross-compile: no GPU is needed.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "_conef_native.so"
OBJ_DIR = HERE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("CONEF_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set CONEF_NVCC")


def sources():
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_fresh() -> bool:
    stamp = OBJ_DIR / "digest.txt"
    return OUT.exists() and stamp.exists() and stamp.read_text() == _digest()


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile and link; returns the path of the shared object."""
    if not force and is_fresh():
        return OUT
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    flags = list(NVCC_FLAGS)
    if ptxas_info:
        flags += ["-Xptxas", "-v"]

    def compile_one(src: Path):
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, obj, res

    objs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        for src, obj, res in pool.map(compile_one, sources()):
            if verbose or ptxas_info or res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")
            objs.append(str(obj))
    tmp = OUT.with_suffix(".so.tmp")         # link aside, then rename: readers never see a half-written library
    link = [nvcc, "-shared", "-o", str(tmp), *objs, "-lcudart"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link failed")
    os.replace(tmp, OUT)
    (OBJ_DIR / "digest.txt").write_text(_digest())
    return OUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)

"""Makes the unmodified reference importable: paths, stand-ins and the two module aliases."""
import importlib
import importlib.util
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BASELINE = os.path.dirname(HERE)
REF = os.path.join(BASELINE, "_ref")


def ensure_reference_copy(source=None):
    """``baseline/_ref`` holds a byte-identical copy of the reference tree (it is not tracked by
    git).  When it is missing and the reference checkout is present, copy it."""
    if os.path.isdir(os.path.join(REF, "communication")):
        return REF
    # default: a checkout named `reference` beside this repository
    source = source or os.environ.get("CONEF_REFERENCE_SRC") or os.path.join(os.path.dirname(os.path.dirname(BASELINE)), "reference")
    if not os.path.isdir(os.path.join(source, "communication")):
        raise FileNotFoundError("no copy of the reference under baseline/_ref and no checkout to copy from")
    os.makedirs(REF, exist_ok=True)
    for name in ("communication", "examples"):
        shutil.copytree(os.path.join(source, name), os.path.join(REF, name), dirs_exist_ok=True)
    return REF


def install():
    """Returns the directory of the reference copy after putting it, and whatever it imports, in reach."""
    ref = ensure_reference_copy()
    if importlib.util.find_spec("cupy") is None or importlib.util.find_spec("pynvrtc") is None:
        standins = os.path.join(HERE, "standins")
        if standins not in sys.path:
            sys.path.insert(0, standins)
    if ref not in sys.path:
        sys.path.insert(0, ref)
    # A regular package named `communication` anywhere on the path would win over the reference's
    # directory, which has no __init__.py: refuse to run anything but the reference's files.
    spec = importlib.util.find_spec("communication.powerSGD_hook")
    if spec is None or not os.path.abspath(spec.origin).startswith(os.path.abspath(ref) + os.sep):
        raise ImportError(f"`communication` resolves to {getattr(spec, 'origin', None)}, not to the reference copy; "
                          "remove the shadowing directory from sys.path")
    # communication/powerSGD_hook.py:8 does `from . import default_hooks`, a file the published tree
    # lacks: it is torch's own module of that name.
    from torch.distributed.algorithms.ddp_comm_hooks import default_hooks
    sys.modules.setdefault("communication.default_hooks", default_hooks)
    # communication/powerSGD_hook.py:9 does `from compressors.CountSketch import DenseCS`: the
    # package lives at communication/compressors.
    compressors = importlib.import_module("communication.compressors")
    sys.modules.setdefault("compressors", compressors)
    sys.modules.setdefault("compressors.CountSketch", importlib.import_module("communication.compressors.CountSketch"))
    return ref

"""ctypes binding of the in-tree native library (``_conef_native.so``).

The library is built by :mod:`conef_b200.ops.build` (``__graft_entry__.build``)
and lives next to this file.  On a machine with a CUDA device the library is
mandatory: :func:`lib` raises instead of silently falling back to PyTorch ops.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Optional

import numpy as np
import torch

_SO = Path(__file__).resolve().parent / "_conef_native.so"
_lib = None

c_ll = C.c_longlong
vp = C.c_void_p


class NativeError(RuntimeError):
    pass


# numpy dtypes mirroring the C structs of csrc/conef.h ---------------------
MAT_DTYPE = np.dtype(
    [("g_off", "<i8"), ("p_off", "<i8"), ("q_off", "<i8"), ("sk_off", "<i8"),
     ("n", "<i4"), ("m", "<i4"), ("r", "<i4"), ("W", "<i4"),
     ("tab_off", "<i4"), ("cnt_off", "<i4"), ("q_rows", "<i4"), ("q_atomic", "<i4"),
     ("src", "<i4"), ("Wp", "<i4"), ("qpk_off", "<i8"), ("ppk_off", "<i8"),
     ("ppk_fold_off", "<i8"), ("fold", "<i4"), ("cb_off", "<i4")], align=True)
SEG_DTYPE = np.dtype([("src_off", "<i8"), ("dst_off", "<i8"), ("len", "<i8")], align=True)
BLK_DTYPE = np.dtype(
    [("g_off", "<i8"), ("numel", "<i8"), ("start", "<i8"), ("block", "<i8"),
     ("stage_off", "<i8"), ("sk_off", "<i8"),
     ("n", "<i4"), ("m", "<i4"), ("W", "<i4"), ("tab_off", "<i4"), ("cnt_off", "<i4"),
     ("scale_off", "<i4"), ("cb_off", "<i4"), ("pad_", "<i4")], align=True)
LAMB_DTYPE = np.dtype(
    [("p", "<u8"), ("g", "<u8"), ("m", "<u8"), ("v", "<u8"), ("numel", "<i8"),
     ("weight_decay", "<f4"), ("pad", "<i4")], align=True)
CORR_DTYPE = np.dtype([("t_off", "<i8"), ("x_off", "<i8", (2,)), ("l_off", "<i8", (2,)), ("r_off", "<i8", (2,)),
                       ("rows_t", "<i4"), ("rows_l", "<i4"), ("c1", "<i4"), ("nterms", "<i4"),
                       ("c2", "<i4", (2,))], align=True)
assert CORR_DTYPE.itemsize == 80
assert MAT_DTYPE.itemsize == 104 and SEG_DTYPE.itemsize == 24 and BLK_DTYPE.itemsize == 80
assert LAMB_DTYPE.itemsize == 48

EF_NONE, EF_DENSE, EF_SKETCH, EF_QUANT8 = 0, 1, 2, 3
PHASE_P, PHASE_Q, PHASE_D, PHASE_ALL = 1, 2, 4, 7


class TileList(C.Structure):
    """Mirror of ``ConefTileList`` (csrc/executor.h)."""
    _fields_ = [("tiles", C.c_void_p), ("n", C.c_int), ("pad", C.c_int)]


class QSet(C.Structure):
    _fields_ = [("tc", TileList), ("simt", TileList)]


class PsgdPlan(C.Structure):
    """Mirror of ``ConefPsgdPlan`` (csrc/executor.h): field order and types must match."""
    _fields_ = [
        ("mats", C.c_void_p),
        ("nrec", C.c_int), ("nm", C.c_int), ("max_rank", C.c_int), ("np_cols", C.c_int), ("max_cols", C.c_int),
        ("unbiased", C.c_int), ("ef_mode", C.c_int), ("lowrank", C.c_int),
        ("use_tc", C.c_int), ("p_zero", C.c_int), ("q_zero", C.c_int),
        ("tables", C.c_void_p), ("counts", C.c_void_p), ("sketch", C.c_void_p), ("dense_err", C.c_void_p),
        ("aux", C.c_void_p),
        ("qz", C.c_void_p), ("total_q", C.c_longlong), ("total_z", C.c_longlong),
        ("pu", C.c_void_p), ("total_p", C.c_longlong), ("total_u", C.c_longlong),
        ("u_old", C.c_void_p), ("qz2", C.c_void_p), ("qpk", C.c_void_p), ("ppk", C.c_void_p),
        ("segs", C.c_void_p), ("nsegs", C.c_int), ("orth_max_rows", C.c_int), ("total_unc", C.c_longlong),
        ("staging", C.c_void_p), ("tc_maps", C.c_void_p),
        ("tc_p", TileList), ("simt_p", TileList),
        ("qset_all", QSet), ("qset_grad", QSet), ("qset_err", QSet),
        ("d_tiles", TileList), ("d_rows", C.c_int), ("d_nblk", C.c_int), ("d_smem", C.c_size_t),
        ("orth_q", TileList), ("orth_p", TileList), ("orth_u", TileList),
        ("chunks_n", TileList), ("chunks_m", TileList),
        ("gram", C.c_void_p), ("cbuf", C.c_void_p),
        ("corr_p", C.c_void_p), ("corr_q", C.c_void_p), ("corr_u", C.c_void_p), ("corr_v", C.c_void_p),
        ("status", C.c_void_p),
        ("world", C.c_int), ("rank", C.c_int), ("has_symm", C.c_int), ("d_rbu", C.c_int),
        ("peer_flags", C.c_void_p), ("my_flags", C.c_void_p),
        ("peer_stage", C.c_void_p * 2), ("peer_p", C.c_void_p * 2), ("peer_q", C.c_void_p * 2),
        ("local_stage", C.c_void_p * 2), ("local_p", C.c_void_p * 2), ("local_q", C.c_void_p * 2),
        ("spin_limit", C.c_longlong),
        ("work", C.c_void_p), ("slot", C.c_int), ("fresh", C.c_int), ("seed", C.c_ulonglong),
        ("epoch", C.c_uint), ("alpha", C.c_float), ("beta", C.c_float), ("eps", C.c_float),
        ("launched", C.c_int),
        ("use_graph", C.c_int), ("epoch_word", C.c_void_p), ("epoch_shadow", C.c_uint),
        ("graph_runs", C.c_int * 2), ("graph_exec", C.c_void_p * 2), ("graph_launched", C.c_int * 2),
        ("graph_ncoll", C.c_int * 2), ("key_work", C.c_void_p),
        ("key_alpha", C.c_float), ("key_beta", C.c_float), ("key_eps", C.c_float),
        ("graph_replays", C.c_int),
        ("topk", C.c_int), ("topk_ratio", C.c_float), ("topk_tiles", TileList), ("topk_scratch", C.c_void_p),
        ("fused", C.c_int), ("has_slots", C.c_int), ("done_word", C.c_void_p),
        ("zpk", C.c_void_p), ("zpk_n", C.c_longlong),
        ("one_launch_orth", C.c_int), ("wait_kernel", C.c_int),
        ("orth_rows_q", C.c_int), ("orth_rows_p", C.c_int), ("orth_rows_u", C.c_int), ("pad3", C.c_int),
    ]

class OrthExtra(C.Structure):
    """Mirror of ``ConefOrthExtra`` (csrc/conef.h)."""
    _fields_ = [
        ("zero0", C.c_void_p), ("zero0_n", C.c_longlong), ("zero1", C.c_void_p), ("zero1_n", C.c_longlong),
        ("seg_mode", C.c_int), ("nsegs", C.c_int), ("segs", C.c_void_p), ("seg_total", C.c_longlong),
        ("bucket", C.c_void_p), ("dense_err", C.c_void_p), ("staging", C.c_void_p), ("peer_staging", C.c_void_p),
        ("seg_scale", C.c_float),
        ("alpha", C.c_float), ("nm", C.c_int), ("tables", C.c_void_p),
        ("bar", C.c_void_p), ("max_rank", C.c_int),
        ("cl_nmat", C.c_int), ("cl_list", C.c_void_p), ("cl_max_rows", C.c_int), ("pad_", C.c_int),
    ]


class RandblockPlan(C.Structure):
    """Mirror of ``ConefRandblockPlan`` (csrc/executor.h): field order and types must match."""
    _fields_ = [
        ("blks", C.c_void_p), ("nblks", C.c_int), ("rows_per_cta", C.c_int),
        ("tiles", TileList),
        ("segs", C.c_void_p), ("nsegs", C.c_int), ("ef_mode", C.c_int),
        ("total_unc", C.c_longlong), ("total_block", C.c_longlong),
        ("staging_unc", C.c_void_p), ("staging_blk", C.c_void_p),
        ("sketch", C.c_void_p), ("tables", C.c_void_p), ("counts", C.c_void_p),
        ("dense_err", C.c_void_p), ("qcodes", C.c_void_p), ("qscales", C.c_void_p),
        ("smem", C.c_size_t), ("status", C.c_void_p),
        ("world", C.c_int), ("rank", C.c_int), ("has_symm", C.c_int), ("unbiased", C.c_int),
        ("peer_flags", C.c_void_p), ("my_flags", C.c_void_p),
        ("peer_unc", C.c_void_p * 2), ("peer_blk", C.c_void_p * 2),
        ("local_unc", C.c_void_p * 2), ("local_blk", C.c_void_p * 2),
        ("spin_limit", C.c_longlong),
        ("work", C.c_void_p), ("slot", C.c_int), ("nblk_tiles", C.c_int),
        ("epoch", C.c_uint), ("alpha", C.c_float), ("beta", C.c_float),
        ("launched", C.c_int),
        ("has_slots", C.c_int), ("two_shot", C.c_int),
        ("peer_red", C.c_void_p * 2), ("local_red", C.c_void_p * 2), ("done_word", C.c_void_p),
    ]


_SIGNATURES = {
    "conef_version": ([], C.c_int),
    "conef_build_hash_table": ([vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp], C.c_int),
    "conef_sketch_query": ([vp, vp, C.c_int, vp, C.c_int, C.c_int, C.c_int, C.c_float, vp], C.c_int),
    "conef_sketch_update": ([vp, vp, C.c_int, vp, vp, C.c_int, C.c_int, C.c_int, C.c_float, vp], C.c_int),
    "conef_sketch3_query": ([vp] * 7 + [C.c_int, C.c_int, C.c_int, C.c_float, vp], C.c_int),
    "conef_sketch3_update": ([vp] * 7 + [C.c_int, C.c_int, C.c_int, C.c_float, vp], C.c_int),
    "conef_psgd_p": ([vp, vp, C.c_int, vp, vp, vp, vp, C.c_int, C.c_int, vp], C.c_int),
    "conef_sketch_project": ([vp, C.c_int, C.c_int, vp, vp, C.c_float, C.c_int, vp], C.c_int),
    "conef_psgd_q": ([vp, vp, C.c_int, vp, vp, vp, vp, C.c_int, vp], C.c_int),
    "conef_orthogonalize_packed": ([vp, vp, C.c_int, C.c_int, C.c_int, vp, C.c_float, vp, vp, C.c_int, C.c_uint32,
                                    vp, c_ll, vp, C.c_int, vp, vp], C.c_int),
    "conef_pack_small": ([vp, C.c_int, C.c_int, vp, vp, C.c_int, vp], C.c_int),
    "conef_psgd_decompress": ([vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp, vp, C.c_float, vp, vp, vp, vp, C.c_float,
                               C.c_float, C.c_int, C.c_int, C.c_size_t, vp, vp], C.c_int),
    "conef_fill_normal": ([vp, c_ll, C.c_uint64, vp], C.c_int),
    "conef_sgd_step": ([vp, C.c_int, vp, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, C.c_int, C.c_int, vp], C.c_int),
    "conef_colsum": ([vp, C.c_int, c_ll, C.c_int, vp, C.c_int, vp, vp], C.c_int),
    "conef_colstats": ([vp, C.c_int, c_ll, C.c_int, C.c_float, C.c_float, vp, C.c_int, vp, vp, vp, vp, vp], C.c_int),
    "conef_coldot": ([vp, vp, C.c_int, c_ll, C.c_int, vp, vp, vp, C.c_int, vp, vp, vp, vp, vp], C.c_int),
    "conef_ln_wgrad": ([vp, vp, C.c_int, c_ll, C.c_int, vp, vp, vp, C.c_int, vp, vp, vp], C.c_int),
    "conef_cast_f32_bf16": ([vp, vp, c_ll, vp], C.c_int),
    "conef_bias_add": ([vp, C.c_int, c_ll, C.c_int, vp, C.c_int, vp], C.c_int),
    "conef_bn_apply": ([vp, vp, C.c_int, c_ll, C.c_int, vp, vp, vp, vp, C.c_int, C.c_int, vp], C.c_int),
    "conef_coldot_relu": ([vp, vp, C.c_int, c_ll, C.c_int, vp, vp, vp, vp, vp, C.c_int, vp, vp, vp, vp, vp], C.c_int),
    "conef_bn_backward_apply": ([vp, vp, vp, C.c_int, c_ll, C.c_int, vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, vp],
                                C.c_int),
    "conef_lowrank_correct": ([vp, C.c_int, vp, C.c_int, vp, C.c_int, vp, vp, vp, vp, C.c_float, vp, vp, vp,
                               C.c_float, vp, vp], C.c_int),
    "conef_tc_supported": ([], C.c_int),
    "conef_tc_encode_maps": ([vp, C.c_int, vp, vp, vp, vp], C.c_int),
    "conef_psgd_tc": ([C.c_int, vp, vp, vp, C.c_int, vp, vp, C.c_int, vp, vp], C.c_int),
    "conef_psgd_tc_signal": ([C.c_int, vp, vp, vp, C.c_int, vp, vp, C.c_int, vp, vp, vp, C.c_int, C.c_int, C.c_uint32,
                              vp, vp], C.c_int),
    "conef_orthogonalize_fused": ([vp, vp, C.c_int, C.c_int, vp, C.c_float, vp, vp, C.c_int, C.c_uint32, vp, c_ll, vp,
                                   C.c_int, vp, vp, C.POINTER(OrthExtra), vp], C.c_int),
    "conef_reduce_q": ([vp, C.c_int, C.c_int, vp, vp, vp, vp, C.c_int, C.c_uint32, C.c_float, C.c_float, vp, c_ll,
                        vp, vp], C.c_int),
    "conef_orth_last_launches": ([], C.c_int),
    "conef_gather_segments": ([vp, C.c_int, vp, vp, vp, c_ll, vp], C.c_int),
    "conef_scatter_segments": ([vp, C.c_int, vp, vp, C.c_int, vp, C.c_float, vp, c_ll, vp], C.c_int),
    "conef_randblock_gather": ([vp, vp, C.c_int, C.c_int, C.c_int, vp, vp, C.c_float, vp, vp, vp, vp, vp, vp,
                                C.c_float, C.c_float, C.c_int, C.c_size_t, vp], C.c_int),
    "conef_randblock_scatter": ([vp, C.c_int, vp, vp, C.c_int, vp, C.c_float, c_ll, vp], C.c_int),
    "conef_quant8_query": ([vp, vp, vp, c_ll, C.c_float, vp], C.c_int),
    "conef_quant8_update": ([vp, vp, vp, c_ll, C.c_float, vp], C.c_int),
    "conef_signal_peers": ([vp, C.c_int, C.c_int, C.c_uint32, vp], C.c_int),
    "conef_allreduce_oneshot": ([vp, vp, vp, vp, C.c_int, C.c_int, C.c_uint32, c_ll, C.c_float, vp, c_ll, vp], C.c_int),
    "conef_wait_flags": ([vp, C.c_int, C.c_uint32, vp, c_ll, vp], C.c_int),
    "conef_ipc_get_handle": ([vp, vp], C.c_int),
    "conef_ipc_open_handle": ([vp, C.POINTER(vp)], C.c_int),
    "conef_ipc_close_handle": ([vp], C.c_int),
    "conef_psgd_run": ([C.POINTER(PsgdPlan), C.c_int, vp], C.c_int),
    "conef_topk_keep": ([vp, C.c_int, vp, C.c_int, vp, C.c_float, vp, vp], C.c_int),
    "conef_topk_chunk": ([], C.c_int),
    "conef_psgd_plan_size": ([], C.c_int),
    "conef_mat_size": ([], C.c_int),
    "conef_randblock_run": ([C.POINTER(RandblockPlan), C.c_int, vp], C.c_int),
    "conef_randblock_plan_size": ([], C.c_int),
    "conef_psgd_step": ([C.POINTER(PsgdPlan), vp], C.c_int),
    "conef_psgd_plan_release": ([C.POINTER(PsgdPlan)], C.c_int),
    "conef_epoch_word": ([vp, C.c_uint32, C.c_int, vp], C.c_int),
    "conef_lamb_step": ([vp, C.c_int, vp, C.c_int, C.c_int, vp, C.c_float, C.c_float, C.c_float, C.c_float,
                         C.c_int, C.c_int, C.c_float, C.c_float, vp], C.c_int),
    "conef_cpu_hash_table": ([vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int], None),
    "conef_cpu_sketch_query": ([vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_float], None),
    "conef_cpu_sketch_update": ([vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_float], None),
    "conef_cpu_gram_schmidt": ([vp, C.c_int, C.c_int, C.c_float], None),
}
_OPTIONAL = {}


# How many kernels one call of an entry point enqueues (memsets not counted);
# everything not listed launches exactly one.  Host-only entry points launch none.
_KERNELS_PER_CALL = {
    "conef_lamb_step": 3, "conef_orthogonalize_packed": 3, "conef_orthogonalize_fused": 3, "conef_lowrank_correct": 2, "conef_topk_keep": 7, "conef_topk_chunk": 0, "conef_orth_last_launches": 0, "conef_psgd_run": 0, "conef_psgd_plan_size": 0, "conef_mat_size": 0, "conef_randblock_run": 0, "conef_randblock_plan_size": 0, "conef_psgd_step": 0, "conef_psgd_plan_release": 0, "conef_version": 0, "conef_tc_supported": 0, "conef_tc_encode_maps": 0, "conef_last_error": 0,
    "conef_ipc_get_handle": 0, "conef_ipc_open_handle": 0, "conef_ipc_close_handle": 0,
    "conef_cpu_hash_table": 0, "conef_cpu_sketch_query": 0, "conef_cpu_sketch_update": 0,
    "conef_cpu_gram_schmidt": 0,
}
launch_count = 0  # kernels enqueued through this binding since import (see reset_launch_count)


def reset_launch_count() -> int:
    global launch_count
    old, launch_count = launch_count, 0
    return old


class _CountingLib:
    """Attribute proxy over the CDLL that counts kernel launches per call."""

    def __init__(self, handle):
        object.__setattr__(self, "_handle", handle)

    def __getattr__(self, name):
        fn = getattr(self._handle, name)
        k = _KERNELS_PER_CALL.get(name, 1)
        if k == 0:
            wrapped = fn
        else:
            def wrapped(*args, _fn=fn, _k=k):
                global launch_count
                launch_count += _k
                return _fn(*args)
        object.__setattr__(self, name, wrapped)
        return wrapped


def so_path() -> Path:
    return _SO


def available() -> bool:
    """True when the shared object exists and loads."""
    try:
        return lib() is not None
    except NativeError:
        return False


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not _SO.exists():
        raise NativeError(
            f"native library {_SO} is missing; run `python -m conef_b200.ops.build` "
            "(or __graft_entry__.build()) first")
    try:
        handle = C.CDLL(str(_SO))
    except OSError as exc:  # pragma: no cover - depends on the machine
        raise NativeError(f"cannot load {_SO}: {exc}") from exc
    handle.conef_last_error.restype = C.c_char_p
    for name, (argtypes, restype) in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.argtypes = argtypes
        fn.restype = restype
    for name, (argtypes, restype) in _OPTIONAL.items():
        if hasattr(handle, name):
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = restype
    if handle.conef_randblock_plan_size() != C.sizeof(RandblockPlan):
        raise NativeError(f"RandblockPlan mirrors {C.sizeof(RandblockPlan)} bytes, the library expects "
                          f"{handle.conef_randblock_plan_size()}: rebuild with `python -m conef_b200.ops.build`")
    if handle.conef_mat_size() != MAT_DTYPE.itemsize:
        raise NativeError(f"MAT_DTYPE mirrors {MAT_DTYPE.itemsize} bytes, the library expects "
                          f"{handle.conef_mat_size()}: rebuild with `python -m conef_b200.ops.build`")
    if handle.conef_psgd_plan_size() != C.sizeof(PsgdPlan):
        raise NativeError(f"PsgdPlan mirrors {C.sizeof(PsgdPlan)} bytes, the library expects "
                          f"{handle.conef_psgd_plan_size()}: rebuild with `python -m conef_b200.ops.build`")
    _lib = _CountingLib(handle)
    return _lib


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = lib().conef_last_error()
        raise NativeError(f"{what} failed (rc={rc}): {msg.decode() if msg else ''}")


def use_native(t: torch.Tensor) -> bool:
    """Decide the execution path for tensor ``t``.

    CUDA tensors run on the native kernels unless ``CONEF_BACKEND=torch`` asks
    for the PyTorch-ops path (the baseline arm of the benchmarks).  A CUDA
    tensor with no loadable library is an error, never a silent fallback.
    """
    if not t.is_cuda:
        return False
    if os.environ.get("CONEF_BACKEND", "native") == "torch":
        return False
    lib()  # raises if missing
    return True


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def upload_struct_array(arr: np.ndarray, device) -> torch.Tensor:
    """Copy a numpy structured array to the device as raw bytes."""
    raw = torch.from_numpy(arr.view(np.uint8).reshape(-1).copy())
    return raw.to(device)

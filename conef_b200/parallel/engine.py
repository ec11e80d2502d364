"""Native (sm_100a) execution of the hooks: per-bucket engines.

An engine is built the first time a bucket is compressed and is reused while
the bucket keeps its layout.  It owns the device-resident descriptor tables
(one ``ConefMat`` / ``ConefSeg`` / ``ConefBlk`` record per tensor, plus tile
tables), the hash-table arena, the symmetric buffers, and it rebinds the
state's persistent tensors (error buffers, sketches, P/Q memory) so that the
state keeps the reference's checkpoint layout while the kernels see flat
arenas.

Per step and bucket the PowerSGD engine makes ONE call into the native executor
(csrc/executor.cu), which enqueues, on a dedicated communication stream that waits for
the gradients and that the returned future publishes:

    Gram-Schmidt(Q) [+ gather(uncompressed), pack, project] -> P = (G+e)Q [publishes the epoch]
    -> allreduce(P)+Gram-Schmidt [+ scatter(uncompressed, reduced in-kernel)] -> Q = M^T P [publishes]
    -> allreduce(Q)/ws + un-projection -> M_hat = P Q^T + error update

with no host synchronisation and no ``.wait()`` on the host (the reference
blocks the host once per bucket, communication/powerSGD_hook.py:552-553).
"""
from __future__ import annotations

import logging
import math
import os
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..compressors import DenseCS, Quant8Error, tables_for
from ..compressors.count_sketch import block_csr_for
from ..compressors.count_sketch import HalfDenseCS
from ..ops import native
from ..ops import reference as ref
from . import plan as planlib
from .symm import DEFAULT_SPIN_LIMIT, LocalSlots, SymmBuffer, SymmUnavailable, comm_backend_choice

logger = logging.getLogger(__name__)

_COMM_STREAMS: Dict[int, "torch.cuda.Stream"] = {}
_SYMM_DISABLED = False

P_ROWS = 32         # rows per CTA of the SIMT P kernel (csrc/powersgd.cu: P_WARPS * P_WROWS)
Q_COLS = 256        # columns per CTA of the Q kernel
Q_MAX_ROWS = 1024
QGROUP = ref.QUANT_GROUP
SMEM_BUDGET = 200 * 1024
TARGET_CTAS = 2 * 148


def comm_stream_for(device: torch.device) -> "torch.cuda.Stream":
    """One high-priority side stream per device, shared by all hooks."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    s = _COMM_STREAMS.get(idx)
    if s is None:
        s = torch.cuda.Stream(device=device, priority=-1)
        _COMM_STREAMS[idx] = s
    return s


def _use_tc() -> bool:
    """tcgen05 tiles for P / Q unless ``CONEF_TC=0``."""
    if os.environ.get("CONEF_TC", "1") == "0":
        return False
    return bool(native.lib().conef_tc_supported())


def _done_on_current_stream(buf: torch.Tensor) -> torch.futures.Future:
    fut = torch.futures.Future(devices=[buf.device])
    fut.set_result(buf)
    return fut


def _try_symm(regions, group, device) -> Optional[SymmBuffer]:
    global _SYMM_DISABLED
    choice = comm_backend_choice()
    if group.size() == 1 or choice == "nccl" or _SYMM_DISABLED:
        return None
    try:
        sb = SymmBuffer(regions, group, device, backend=choice)
        logger.info("symmetric buffer (%s backend): %d bytes per rank", sb.backend, sb.total_bytes)
        return sb
    except SymmUnavailable as exc:
        if choice != "auto":
            raise
        logger.warning("peer-memory collectives unavailable, using NCCL: %s", exc)
        _SYMM_DISABLED = True
        return None


_STATUS_WORDS: Dict[int, torch.Tensor] = {}


def _status_words(device: torch.device) -> torch.Tensor:
    """One status word block per device, shared by every engine of the process: a wait that gave
    up anywhere is seen by whichever hook call looks next."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _STATUS_WORDS.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=device)
        _STATUS_WORDS[idx] = t
    return t


class _EngineBase:
    def __init__(self, device):
        self.device = device
        self.status = _status_words(device)
        self.epoch = 0
        self.step = 0
        self.symm: Optional[SymmBuffer] = None
        self.lib = native.lib()

    def check_status(self) -> None:
        code = int(self.status[0].item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(
                f"device-side wait gave up (status {code}): a peer rank did not signal in time; "
                "the gradients of the affected step are not valid")

    def _nccl_sum(self, t: torch.Tensor, group, average=False) -> None:
        if group.size() == 1 or t.numel() == 0:
            return
        if average:
            dist.all_reduce(t, op=dist.ReduceOp.AVG, group=group)
        else:
            dist.all_reduce(t, group=group)


# ==========================================================================
# PowerSGD family
# ==========================================================================
class PowerSGDEngine(_EngineBase):
    """One bucket of the PowerSGD family (layer-wise, batched, transposed-sketch, unbiased)."""

    def __init__(self, state, buf: torch.Tensor, grads, group, variant: str, bidx: int = 0):
        super().__init__(buf.device)
        self.variant = variant
        self.group = group
        self.world = group.size()
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.buf_ptr = buf.data_ptr()
        self.buf_numel = buf.numel()
        dev = self.device
        if variant == "batched":
            self.plan, self.side = planlib.build_batched_plan(buf.numel(), state.matrix_approximation_rank, dev, buf.dtype)
            self.work = torch.zeros(self.side * self.side, device=dev, dtype=torch.float32)
        else:
            self.plan = planlib.build_powersgd_plan(buf, grads, state.matrix_approximation_rank,
                                                    state.min_compression_rate)
            self.work = None
        plan = self.plan
        self.max_rank = max(plan.max_rank, 1)
        if self.max_rank > 32:
            raise native.NativeError("matrix_approximation_rank > 32 is not supported by the native kernels")

        # ---- error-feedback mode ------------------------------------------
        ef = getattr(state, "use_error_feedback", False) and variant != "unbiased"
        ec = ef and getattr(state, "use_error_compression", False)
        if variant == "batched":
            ec = False
        kind = getattr(state, "error_compressor", "count_sketch")
        if not ef:
            self.ef_mode, self.external = native.EF_NONE, False
        elif not ec:
            self.ef_mode, self.external = native.EF_DENSE, False
        elif kind == "count_sketch" and variant == "powersgd":
            self.ef_mode, self.external = native.EF_SKETCH, False
        elif kind == "lowrank" and variant == "powersgd" and os.environ.get("CONEF_LOWRANK_NATIVE", "1") == "1":
            self.ef_mode, self.external = native.EF_NONE, False       # factors handled by run()'s low-rank branch
        elif kind == "topk" and variant == "powersgd" and self._coeffs(state) == (1.0, 0.0) \
                and os.environ.get("CONEF_TOPK_NATIVE", "1") == "1":
            # top-k store: a dense error buffer (the reference stores it dense as well,
            # communication/hPowerSGD_hook.py:90-97) that enters the products like dense error
            # feedback and is pruned to its largest entries by one grouped radix select per step
            self.ef_mode, self.external = native.EF_DENSE, False
        else:
            self.ef_mode, self.external = native.EF_NONE, True
        self.topk = ef and ec and kind == "topk" and self.ef_mode == native.EF_DENSE
        self.topk_ratio = float(getattr(state, "topk_ratio", 0.4))
        # Low-rank error store e = U V^T: its factors enter the products as small corrections
        # (P += a U (V^T Q), Q' += a V (U^T P)) and are refreshed by one power-iteration step
        # U' = orth(T V), V' = T^T U' on T = G + (a+b) U V^T - P Q^T, computed without forming T:
        # the extra records multiply G by V and G^T by U'.
        self.lowrank = ef and ec and kind == "lowrank" and not self.external and variant == "powersgd"
        # The remembered error enters the two products as extra records of the same launches
        # (P = G Q + e Q, Q' = G^T P + e^T P); the corrected matrix is never written.
        self.fused_err = self.ef_mode in (native.EF_SKETCH, native.EF_DENSE)

        # ---- descriptor records -----------------------------------------------
        nm = len(plan.mats)
        self.nm = nm
        nrec = nm * (2 if (self.fused_err or self.lowrank) else 1)
        mats = np.zeros(nrec, dtype=native.MAT_DTYPE)
        mats["cb_off"] = -1
        sk_off = tab_off = cnt_off = z_off = u_off = 0
        err_rank = int(getattr(state, "error_rank", None) or state.matrix_approximation_rank) if self.lowrank else 0
        table_chunks, count_chunks = [], []
        table_index: Dict[tuple, tuple] = {}
        self.widths = []
        seeds = ref.derive_hash_seeds(getattr(state, "hash_seed", 0), 1)[0]
        for k, e in enumerate(plan.mats):
            W = ref.sketch_width(e.m, state.sketch_size) if self.ef_mode == native.EF_SKETCH else 0
            self.widths.append(W)
            rec = mats[k]
            rec["g_off"], rec["p_off"], rec["q_off"] = e.g_off, e.p_off, e.q_off
            rec["n"], rec["m"], rec["r"], rec["W"] = e.n, e.m, e.r, W
            rec["sk_off"], rec["tab_off"], rec["cnt_off"] = -1, -1, -1
            if self.ef_mode == native.EF_SKETCH:
                Wp = (W + 3) // 4 * 4       # row pitch: 16-byte multiple so that TMA can address the sketch
                rec["sk_off"], rec["Wp"] = sk_off, Wp
                key = (e.m, W)
                if key not in table_index:
                    _, _, packed, counts = tables_for(dev, e.m, W, seeds[0], seeds[1])
                    table_chunks.append(packed)
                    count_chunks.append(counts)
                    cb_off = -1
                    # block layout of the hash: the groups regrouped by cell block follow the column
                    # table in the same arena, on an 8-byte boundary (two-word records)
                    csr = block_csr_for(dev, e.m, W, seeds[0], seeds[1]) if self.ef_mode == native.EF_SKETCH else None
                    if csr is not None:
                        pad = (tab_off + e.m) & 1
                        if pad:
                            table_chunks.append(torch.zeros(1, dtype=torch.int32, device=dev))
                        cb_off = tab_off + e.m + pad
                        table_chunks.append(csr)
                    table_index[key] = (tab_off, cnt_off, cb_off)
                    tab_off = sum(int(c.numel()) for c in table_chunks)
                    cnt_off += W
                rec["tab_off"], rec["cnt_off"], rec["cb_off"] = table_index[key]
                # record nm + k: the (n x W) sketch as a matrix; Z / Y (W x r) live behind the Q blocks
                err = mats[nm + k]
                # (its pad columns stay zero and meet zero rows of Z / produce unused rows of Y)
                err["src"], err["g_off"], err["n"], err["m"], err["r"] = 1, sk_off, e.n, Wp, e.r
                err["p_off"], err["q_off"] = e.p_off, plan.total_q + z_off
                err["sk_off"], err["tab_off"], err["cnt_off"] = -1, -1, -1
                sk_off += e.n * Wp
                z_off += Wp * e.r
            elif self.ef_mode == native.EF_DENSE:
                err = mats[nm + k]
                err["src"], err["g_off"], err["n"], err["m"], err["r"] = 1, e.g_off, e.n, e.m, e.r
                err["p_off"], err["q_off"] = e.p_off, e.q_off
                err["sk_off"], err["tab_off"], err["cnt_off"] = -1, -1, -1
            elif self.lowrank:
                # record nm + k: the same gradient matrix against the error factors: V (m x k) sits
                # behind the Q blocks, G V / U' (n x k) behind the P blocks
                kk = min(err_rank, e.n, e.m)
                err = mats[nm + k]
                err["src"], err["g_off"], err["n"], err["m"], err["r"] = 0, e.g_off, e.n, e.m, kk
                err["p_off"], err["q_off"] = plan.total_p + u_off, plan.total_q + z_off
                err["sk_off"], err["tab_off"], err["cnt_off"] = -1, -1, -1
                u_off += e.n * kk
                z_off += e.m * kk
        self.total_z, self.total_u = z_off, u_off
        if self.lowrank:
            self.max_rank = max(self.max_rank, err_rank)
        self.max_cols = max((e.m for e in plan.mats), default=0)
        # packed copies of the small operands for the tensor-core kernel: rows padded to a
        # multiple of 32, columns to NP; an error record that shares a block shares its copy
        self.np_cols = 16 if self.max_rank <= 16 else 32
        # A row pitch that is not a multiple of 16 bytes (m % 4 != 0: the LSTM's 650 columns) cannot be
        # described to TMA.  `fold` consecutive rows read as one row of fold * m elements can: the same
        # memory as an (n / fold) x (fold * m) matrix (csrc/conef.h:ConefMat).  It needs n % fold == 0
        # and fold * r accumulator columns.
        for k in range(nm):
            n_, m_, r_ = int(mats[k]["n"]), int(mats[k]["m"]), int(mats[k]["r"])
            fold = 4 // math.gcd(m_, 4)
            ok_fold = fold > 1 and n_ % fold == 0 and fold * r_ <= self.np_cols and \
                os.environ.get("CONEF_TC_FOLD", "1") == "1"
            mats[k]["fold"] = fold if ok_fold else 1
            mats[k]["ppk_fold_off"] = -1
            if self.ef_mode == native.EF_DENSE:
                mats[nm + k]["fold"], mats[nm + k]["ppk_fold_off"] = mats[k]["fold"], -1
        qpk = ppk = 0
        pad32 = lambda x: (x + 31) // 32 * 32
        for k in range(nm):
            f = int(mats[k]["fold"])
            mats[k]["qpk_off"], mats[k]["ppk_off"] = qpk, ppk
            qpk += pad32(int(mats[k]["m"]) * f) * self.np_cols
            ppk += pad32(int(mats[k]["n"])) * self.np_cols
            if f > 1:
                mats[k]["ppk_fold_off"] = ppk
                ppk += pad32(int(mats[k]["n"]) // f) * self.np_cols
        if self.lowrank:
            for k in range(nm, nrec):
                mats[k]["qpk_off"], mats[k]["ppk_off"] = qpk, ppk
                qpk += pad32(int(mats[k]["m"])) * self.np_cols
                ppk += pad32(int(mats[k]["n"])) * self.np_cols
        self.zpk_off = qpk         # the sketch records' packed operands follow the Q blocks'
        if self.fused_err:
            for k in range(nm):
                err = mats[nm + k]
                err["ppk_off"] = mats[k]["ppk_off"]
                if self.ef_mode == native.EF_DENSE:
                    err["qpk_off"] = mats[k]["qpk_off"]
                    err["ppk_fold_off"] = mats[k]["ppk_fold_off"]
                else:
                    err["qpk_off"] = qpk
                    qpk += pad32(int(err["m"])) * self.np_cols
        self.qpk_total, self.ppk_total = qpk, ppk
        # row blocks of the SIMT Q kernel
        total_cb = sum((int(r["m"]) + Q_COLS - 1) // Q_COLS for r in mats) or 1
        want_rb = max(1, math.ceil(TARGET_CTAS / total_cb))
        for rec in mats:
            n = int(rec["n"])
            nrb = max(1, min(want_rb, math.ceil(n / 64)))
            q_rows = min(Q_MAX_ROWS, ((math.ceil(n / nrb) + 7) // 8) * 8)
            rec["q_rows"] = q_rows
            shared_out = self.ef_mode == native.EF_DENSE      # gradient and error record feed one Q block
            rec["q_atomic"] = int(math.ceil(n / q_rows) > 1 or shared_out)
        self.mats_host = mats
        self.mats_dev = native.upload_struct_array(mats, dev) if nrec else None
        self.tables = torch.cat(table_chunks) if table_chunks else None
        self.counts = torch.cat(count_chunks) if count_chunks else None
        # 512-row chunks for the row-parallel Gram-Schmidt and correction kernels
        OC = 512
        chunk = lambda ks, field: [(k, c) for k in ks for c in range(math.ceil(int(mats[k][field]) / OC))]
        tl = lambda lst: (self._tiles(lst), len(lst))

        def orth_list(ks, field):
            """(tiles, number of tiles, number of records): the tiles by chunk of rows, followed by one entry
            per record for the form that gives every block a thread-block cluster."""
            ks, lst = list(ks), chunk(ks, field)
            return self._tiles(lst + [(k, int(mats[k][field])) for k in ks]), len(lst), len(ks)
        self.orth_tiles = {(0, "grad"): orth_list(range(nm), "n"), (1, "grad"): orth_list(range(nm), "m"),
                           (0, "err"): orth_list(range(nm, nrec) if self.lowrank else [], "n")}
        self.orth_max_rows = 0
        if nrec and os.environ.get("CONEF_ORTH_CLUSTER", "1") == "1":
            self.orth_max_rows = int(max(int(mats["n"].max()), int(mats["m"][:nm].max())))
        self.chunks_n, self.chunks_m = tl(chunk(range(nm), "n")), tl(chunk(range(nm), "m"))
        max_tiles = max((n for _, n, _ in self.orth_tiles.values()), default=1)
        self.gram = torch.zeros(max(max_tiles, 1) * 2 * 1024, device=dev, dtype=torch.float32)

        # decompress: rows per CTA in {8, 4, 2, 1}: the most that fit in shared memory (one
        # accumulator row of the sketch width per matrix row) while still giving every SM a few CTAs
        maxW = max(self.widths, default=0)
        if maxW * 4 > SMEM_BUDGET:
            raise native.NativeError(f"sketch width {maxW} does not fit in shared memory")
        total_rows = sum(e.n for e in plan.mats)
        self.d_rows = 1
        for cand in (8, 4, 2):
            if cand * maxW * 4 <= SMEM_BUDGET // 4 and total_rows // cand >= 3 * 148:
                self.d_rows = cand
                break
        if os.environ.get("CONEF_D_ROWS"):
            self.d_rows = int(os.environ["CONEF_D_ROWS"])
        self.d_smem = self.d_rows * maxW * 4
        # matrices on the block layout of the hash first: they run on the atomics-free kernel, whose tile
        # is a chunk of eight (row block, cell block) units, one per warp; the others by row block
        on_blocks = [int(mats[k]["cb_off"]) >= 0 for k in range(nm)]
        self.d_rbu = int(os.environ.get("CONEF_D_RBU", "1"))

        def units(e, W):      # (row blocks of a unit, cell block); matrices with more than 32 windows: one row block
            nb = W // 32
            windows = math.ceil(math.ceil(e.m / 32) / nb)
            per_unit = self.d_rbu if windows <= 32 else 1
            return math.ceil(math.ceil(e.n / self.d_rows) / per_unit) * nb
        d_tiles = [(k, ch) for k, e in enumerate(plan.mats) if on_blocks[k]
                   for ch in range(math.ceil(units(e, self.widths[k]) / 8))]
        self.d_nblk = len(d_tiles)
        d_tiles += [(k, rb) for k, e in enumerate(plan.mats) if not on_blocks[k]
                    for rb in range(math.ceil(e.n / self.d_rows))]
        self.d_tiles = self._tiles(d_tiles)
        self.n_d_tiles = len(d_tiles)
        segs = np.zeros(len(plan.segs), dtype=native.SEG_DTYPE)
        for k, s in enumerate(plan.segs):
            segs[k] = (s.g_off, s.dst_off, s.numel)
        self.segs_dev = native.upload_struct_array(segs, dev) if len(segs) else None

        # ---- buffers ---------------------------------------------------------------
        self.topk_arena = self.topk_scratch = self.topk_tiles = None
        self.n_topk_tiles = 0
        if self.topk:
            self.topk_arena = torch.zeros(max(buf.numel(), 1), device=dev, dtype=torch.float32)
            ch = self.lib.conef_topk_chunk()
            tk = [(k, c) for k, e in enumerate(plan.mats) for c in range(math.ceil(e.n * e.m / ch))]
            self.topk_tiles, self.n_topk_tiles = self._tiles(tk), len(tk)
            self.topk_scratch = torch.zeros(max(nm, 1) * (2048 + 2), device=dev, dtype=torch.int32)
        self.sketch_arena = None
        if self.ef_mode == native.EF_SKETCH:
            self.sketch_arena = torch.zeros(max(sk_off, 1), device=dev, dtype=torch.float32)
        # Q blocks followed by the Z / Y blocks of the sketch records
        self.qz = torch.zeros(max(plan.total_q + self.total_z, 1), device=dev, dtype=torch.float32)
        self.staging = torch.empty(max(plan.total_unc, 1), device=dev, dtype=torch.float32)
        self.qpk = self.ppk = None       # allocated (zeroed: pad cells stay zero) when the tensor-core path is on
        # P blocks followed by the U blocks of the low-rank records
        self.pu = torch.zeros(max(plan.total_p + self.total_u, 1), device=dev, dtype=torch.float32)
        self.u_old = self.qz2 = None
        if self.lowrank:
            self.u_old = torch.zeros(max(self.total_u, 1), device=dev, dtype=torch.float32)
            self.qz2 = torch.zeros_like(self.qz)
            self._build_corrections()
        regions = [max(plan.total_unc, 4), max(plan.total_p + self.total_u, 4), max(plan.total_q + self.total_z, 4)]
        self.symm = _try_symm(regions, group, dev) if self.world > 1 else None
        # the slot buffers the fused pipeline accumulates into: peer-addressable, or local for one rank
        self.slots = self.symm if self.symm is not None else (LocalSlots(regions, dev) if self.world == 1 else None)
        self._bound = None
        self.aux_ptr = -1
        self.use_tc = False
        self.exec_plan = None
        self.epoch_word = None
        self.tc_maps = None
        self.bind_state(state, bidx)
        self._bound = getattr(state, "error_dict", {}).get(bidx, False) if hasattr(state, "error_dict") else None

    @staticmethod
    def _coeffs(state):
        from .hooks import _ef_coeffs
        return _ef_coeffs(state)

    def _dense_err(self, state, bidx) -> Optional[torch.Tensor]:
        """The dense error buffer laid out like the bucket (None unless dense or top-k feedback)."""
        if self.ef_mode != native.EF_DENSE:
            return None
        return self.topk_arena if self.topk else state.error_dict[bidx]

    # -- auxiliary (error) buffer and tile tables ----------------------------------------
    def _aux(self, state, bidx) -> Optional[torch.Tensor]:
        if self.ef_mode == native.EF_SKETCH:
            return self.sketch_arena
        if self.ef_mode == native.EF_DENSE:
            return self._dense_err(state, bidx)
        return None

    def _build_tiles(self, work: torch.Tensor, aux: Optional[torch.Tensor]) -> None:
        """SIMT tile lists, and - for the records TMA can address - tensor maps plus split-K
        tile lists of the tensor-core kernel."""
        dev, recs = self.device, self.mats_host
        nrec = len(recs)
        self.aux_ptr = native.ptr(aux)
        self.use_tc = False
        ok = np.zeros(nrec, dtype=np.uint8)
        if nrec and _use_tc():
            maps = np.zeros(nrec * 256, dtype=np.uint8)   # two 128-byte tensor maps per record
            host = np.ascontiguousarray(recs)
            native.check(self.lib.conef_tc_encode_maps(host.ctypes.data, nrec, work.data_ptr(), self.aux_ptr,
                                                       maps.ctypes.data, ok.ctypes.data), "tc_encode_maps")
            if ok.any():
                self.tc_maps = torch.from_numpy(maps).to(dev)
                assert self.tc_maps.data_ptr() % 128 == 0
                self.use_tc = True
                if self.qpk is None:
                    self.qpk = torch.zeros(max(self.qpk_total, 1), device=dev, dtype=torch.float32)
                    self.ppk = torch.zeros(max(self.ppk_total, 1), device=dev, dtype=torch.float32)
        self.tc_ok = ok.astype(bool)
        good = [k for k in range(nrec) if self.tc_ok[k]]
        bad = [k for k in range(nrec) if not self.tc_ok[k]]

        waves = float(os.environ.get("CONEF_TC_WAVES", 3))
        min_k = int(os.environ.get("CONEF_TC_MIN_K", 384))
        max_k = int(os.environ.get("CONEF_TC_MAX_K", 1024))

        def split_tiles(mode):
            # mode 0 (P): output rows = n, K = m.  mode 1 (Q): output rows = m, K = n.
            # Every tile gets about the same K extent, chosen so that the launch has a few
            # waves of CTAs (two CTAs fit on an SM) without making tiles too short.
            def view(k):        # (output rows, K) of record k, in its folded view when it has one
                n_, m_, f = int(recs[k]["n"]), int(recs[k]["m"]), max(1, int(recs[k]["fold"]))
                return (m_ * f, n_ // f) if mode else (n_ // f, m_ * f)
            dims = [view(k) for k in good]
            work = sum(math.ceil(mn / 128) * K for mn, K in dims)
            klen_t = work / max(1.0, waves * TARGET_CTAS)
            klen_t = int(min(max_k, max(min_k, math.ceil(klen_t / 32) * 32)))
            tiles = []
            for k, (mn, K) in zip(good, dims):
                splits = max(1, round(K / klen_t))
                klen = math.ceil(math.ceil(K / splits) / 32) * 32
                splits = math.ceil(K / klen)
                shared = self.fused_err if mode == 0 else self.ef_mode == native.EF_DENSE
                folded_q = mode == 1 and int(recs[k]["fold"]) > 1       # its row blocks add into one Q block
                flag = (1 << 30) if (splits > 1 or shared or folded_q) else 0
                for mb in range(math.ceil(mn / 128)):
                    for sp in range(splits):
                        tiles.append((k | flag, mb * 128, sp * klen, klen))
            t = torch.from_numpy(np.asarray(tiles, dtype=np.int32).reshape(-1, 4)).to(dev) if tiles else None
            return t, len(tiles)

        self.tc_p_tiles, self.n_tc_p = split_tiles(0)
        p_tiles = [(k, rb) for k in bad for rb in range(math.ceil(int(recs[k]["n"]) / P_ROWS))]
        self.p_tiles, self.n_p_tiles = self._tiles(p_tiles), len(p_tiles)
        # Q tiles for all records, and separately for the gradient records and the extra records
        # (the low-rank store runs them as two passes)
        all_good, all_bad = good, bad
        self.qsets = {}
        for name, keep in (("all", lambda k: True), ("grad", lambda k: k < self.nm), ("err", lambda k: k >= self.nm)):
            good = [k for k in all_good if keep(k)]
            tc_t, n_tc = split_tiles(1)
            q_tiles = []
            for k in (k for k in all_bad if keep(k)):
                nrb = math.ceil(int(recs[k]["n"]) / int(recs[k]["q_rows"]))
                ncb = (int(recs[k]["m"]) + Q_COLS - 1) // Q_COLS
                q_tiles += [(k, t) for t in range(nrb * ncb)]
            self.qsets[name] = (tc_t, n_tc, self._tiles(q_tiles), len(q_tiles))
        good = all_good
        # outputs that are accumulated must start from zero
        self.p_zero = self.fused_err or self.use_tc
        self.q_zero = self.fused_err or self.use_tc or bool(recs["q_atomic"].any()) if nrec else False

    def _build_corrections(self) -> None:
        """Per-matrix offset tables of the four small-factor corrections of the low-rank store.
        Buffers: ``pu`` = [P | U'], ``u_old`` = U, ``qz`` = [Q | V], ``qz2`` = [. | V']."""
        nm, recs, plan = self.nm, self.mats_host, self.plan

        def table(rows):
            arr = np.zeros(nm, dtype=native.CORR_DTYPE)
            for k in range(nm):
                t_off, rows_t, rows_l, c1, terms = rows(recs[k], recs[nm + k])
                rec = arr[k]
                rec["t_off"], rec["rows_t"], rec["rows_l"], rec["c1"], rec["nterms"] = t_off, rows_t, rows_l, c1, len(terms)
                for i, (x, l, r, c2) in enumerate(terms):
                    rec["x_off"][i], rec["l_off"][i], rec["r_off"][i], rec["c2"][i] = x, l, r, c2
            return native.upload_struct_array(arr, self.device)
        I = lambda v: int(v)
        uo = lambda e: I(e["p_off"]) - plan.total_p          # offset inside u_old
        self.corr = {
            # P += a U (V^T Q):   T = P,  X = U (u_old), L = V (qz), Rm = Q (qz)
            "p": table(lambda g, e: (I(g["p_off"]), I(g["n"]), I(g["m"]), I(g["r"]),
                                     [(uo(e), I(e["q_off"]), I(g["q_off"]), I(e["r"]))])),
            # Q' += a V (U^T P):  T = Q', X = V (qz), L = U (u_old), Rm = P (pu)
            "q": table(lambda g, e: (I(g["q_off"]), I(g["m"]), I(g["n"]), I(g["r"]),
                                     [(I(e["q_off"]), uo(e), I(g["p_off"]), I(e["r"]))])),
            # G V += (a+b) U (V^T V) - P (Q^T V):  T = pu tail; term 0: X = U (u_old), L = V, Rm = V (qz);
            #                                      term 1: X = P (pu), L = Q (qz), Rm = V (qz)
            "u": table(lambda g, e: (I(e["p_off"]), I(g["n"]), I(g["m"]), I(e["r"]),
                                     [(uo(e), I(e["q_off"]), I(e["q_off"]), I(e["r"])),
                                      (I(g["p_off"]), I(g["q_off"]), I(e["q_off"]), I(g["r"]))])),
            # G^T U' += (a+b) V (U^T U') - Q (P^T U'):  T = qz2 tail; term 0: X = V (qz), L = U (u_old), Rm = U' (pu);
            #                                           term 1: X = Q (qz), L = P (pu), Rm = U' (pu)
            "v": table(lambda g, e: (I(e["q_off"]), I(g["m"]), I(g["n"]), I(e["r"]),
                                     [(I(e["q_off"]), uo(e), I(e["p_off"]), I(e["r"])),
                                      (I(g["q_off"]), I(g["p_off"]), I(e["p_off"]), I(g["r"]))])),
        }
        self.cbuf = torch.zeros(max(nm, 1) * 2 * 1024, device=self.device, dtype=torch.float32)

    # The three helpers below launch single stages on their own; the kernel micro-benchmark
    # (utils/kernel_bench.py) times them.  A training step goes through the native executor.
    def _orth(self, which: int, subset: str, buf: torch.Tensor, eps: float, st, peers=0, flags=0, world=1, epoch=0,
              packed: bool = False) -> None:
        tiles, n, _ = self.orth_tiles[(which, subset)]
        if not n:
            return
        native.check(self.lib.conef_orthogonalize_packed(
            self.mats_dev.data_ptr(), tiles.data_ptr(), n, len(self.mats_host), which, buf.data_ptr(), float(eps),
            peers, flags, world, epoch, self.status.data_ptr(), DEFAULT_SPIN_LIMIT if world > 1 else 0,
            native.ptr(self.ppk if which == 0 else self.qpk) if (packed and self.use_tc) else 0, self.np_cols,
            self.gram.data_ptr(), st), "orthogonalize")

    def _tiles(self, tiles) -> Optional[torch.Tensor]:
        if not tiles:
            return None
        return torch.from_numpy(np.asarray(tiles, dtype=np.int32).reshape(-1, 2)).to(self.device)

    # -- binding of state tensors ---------------------------------------------
    def bind_state(self, state, bidx: int) -> None:
        plan, dev = self.plan, self.device
        n_err = self.side * self.side if self.variant == "batched" else self.buf_numel
        if self.topk:
            from ..compressors import TopKError
            comps = state.error_dict.get(bidx)
            if not isinstance(comps, dict):
                comps = {}
                state.error_dict[bidx] = comps
            for cnt, e in enumerate(plan.mats):
                view = self.topk_arena[e.g_off : e.g_off + e.n * e.m].view(e.n, e.m)
                old = comps.get(cnt)
                if not (isinstance(old, TopKError) and (old.N, old.D) == (e.n, e.m)):
                    old = TopKError(e.n, e.m, self.topk_ratio, device="cpu")
                    comps[cnt] = old
                if old.err.data_ptr() != view.data_ptr():
                    view.copy_(old.err.to(dev))
                    old.err = view
        elif self.ef_mode == native.EF_DENSE:
            cur = state.error_dict.get(bidx)
            if not (torch.is_tensor(cur) and cur.numel() == n_err and cur.device == dev
                    and cur.dtype == torch.float32 and cur.is_contiguous()):
                if torch.is_tensor(cur) and cur.numel() == n_err:
                    state.error_dict[bidx] = cur.to(dev, torch.float32).contiguous()
                else:
                    logger.info("A zero tensor of length %d that represents local error is created.", n_err)
                    state.error_dict[bidx] = torch.zeros(n_err, device=dev, dtype=torch.float32)
        elif self.ef_mode == native.EF_SKETCH:
            comps = state.error_dict.get(bidx)
            if not isinstance(comps, dict):
                comps = {}
                state.error_dict[bidx] = comps
            for cnt, (e, rec) in enumerate(zip(plan.mats, self.mats_host)):
                W, Wp = int(rec["W"]), int(rec["Wp"])
                # (n, W) view with row pitch Wp into the arena
                view = self.sketch_arena[int(rec["sk_off"]) : int(rec["sk_off"]) + e.n * Wp].view(e.n, Wp)[:, :W]
                old = comps.get(cnt)
                if isinstance(old, DenseCS) and not isinstance(old, HalfDenseCS) \
                        and (old.N, old.D, old.range) == (e.n, e.m, W):
                    if old.cs.data_ptr() != view.data_ptr():
                        view.copy_(old.cs.to(dev))
                        old.cs = view
                else:
                    comp = DenseCS(e.n, e.m, state.sketch_size, device="cpu", seed=getattr(state, "hash_seed", 0))
                    comp.cs = view
                    comps[cnt] = comp
        elif self.lowrank:
            from ..compressors import LowRankError
            comps = state.error_dict.get(bidx)
            if not isinstance(comps, dict):
                comps = {}
                state.error_dict[bidx] = comps
            nm = self.nm
            for cnt, e in enumerate(plan.mats):
                rec = self.mats_host[nm + cnt]
                kk = int(rec["r"])
                u0 = int(rec["p_off"]) - plan.total_p
                uview = self.u_old[u0 : u0 + e.n * kk].view(e.n, kk)
                vview = self.qz[int(rec["q_off"]) : int(rec["q_off"]) + e.m * kk].view(e.m, kk)
                old = comps.get(cnt)
                if not (isinstance(old, LowRankError) and (old.N, old.D, old.rank) == (e.n, e.m, kk)):
                    old = LowRankError(e.n, e.m, kk, device="cpu", seed=getattr(state, "hash_seed", 0))
                    comps[cnt] = old
                if old.U.data_ptr() != uview.data_ptr():
                    uview.copy_(old.U.to(dev))
                    vview.copy_(old.V.to(dev))
                    old.U, old.V = uview, vview
        elif self.external:
            from .hooks import _make_matrix_compressor
            comps = state.error_dict.get(bidx)
            if not isinstance(comps, dict):
                comps = {}
                state.error_dict[bidx] = comps
            for cnt, e in enumerate(plan.mats):
                if cnt not in comps:
                    comps[cnt] = _make_matrix_compressor(state, e.n, e.m, dev, self.variant == "c2cs")
        # tile tables and tensor maps depend on where the error buffer lives
        aux = self._aux(state, bidx) if hasattr(state, "error_dict") else None
        if native.ptr(aux) != self.aux_ptr:
            work = self.work if self.variant == "batched" else None
            self._build_tiles(work if work is not None else _PtrOnly(self.buf_ptr), aux)
        self._build_exec(state, bidx)

    def _build_exec(self, state, bidx: int) -> None:
        """Fill the plan of the native executor (csrc/executor.h): every pointer and size the
        pipeline needs, so that one host call per step enqueues all of it."""
        self._release_exec()
        P, plan = native.PsgdPlan(), self.plan
        ptr = native.ptr

        def tl(t, n):
            return native.TileList(ptr(t) if n else None, int(n), 0)

        def qset(name):
            tc_t, n_tc, q_t, n_q = self.qsets[name]
            return native.QSet(tl(tc_t, n_tc), tl(q_t, n_q))
        nrec = len(self.mats_host)
        P.mats, P.nrec, P.nm = ptr(self.mats_dev), nrec, self.nm
        P.max_rank, P.np_cols, P.max_cols = self.max_rank, self.np_cols, self.max_cols
        P.unbiased, P.ef_mode, P.lowrank = int(self.variant == "unbiased"), self.ef_mode, int(self.lowrank)
        P.use_tc, P.p_zero, P.q_zero = int(self.use_tc), int(bool(self.p_zero)), int(bool(self.q_zero))
        P.tables, P.counts, P.sketch = ptr(self.tables), ptr(self.counts), ptr(self.sketch_arena)
        P.dense_err = ptr(self._dense_err(state, bidx))
        P.topk, P.topk_ratio = int(self.topk), self.topk_ratio
        if self.topk:
            P.topk_tiles = tl(self.topk_tiles, self.n_topk_tiles)
            P.topk_scratch = ptr(self.topk_scratch)
        P.aux = self.aux_ptr if (self.fused_err and self.aux_ptr > 0) else None
        P.qz, P.total_q, P.total_z = ptr(self.qz), plan.total_q, self.total_z
        P.pu, P.total_p, P.total_u = ptr(self.pu), plan.total_p, self.total_u
        P.u_old, P.qz2, P.qpk, P.ppk = ptr(self.u_old), ptr(self.qz2), ptr(self.qpk), ptr(self.ppk)
        P.segs, P.nsegs, P.total_unc = ptr(self.segs_dev), len(plan.segs), plan.total_unc
        P.staging = ptr(self.staging)
        P.tc_maps = ptr(self.tc_maps) if self.use_tc else None
        P.tc_p, P.simt_p = tl(self.tc_p_tiles, self.n_tc_p), tl(self.p_tiles, self.n_p_tiles)
        P.qset_all, P.qset_grad, P.qset_err = qset("all"), qset("grad"), qset("err")
        P.d_tiles, P.d_rows, P.d_smem = tl(self.d_tiles, self.n_d_tiles), self.d_rows, self.d_smem
        P.d_nblk, P.d_rbu = self.d_nblk, self.d_rbu
        otl = lambda t, n, nmat: native.TileList(ptr(t) if n else None, n, nmat if n else 0)
        P.orth_q, P.orth_p = otl(*self.orth_tiles[(1, "grad")]), otl(*self.orth_tiles[(0, "grad")])
        P.orth_u = otl(*self.orth_tiles[(0, "err")])
        P.orth_max_rows = self.orth_max_rows
        mats, nm = self.mats_host, self.nm
        P.orth_rows_q = int(mats["m"][:nm].max()) if nm else 0
        P.orth_rows_p = int(mats["n"][:nm].max()) if nm else 0
        P.orth_rows_u = int(mats["n"][nm:].max()) if self.lowrank and len(mats) > nm else 0
        P.chunks_n, P.chunks_m = tl(*self.chunks_n), tl(*self.chunks_m)
        P.gram = ptr(self.gram)
        if self.lowrank:
            P.cbuf = ptr(self.cbuf)
            P.corr_p, P.corr_q = ptr(self.corr["p"]), ptr(self.corr["q"])
            P.corr_u, P.corr_v = ptr(self.corr["u"]), ptr(self.corr["v"])
        P.status = ptr(self.status)
        P.world, P.rank, P.has_symm = self.world, self.rank, int(self.symm is not None)
        symm = self.symm
        if symm is not None:
            P.peer_flags, P.my_flags = symm.peer_flags_dev(), symm.flags_ptr()
        slots = self.slots
        if slots is not None:
            for slot in (0, 1):
                P.peer_stage[slot], P.peer_p[slot], P.peer_q[slot] = (slots.peer_ptrs_dev(slot, r) for r in range(3))
                P.local_stage[slot], P.local_p[slot], P.local_q[slot] = (ptr(slots.local(slot, r)) for r in range(3))
        P.has_slots = int(slots is not None)
        P.spin_limit = DEFAULT_SPIN_LIMIT
        # steps that draw no new random Q are captured into a CUDA graph per buffer slot and replayed
        P.use_graph = int(os.environ.get("CONEF_GRAPH", "1") == "1")
        if self.epoch_word is None:
            self.epoch_word = torch.zeros(8, dtype=torch.int32, device=self.device)   # epoch base, tile counter, barrier words
        P.epoch_word = ptr(self.epoch_word)
        P.epoch_shadow = 0
        # Fused pipeline (csrc/executor.cu:run_fused): both products must have tensor-core tiles, whose
        # last CTA publishes the epoch; the low-rank store and the unbiased variant keep the long form.
        P.done_word = ptr(self.epoch_word) + 4
        self.fused = bool(slots is not None and self.use_tc and self.nm > 0 and self.n_tc_p > 0
                          and self.qsets["all"][1] > 0 and not self.lowrank and self.variant != "unbiased"
                          and os.environ.get("CONEF_FUSED", "1") == "1")
        P.fused = int(self.fused)
        P.one_launch_orth = int(os.environ.get("CONEF_ORTH_ONE", "1") == "1")
        P.wait_kernel = int(os.environ.get("CONEF_WAIT_KERNEL", "1") == "1")
        if self.ef_mode == native.EF_SKETCH and self.qpk is not None:
            P.zpk, P.zpk_n = ptr(self.qpk) + 4 * self.zpk_off, self.qpk_total - self.zpk_off
        self.exec_plan = P

    def _release_exec(self) -> None:
        plan = getattr(self, "exec_plan", None)
        self.exec_plan = None
        if plan is not None:
            try:
                self.lib.conef_psgd_plan_release(plan)
            except Exception:       # interpreter shutdown
                pass

    def __del__(self):
        self._release_exec()

    def _run_native(self, state, work, alpha: float, beta: float, fresh: bool, eps: float, st) -> None:
        """One step through the native executor: one host call (three when the reductions
        go through NCCL because no peer memory could be set up)."""
        P, lib, plan = self.exec_plan, self.lib, self.plan
        P.work, P.slot, P.epoch = work.data_ptr(), self.step & 1, self.epoch & 0xFFFFFFFF
        P.fresh = int(fresh and self.nm > 0)
        P.seed = int(state.rng.randint(1_000_000_000)) if P.fresh else 0
        P.alpha, P.beta, P.eps = alpha, beta, eps
        timers = getattr(state, "_timers", None)
        if timers is not None and (self.world == 1 or self.symm is not None):
            for name, phase in (("psgd/P=GQ", native.PHASE_P), ("psgd/reduce+orth+Q=GtP", native.PHASE_Q),
                                ("psgd/reduce+decompress", native.PHASE_D)):
                with timers.phase(name, self.device):
                    native.check(lib.conef_psgd_run(P, phase, st), "psgd_run")
                native.launch_count += P.launched
        elif self.world == 1 or self.symm is not None:
            native.check(lib.conef_psgd_step(P, st), "psgd_step")
            native.launch_count += P.launched
        else:
            native.check(lib.conef_psgd_run(P, native.PHASE_P, st), "psgd_run(P)")
            native.launch_count += P.launched
            if plan.total_unc:
                self._nccl_sum(self.staging[: plan.total_unc], self.group)
            if self.nm:
                self._nccl_sum(self.pu[: plan.total_p], self.group, average=self.variant == "unbiased")
            native.check(lib.conef_psgd_run(P, native.PHASE_Q, st), "psgd_run(Q)")
            native.launch_count += P.launched
            if self.nm and self.variant != "unbiased":
                self._nccl_sum(self.qz[: plan.total_q], self.group, average=True)
            native.check(lib.conef_psgd_run(P, native.PHASE_D, st), "psgd_run(D)")
            native.launch_count += P.launched
        self.epoch = int(P.epoch)

    def _pq_memory(self, state, bidx):
        """Flat P/Q tensors of the state; Q is a view of the engine's combined Q|Z buffer.
        Returns (pmem, qmem, fresh)."""
        plan, dev = self.plan, self.device
        warm = getattr(state, "warm_start", False) and self.variant != "unbiased"
        p, q = state.p_memory_dict.get(bidx), state.q_memory_dict.get(bidx)
        ok = (torch.is_tensor(p) and torch.is_tensor(q) and p.numel() == plan.total_p
              and q.numel() == plan.total_q and p.device == dev)
        fresh = (not warm) or not ok
        qview, pview = self.qz[: plan.total_q], self.pu[: plan.total_p]
        if ok and q.data_ptr() != qview.data_ptr():
            qview.copy_(q.to(dev))                    # restored from a checkpoint or set by the user
        if ok and p.data_ptr() != pview.data_ptr():
            pview.copy_(p.to(dev))
        if not ok and warm:
            logger.info("Allocating contiguous memory of length %d for Ps, and of length %d for Qs.",
                        plan.total_p, plan.total_q)
        state.p_memory_dict[bidx], state.q_memory_dict[bidx] = pview, qview
        return pview, qview, fresh

    # -- one step ------------------------------------------------------------------
    def run(self, state, bucket, buf: torch.Tensor) -> None:
        """Enqueue the whole compression pipeline for one bucket on the current stream."""
        lib, plan, dev = self.lib, self.plan, self.device
        bidx = bucket.index()
        ws = self.world
        st = native.stream_ptr(dev)
        nm = self.nm
        edict = getattr(state, "error_dict", None)
        if edict is not None and edict.get(bidx, False) is not self._bound:
            self.bind_state(state, bidx)
            self._bound = edict.get(bidx, False)
        state.total_numel_before_compression += plan.numel_before
        state.total_numel_after_compression += plan.numel_after
        state.account_wire(plan.numel_after, plan.numel_before, bucket)

        if self.variant == "batched":
            work = self.work
            work[: self.buf_numel].copy_(buf)
            work[self.buf_numel :].zero_()
        else:
            work = buf
        wp = work.data_ptr()

        alpha, beta = (1.0 - getattr(state, "beta", 0.0), getattr(state, "beta", 0.0))
        if self.external or self.lowrank:
            from .hooks import _ef_coeffs
            alpha, beta = _ef_coeffs(state)
        # external error compressors: query before, clone, update after
        copy = None
        if self.external:
            comps = state.error_dict[bidx]
            for cnt, e in enumerate(plan.mats):
                comps[cnt].query(work[e.g_off : e.g_off + e.numel], alpha)
            copy = work.clone()

        pmem, qmem, fresh = self._pq_memory(state, bidx)
        eps = float(getattr(state, "orthogonalization_epsilon", 0) or 0)
        # the whole pipeline: one call into the native executor (csrc/executor.cu)
        self._run_native(state, work, alpha, beta, fresh, eps, st)

        if self.external:
            copy.sub_(work)
            comps = state.error_dict[bidx]
            for cnt, e in enumerate(plan.mats):
                comps[cnt].update(copy[e.g_off : e.g_off + e.numel], beta)
        if self.variant == "batched":
            buf.copy_(work[: self.buf_numel])
        if not getattr(state, "warm_start", False) or self.variant == "unbiased":
            state.p_memory_dict.pop(bidx, None)
            state.q_memory_dict.pop(bidx, None)
        self.step += 1

    def _launch_p(self, wp, aux, small: torch.Tensor, p_target: torch.Tensor, st) -> None:
        """P (+)= A Q over every record: tcgen05 tiles where TMA can address the matrix, SIMT elsewhere.
        ``small`` is the flat Q|Z buffer; the tensor-core kernel reads its packed copy."""
        lib = self.lib
        if self.use_tc and self.n_tc_p:
            native.check(lib.conef_pack_small(self.mats_dev.data_ptr(), len(self.mats_host), 1, small.data_ptr(),
                                              self.qpk.data_ptr(), self.max_rank, st), "pack_small(Q)")
            native.check(lib.conef_psgd_tc(0, self.mats_dev.data_ptr(), self.tc_maps.data_ptr(),
                                           self.tc_p_tiles.data_ptr(), self.n_tc_p, self.qpk.data_ptr(),
                                           p_target.data_ptr(), self.max_rank, self.status.data_ptr(), st), "psgd_tc(P)")
        if self.n_p_tiles:
            native.check(lib.conef_psgd_p(self.mats_dev.data_ptr(), self.p_tiles.data_ptr(), self.n_p_tiles, wp, aux,
                                          small.data_ptr(), p_target.data_ptr(), int(self.p_zero), self.max_rank, st),
                         "psgd_p")

    def _launch_q(self, wp, aux, pmem: torch.Tensor, q_target: torch.Tensor, st, packed: bool = False,
                  subset: str = "all") -> None:
        """Q (+)= A^T P over the records of ``subset``.  ``packed`` says the packed copy of the small
        operand is already up to date (the Gram-Schmidt kernel writes it)."""
        lib = self.lib
        tc_tiles, n_tc, q_tiles, n_q = self.qsets[subset]
        if self.use_tc and n_tc:
            if not packed:
                native.check(lib.conef_pack_small(self.mats_dev.data_ptr(), self.nm, 0, pmem.data_ptr(),
                                                  self.ppk.data_ptr(), self.max_rank, st), "pack_small(P)")
            native.check(lib.conef_psgd_tc(1, self.mats_dev.data_ptr(), self.tc_maps.data_ptr(),
                                           tc_tiles.data_ptr(), n_tc, self.ppk.data_ptr(),
                                           q_target.data_ptr(), self.max_rank, self.status.data_ptr(), st), "psgd_tc(Q)")
        if n_q:
            native.check(lib.conef_psgd_q(self.mats_dev.data_ptr(), q_tiles.data_ptr(), n_q, wp, aux,
                                          pmem.data_ptr(), q_target.data_ptr(), self.max_rank, st), "psgd_q")


class _PtrOnly:
    """Carries a raw device address where only ``data_ptr()`` is needed."""

    def __init__(self, ptr: int):
        self._ptr = ptr

    def data_ptr(self) -> int:
        return self._ptr


def _get_engine(state, bucket, buf, group, factory):
    bidx = bucket.index()
    eng = state._engines.get(bidx)
    if eng is None or eng.buf_ptr != buf.data_ptr() or eng.buf_numel != buf.numel():
        eng = factory()
        state._engines[bidx] = eng
    return eng


def run_powersgd_native(state, bucket, group, variant: str) -> torch.futures.Future:
    buf = bucket.buffer()
    dev = buf.device
    stream = comm_stream_for(dev)
    stream.wait_stream(torch.cuda.current_stream(dev))
    state.poll_status()
    with torch.cuda.stream(stream):
        eng = _get_engine(state, bucket, buf, group,
                          lambda: PowerSGDEngine(state, buf, bucket.gradients(), group, variant, bucket.index()))
        eng.run(state, bucket, buf)
        fut = _done_on_current_stream(buf)
    if bucket.is_last() and eng.world > 1:
        state.post_status(eng.status, stream)
    state.maybe_increase_iter(bucket)
    return fut


# ==========================================================================
# random block
# ==========================================================================
class RandBlockEngine(_EngineBase):
    def __init__(self, state, buf, grads, group, unbiased: bool):
        super().__init__(buf.device)
        dev = self.device
        self.group, self.world = group, group.size()
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.buf_ptr, self.buf_numel = buf.data_ptr(), buf.numel()
        self.unbiased = unbiased
        self.plan = planlib.build_block_plan(buf, grads, state.compression_ratio)
        plan = self.plan
        ef = (not unbiased) and state.use_error_feedback
        ec = ef and state.use_error_compression
        kind = getattr(state, "error_compressor", "count_sketch")
        if not ef:
            self.ef_mode = native.EF_NONE
        elif not ec:
            self.ef_mode = native.EF_DENSE
        elif kind == "count_sketch":
            self.ef_mode = native.EF_SKETCH
        elif kind == "quant8":
            self.ef_mode = native.EF_QUANT8
        else:
            raise native.NativeError(f"random block + {kind}: not fused")  # caller falls back

        blks = np.zeros(len(plan.blocks), dtype=native.BLK_DTYPE)
        self.nblk_tiles = 0
        seeds = ref.derive_hash_seeds(getattr(state, "hash_seed", 0), 1)[0]
        arena = tab_off = cnt_off = scale_off = 0
        table_index, table_chunks, count_chunks = {}, [], []
        widths = []
        for k, b in enumerate(plan.blocks):
            rec = blks[k]
            rec["g_off"], rec["numel"], rec["block"], rec["stage_off"] = b.g_off, b.numel, b.block, b.stage_off
            rec["n"], rec["m"] = b.n, b.m
            rec["tab_off"], rec["cnt_off"], rec["cb_off"] = -1, -1, -1
            rec["sk_off"] = arena
            if self.ef_mode == native.EF_SKETCH:
                W = ref.sketch_width(b.m, state.sketch_size)
                widths.append(W)
                rec["W"] = W
                key = (b.m, W)
                if key not in table_index:
                    _, _, packed, counts = tables_for(dev, b.m, W, seeds[0], seeds[1])
                    table_chunks.append(packed)
                    count_chunks.append(counts)
                    cb_off = -1
                    csr = block_csr_for(dev, b.m, W, seeds[0], seeds[1])      # block layout: regrouped records
                    if csr is not None:
                        pad = (tab_off + b.m) & 1
                        if pad:
                            table_chunks.append(torch.zeros(1, dtype=torch.int32, device=dev))
                        cb_off = tab_off + b.m + pad
                        table_chunks.append(csr)
                    table_index[key] = (tab_off, cnt_off, cb_off)
                    tab_off = sum(int(c.numel()) for c in table_chunks)
                    cnt_off += W
                rec["tab_off"], rec["cnt_off"], rec["cb_off"] = table_index[key]
                arena += b.n * W
            else:
                arena += b.numel
                rec["scale_off"] = scale_off
                scale_off += (b.numel + QGROUP - 1) // QGROUP
        self.blks_host = blks
        self.arena_elems, self.n_scales = arena, scale_off
        self.tables = torch.cat(table_chunks) if table_chunks else None
        self.counts = torch.cat(count_chunks) if count_chunks else None
        if self.ef_mode == native.EF_SKETCH:
            maxW = max(widths, default=1)
            if maxW * 4 > SMEM_BUDGET:
                raise native.NativeError(f"sketch width {maxW} does not fit in shared memory")
            self.rows = int(max(1, min(8, SMEM_BUDGET // (maxW * 8))))     # accumulators + a copy of the old rows
            self.smem = self.rows * maxW * 4
            # tensors on the block layout of the hash first: their tile is a chunk of eight (block of 8 rows,
            # cell block) units of the atomics-free kernel; the others go by blocks of `rows` rows
            on_blocks = [int(blks[k]["cb_off"]) >= 0 for k in range(len(plan.blocks))]
            tiles = [(k, ch) for k, b in enumerate(plan.blocks) if on_blocks[k]
                     for ch in range(math.ceil(math.ceil(b.n / 8) * (int(blks[k]["W"]) // 32) / 8))]
            self.nblk_tiles = len(tiles)
            tiles += [(k, rb) for k, b in enumerate(plan.blocks) if not on_blocks[k]
                      for rb in range(math.ceil(b.n / self.rows))]
        else:
            # flat modes: `rows` is the number of 256-element groups a warp walks (loads of the next group in flight)
            self.rows, self.smem = int(os.environ.get("CONEF_RB_GROUPS", "8")), 0
            tiles = [(k, g) for k, b in enumerate(plan.blocks)
                     for g in range(math.ceil(((b.numel + QGROUP - 1) // QGROUP) / self.rows))]
        self.n_tiles = len(tiles)
        self.tiles = torch.from_numpy(np.asarray(tiles, dtype=np.int32).reshape(-1, 2)).to(dev) if tiles else None
        segs = np.zeros(len(plan.segs), dtype=native.SEG_DTYPE)
        for k, s in enumerate(plan.segs):
            segs[k] = (s.g_off, s.dst_off, s.numel)
        self.segs_dev = native.upload_struct_array(segs, dev) if len(segs) else None
        self.blks_dev = torch.empty(max(blks.nbytes, 1), dtype=torch.uint8, device=dev)
        # two pinned staging copies of the block table (the block offsets change every step); an
        # event per copy says when its upload has been consumed
        self._pin = [torch.empty(max(blks.nbytes, 1), dtype=torch.uint8).pin_memory() for _ in range(2)] \
            if dev.type == "cuda" else None
        self._pin_evt = [None, None]
        self.staging_unc = torch.empty(max(plan.total_unc, 1), device=dev, dtype=torch.float32)
        self.staging_blk = torch.empty(max(plan.total_block, 1), device=dev, dtype=torch.float32)
        self.err_arena = self.codes = self.scales = None
        # regions: staged uncompressed tensors, staged blocks, and the reduced blocks of the two-shot form
        # (payloads above CONEF_TWO_SHOT_BYTES: each rank sums a 1/world slice and pushes it to the peers)
        pad4 = lambda x: (max(x, 4) + 3) // 4 * 4
        self.two_shot = self.world > 1 and 4 * plan.total_block >= int(os.environ.get("CONEF_TWO_SHOT_BYTES", 1 << 20))
        regions = [pad4(plan.total_unc), pad4(plan.total_block), pad4(plan.total_block) if self.two_shot else 4]
        self.symm = _try_symm(regions, group, dev) if self.world > 1 else None
        self.slots = self.symm if self.symm is not None else (LocalSlots(regions, dev) if self.world == 1 else None)
        self.done_word = torch.zeros(4, dtype=torch.int32, device=dev)
        self.exec_plan, self._exec_key = None, None

    def bind_state(self, state, bidx):
        if self.ef_mode == native.EF_NONE:
            return
        plan, dev = self.plan, self.device
        errs = state.error_dict.get(bidx)
        errs = errs if isinstance(errs, list) else []
        new = []
        if self.ef_mode == native.EF_QUANT8:
            if self.codes is None:
                self.codes = torch.zeros(max(self.arena_elems, 1), dtype=torch.int8, device=dev)
                self.scales = torch.zeros(max(self.n_scales, 1), dtype=torch.float32, device=dev)
            for k, (b, rec) in enumerate(zip(plan.blocks, self.blks_host)):
                c0, s0 = int(rec["sk_off"]), int(rec["scale_off"])
                ng = (b.numel + QGROUP - 1) // QGROUP
                cv, sv = self.codes[c0 : c0 + b.numel], self.scales[s0 : s0 + ng]
                old = errs[k] if k < len(errs) else None
                if isinstance(old, Quant8Error) and old.codes.numel() == b.numel:
                    if old.codes.data_ptr() != cv.data_ptr():
                        cv.copy_(old.codes.to(dev)); sv.copy_(old.scales.to(dev))
                        old.codes, old.scales = cv, sv
                    new.append(old)
                else:
                    new.append(Quant8Error(b.n, b.m, device=dev, codes=cv, scales=sv))
        else:
            if self.err_arena is None:
                self.err_arena = torch.zeros(max(self.arena_elems, 1), dtype=torch.float32, device=dev)
            for k, (b, rec) in enumerate(zip(plan.blocks, self.blks_host)):
                o = int(rec["sk_off"])
                old = errs[k] if k < len(errs) else None
                if self.ef_mode == native.EF_DENSE:
                    view = self.err_arena[o : o + b.numel].view(b.n, b.m)
                    if torch.is_tensor(old) and old.numel() == b.numel and old.data_ptr() != view.data_ptr():
                        view.copy_(old.to(dev).view(b.n, b.m))
                    new.append(view)
                else:
                    W = int(rec["W"])
                    view = self.err_arena[o : o + b.n * W]
                    if isinstance(old, DenseCS) and (old.N, old.D, old.range) == (b.n, b.m, W):
                        if old.cs.data_ptr() != view.data_ptr():
                            view.copy_(old.cs.reshape(-1).to(dev))
                            old.cs = view.view(b.n, W)
                        new.append(old)
                    else:
                        new.append(DenseCS(b.n, b.m, state.sketch_size, device=dev,
                                           seed=getattr(state, "hash_seed", 0), storage=view))
        state.error_dict[bidx] = new

    def _build_exec(self) -> None:
        """Plan of the native executor (csrc/executor.h:ConefRandblockPlan)."""
        P, plan, ptr = native.RandblockPlan(), self.plan, native.ptr
        P.blks, P.nblks, P.rows_per_cta = ptr(self.blks_dev), len(plan.blocks), self.rows
        P.tiles = native.TileList(ptr(self.tiles) if self.n_tiles else None, self.n_tiles, 0)
        P.nblk_tiles = self.nblk_tiles
        P.segs, P.nsegs, P.ef_mode = ptr(self.segs_dev), len(plan.segs), self.ef_mode
        P.total_unc, P.total_block = plan.total_unc, plan.total_block
        P.staging_unc, P.staging_blk = ptr(self.staging_unc), ptr(self.staging_blk)
        P.sketch = ptr(self.err_arena) if self.ef_mode == native.EF_SKETCH else None
        P.dense_err = ptr(self.err_arena) if self.ef_mode == native.EF_DENSE else None
        P.tables, P.counts = ptr(self.tables), ptr(self.counts)
        P.qcodes, P.qscales = ptr(self.codes), ptr(self.scales)
        P.smem, P.status = self.smem, ptr(self.status)
        P.world, P.rank, P.has_symm, P.unbiased = self.world, self.rank, int(self.symm is not None), int(self.unbiased)
        symm = self.symm
        if symm is not None:
            P.peer_flags, P.my_flags = symm.peer_flags_dev(), symm.flags_ptr()
        slots = self.slots if os.environ.get("CONEF_FUSED", "1") == "1" else symm
        if slots is not None:
            for slot in (0, 1):
                P.peer_unc[slot], P.peer_blk[slot] = slots.peer_ptrs_dev(slot, 0), slots.peer_ptrs_dev(slot, 1)
                P.local_unc[slot], P.local_blk[slot] = ptr(slots.local(slot, 0)), ptr(slots.local(slot, 1))
                P.peer_red[slot], P.local_red[slot] = slots.peer_ptrs_dev(slot, 2), ptr(slots.local(slot, 2))
        P.has_slots = int(slots is not None and os.environ.get("CONEF_FUSED", "1") == "1")
        P.two_shot = int(self.two_shot)
        P.done_word = ptr(self.done_word)
        P.spin_limit = DEFAULT_SPIN_LIMIT
        self.exec_plan = P
        self._exec_key = (ptr(self.err_arena), ptr(self.codes))

    def _run_native(self, state, buf, stage_unc, stage_blk, st) -> None:
        """One step through the native executor: one host call (two with NCCL in between when no
        peer memory could be set up)."""
        if self.exec_plan is None or self._exec_key != (native.ptr(self.err_arena), native.ptr(self.codes)):
            self._build_exec()
        P, lib, plan = self.exec_plan, self.lib, self.plan
        beta = getattr(state, "beta", 0.0)
        P.work, P.slot, P.epoch = buf.data_ptr(), self.step & 1, self.epoch & 0xFFFFFFFF
        P.alpha, P.beta = 1.0 - beta, beta
        if self.world == 1 or self.symm is not None:
            native.check(lib.conef_randblock_run(P, 3, st), "randblock_run")
            native.launch_count += P.launched
        else:
            native.check(lib.conef_randblock_run(P, 1, st), "randblock_run(gather)")
            native.launch_count += P.launched
            if plan.total_unc:
                self._nccl_sum(stage_unc[: plan.total_unc], self.group)
            if len(plan.blocks):
                self._nccl_sum(stage_blk[: plan.total_block], self.group)
            native.check(lib.conef_randblock_run(P, 2, st), "randblock_run(scatter)")
            native.launch_count += P.launched
        self.epoch = int(P.epoch)

    def run(self, state, bucket, buf):
        lib, plan, dev = self.lib, self.plan, self.device
        bidx, ws = bucket.index(), self.world
        st = native.stream_ptr(dev)
        if self.step == 0 or self.ef_mode != native.EF_NONE and not isinstance(state.error_dict.get(bidx), list):
            self.bind_state(state, bidx)
        nb = len(plan.blocks)
        # shared-RNG block offsets: one draw per compressed tensor, in bucket order
        blks = self.blks_host
        for k, b in enumerate(plan.blocks):
            blks["start"][k] = int(state.rng.choice(b.numel))
        if nb:
            k = self.step & 1
            if self._pin_evt[k] is not None:
                self._pin_evt[k].synchronize()          # the upload of two steps ago (long done)
            raw = blks.view(np.uint8).reshape(-1)
            self._pin[k].numpy()[: raw.size] = raw
            self.blks_dev[: raw.size].copy_(self._pin[k][: raw.size], non_blocking=True)
            if self._pin_evt[k] is None:
                self._pin_evt[k] = torch.cuda.Event()
            self._pin_evt[k].record()
        symm, slot = self.symm, self.step & 1
        fused = self.slots is not None and os.environ.get("CONEF_FUSED", "1") == "1"
        holder = self.slots if fused else symm
        stage_unc = holder.local(slot, 0) if holder else self.staging_unc
        stage_blk = holder.local(slot, 1) if holder else self.staging_blk
        state.compressed_tensor_memory[bidx] = stage_blk[: plan.total_block]
        state.account_wire(plan.total_unc + plan.total_block, buf.numel(), bucket)
        self._run_native(state, buf, stage_unc, stage_blk, st)
        self.step += 1


def run_randblock_native(state, bucket, group, unbiased: bool) -> torch.futures.Future:
    from .hooks import _randblock_torch

    buf = bucket.buffer()
    dev = buf.device
    stream = comm_stream_for(dev)
    stream.wait_stream(torch.cuda.current_stream(dev))
    state.poll_status()
    with torch.cuda.stream(stream):
        try:
            eng = _get_engine(state, bucket, buf, group,
                              lambda: RandBlockEngine(state, buf, bucket.gradients(), group, unbiased))
        except native.NativeError as exc:
            if "not fused" not in str(exc):
                raise
            # compressors without a fused kernel: PyTorch ops + the stand-alone native kernels
            return _randblock_torch(state, bucket, group, unbiased=unbiased)
        eng.run(state, bucket, buf)
        fut = _done_on_current_stream(buf)
    if bucket.is_last() and eng.world > 1:
        state.post_status(eng.status, stream)
    state.maybe_increase_iter(bucket)
    return fut

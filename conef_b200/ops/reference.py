"""Plain PyTorch / NumPy restatement of every numerical op in the library.

These functions are the numerics oracle for the CUDA kernels and, at the same
time, the execution path on CPU tensors (gloo ranks).  They are written for
clarity, in fp32, with no device-specific code.

Behavioural spec (paths are relative to the reference project):
  * hash / sign           communication/compressors/CountSketch.py:7-18,60-62
  * 1-row sketch update   communication/compressors/CountSketch.py:27-67
  * 1-row sketch query    communication/compressors/CountSketch.py:70-98
  * 3-row sketch          communication/compressors/CountSketchHash3.py:27-147
  * Gram-Schmidt          communication/powerSGD_hook.py:12-43
  * compress decision     communication/powerSGD_hook.py:46-70
  * top-k sparsifier      communication/hPowerSGD_hook.py:90-97
"""
from __future__ import annotations

import functools
import os
import math
from typing import Optional, Tuple

import numpy as np
import torch

# Hash constants of the reference's single-row sketch (CountSketch.py:112-113)
# and of its three-row sketch (CountSketchHash3.py:40-41).
DEFAULT_A = 994443
DEFAULT_B = 609478
HASH3_A = (994443, 4113759, 9171025)
HASH3_B = (609478, 2949676, 2171464)
# Offsets added to (a, b) to derive the sign hash of each row
# (CountSketchHash3.py:73,81,85).  The reference's query kernel uses (8, 7)
# for the third row while its update kernel uses (8, 4); we use (8, 4) in both.
SIGN_OFFSETS = ((2, 3), (4, 5), (8, 4))

_M32 = np.uint64(0xFFFFFFFF)


def _to_signed32(x: np.ndarray) -> np.ndarray:
    x = (x & _M32).astype(np.int64)
    return np.where(x >= 2 ** 31, x - 2 ** 32, x)


def hash32(value, rng: int, a: int, b: int) -> np.ndarray:
    """Bit-exact emulation of the reference's ``hash(value, range, a, b)``.

    The reference computes on *signed* 32-bit ints with wrapping multiplies
    and arithmetic right shifts; the last shift-xor clears the sign bit so
    the C remainder is non-negative.
    """
    v = np.asarray(value, dtype=np.int64)
    a64 = np.int64(np.int32(np.uint32(a & 0xFFFFFFFF)))
    b64 = np.int64(np.int32(np.uint32(b & 0xFFFFFFFF)))
    h = _to_signed32((a64 * v + b64).astype(np.uint64))
    h = _to_signed32((h ^ (h >> 16)).astype(np.uint64))
    h = _to_signed32((h.astype(np.uint64) & _M32) * np.uint64(0x85EBCA6B))
    h = _to_signed32((h ^ (h >> 13)).astype(np.uint64))
    h = _to_signed32((h.astype(np.uint64) & _M32) * np.uint64(0xC2B2AE35))
    h = _to_signed32((h ^ (h >> 16)).astype(np.uint64))
    return (h % np.int64(rng)).astype(np.int64)


def hash_layout() -> str:
    """``block`` (default) or ``universal`` (``CONEF_HASH=universal``): see :func:`_hash_table_cached`."""
    return "universal" if os.environ.get("CONEF_HASH", "block").lower().startswith("u") else "block"


BLOCK_MIN_WIDTH = 64      # sketch rows narrower than this keep the per-element hash


def _hash_table_np(D: int, W: int, a: int, b: int, sa: int, sb: int, layout: Optional[str] = None):
    return _hash_table_cached(D, W, a, b, sa, sb, layout or hash_layout())


def _block_hash_np(D: int, W: int, a: int, b: int):
    """Block layout: (cell block u_g, lane mask x_g) of every aligned group of 32 columns, and
    ``order[s, c]`` = position inside window s of the group that goes to cell block c."""
    nb, ng = W // 32, (D + 31) // 32
    S = (ng + nb - 1) // nb
    key = hash32(np.arange(S * nb, dtype=np.int64), 1 << 30, a, b).reshape(S, nb)
    order = np.argsort(key, axis=1, kind="stable")
    rank = np.empty_like(order)
    rank[np.arange(S)[:, None], order] = np.arange(nb)[None, :]
    u = rank.reshape(-1)[:ng]
    x = hash32(np.arange(ng, dtype=np.int64), 32, a + 11, b + 13)
    return u, x, order


@functools.lru_cache(maxsize=512)
def _hash_table_cached(D: int, W: int, a: int, b: int, sa: int, sb: int, layout: str):
    """Bucket and sign of every column.

    ``universal``: h_j = hash(j, W), the reference's per-element hash (CountSketch.py:7-18,60-62), bit
    for bit.

    ``block``: columns are hashed in aligned groups of 32, and the groups in windows of
    nb = W // 32 consecutive groups.  Inside window s a pseudo-random permutation (the ranks of
    hash(g, 2**30) among the window's nb group numbers, the ones past the end of the row included)
    sends every group to a cell block of its own, u_g; column 32 g + k goes to cell
    32 u_g + (k xor x_g) with x_g = hash(g, 32).  Two columns of different windows share a cell with
    probability 1 / (32 nb), columns of one window never do, and the signs stay per column: the
    sketch is unbiased, with at most the per-element variance of the universal hash; up to 31 cells
    at the end of a sketch row stay unused.  What it buys on the GPU: the 32 columns a warp handles
    together land in 32 different shared-memory banks (a uniformly random cell costs about 3.5
    serialised passes per warp-wide atomic); every cell block receives exactly one group per window,
    so a warp that walks the groups of ONE cell block (:func:`block_csr`) keeps that block's 32 sums
    in registers, with no atomics and no imbalance between warps; and the warps of a CTA, which
    take neighbouring cell blocks, read inside the same window of 128 nb bytes per row at the same
    time.  Rows narrower than ``BLOCK_MIN_WIDTH`` cells use ``universal``.
    """
    cols = np.arange(D, dtype=np.int64)
    if layout == "block" and W >= BLOCK_MIN_WIDTH:
        u, x, _ = _block_hash_np(D, W, a, b)
        idx = 32 * u[cols >> 5] + ((cols & 31) ^ x[cols >> 5])
    else:
        idx = hash32(cols, W, a, b)
    sign_bit = hash32(cols, W, a + sa, b + sb) & 1
    sign = np.where(sign_bit == 1, 1.0, -1.0).astype(np.float32)
    return idx, sign


def hash_table(D: int, W: int, a: int = DEFAULT_A, b: int = DEFAULT_B,
               sign_offset: Tuple[int, int] = SIGN_OFFSETS[0], device="cpu", layout: Optional[str] = None):
    """Column table ``(bucket index h_j, sign s_j)`` for ``j in [0, D)``.

    The hash depends only on the column, so one table serves every row of a
    matrix: sketch = M @ H, unsketch = S @ H^T with H in {0, +1, -1}^{D x W}.
    """
    idx, sign = _hash_table_np(int(D), int(W), int(a), int(b), int(sign_offset[0]), int(sign_offset[1]), layout)
    return (torch.from_numpy(idx).to(device), torch.from_numpy(sign).to(device))


def packed_hash_table(D: int, W: int, a: int, b: int, sign_offset=SIGN_OFFSETS[0],
                      layout: Optional[str] = None) -> np.ndarray:
    """``h_j | (sign_bit_j << 31)`` as int32 — the layout the CUDA kernels read."""
    idx, sign = _hash_table_np(int(D), int(W), int(a), int(b), int(sign_offset[0]), int(sign_offset[1]), layout)
    packed = idx.astype(np.uint32) | ((sign > 0).astype(np.uint32) << np.uint32(31))
    return packed.view(np.int32)


NO_GROUP = 0x7FFFFFF


@functools.lru_cache(maxsize=512)
def _block_csr_cached(D: int, W: int, a: int, b: int, sa: int, sb: int):
    u, x, order = _block_hash_np(D, W, a, b)
    _, sign = _hash_table_cached(D, W, a, b, sa, sb, "block")
    nb, ng = W // 32, (D + 31) // 32
    S = order.shape[0]
    bits = np.zeros(ng * 32, dtype=np.uint32)
    bits[:D] = (sign > 0).astype(np.uint32)
    words = (bits.reshape(ng, 32) << np.arange(32, dtype=np.uint32)).sum(axis=1, dtype=np.uint64).astype(np.uint32)
    g = (np.arange(S, dtype=np.int64)[:, None] * nb + order)          # (S, nb): group of cell block c in window s
    real = g < ng
    gc = np.where(real, g, 0)
    rec = np.empty((S, nb, 2), dtype=np.uint32)
    rec[..., 0] = np.where(real, gc.astype(np.uint32) | (x[gc].astype(np.uint32) << np.uint32(27)), np.uint32(NO_GROUP))
    rec[..., 1] = np.where(real, words[gc], np.uint32(0))
    return rec.reshape(-1).view(np.int32)


def block_csr(D: int, W: int, a: int, b: int, sign_offset=SIGN_OFFSETS[0]) -> Optional[np.ndarray]:
    """The block layout regrouped by cell block, as one int32 array, or ``None`` when the layout of
    this (D, W) is not ``block``.

    ``S = ceil(ceil(D / 32) / nb)`` windows times ``nb = W // 32`` cell blocks two-word records,
    window-major: record ``s * nb + c`` names the group that cell block c receives from window s as
    ``g | x_g << 27`` (``NO_GROUP``: none, past the end of the row; so D < 2**32) and the 32 sign bits
    of the group's columns (bit k: column 32 g + k has sign +1).
    """
    if hash_layout() != "block" or W < BLOCK_MIN_WIDTH:
        return None
    return _block_csr_cached(int(D), int(W), int(a), int(b), int(sign_offset[0]), int(sign_offset[1]))


def derive_hash_seeds(seed: int, rows: int):
    """Seed-derived ``(a_k, b_k)`` pairs for ``rows`` hash rows.

    ``seed == 0`` reproduces the reference constants so that sketches are
    bit-compatible with the reference's default.
    """
    if seed == 0:
        if rows == 1:
            return [(DEFAULT_A, DEFAULT_B)]
        if rows <= 3:
            return list(zip(HASH3_A[:rows], HASH3_B[:rows]))
    rs = np.random.RandomState(seed & 0x7FFFFFFF)
    out = []
    for _ in range(rows):
        a = int(rs.randint(1, 2 ** 23)) | 1
        b = int(rs.randint(0, 2 ** 23))
        out.append((a, b))
    return out


def sketch_width(D: int, sketch_size: float) -> int:
    return max(int(D * sketch_size), 1)


# --------------------------------------------------------------------------
# single-row count sketch
# --------------------------------------------------------------------------
def sketch_query_ref(mat: torch.Tensor, cs: torch.Tensor, idx: torch.Tensor,
                     sign: torch.Tensor, alpha: float) -> None:
    """``mat[i, j] += alpha * s_j * cs[i, h_j]`` in place."""
    mat.add_(cs.to(mat.dtype)[:, idx] * sign.to(mat.dtype), alpha=alpha)


def sketch_update_ref(vec: torch.Tensor, cs: torch.Tensor, idx: torch.Tensor,
                      sign: torch.Tensor, beta: float) -> None:
    """``cs <- cs + sketch(vec) - (1 - beta) * k_h * cs`` in place.

    ``k_h`` is the number of columns hashing to bucket ``h``: the reference
    subtracts ``(1-beta) * cs_old[h_j]`` once per column ``j``.
    """
    W = cs.shape[1]
    cnt = torch.bincount(idx, minlength=W).to(cs.dtype)
    add = torch.zeros_like(cs)
    add.index_add_(1, idx, (vec * sign).to(cs.dtype))
    cs.mul_(1.0 - (1.0 - beta) * cnt).add_(add)


# --------------------------------------------------------------------------
# three-row count sketch with a median estimator
# --------------------------------------------------------------------------
def median3(a, b, c):
    return torch.maximum(torch.minimum(a, b), torch.minimum(torch.maximum(a, b), c))


def sketch3_query_ref(mat, cs_rows, tables, alpha: float) -> None:
    est = [alpha * cs[:, idx] * sign for cs, (idx, sign) in zip(cs_rows, tables)]
    mat.add_(median3(*est))


def sketch3_update_ref(vec, cs_rows, tables, beta: float) -> None:
    est = [-(1.0 - beta) * sign * cs[:, idx] for cs, (idx, sign) in zip(cs_rows, tables)]
    u = median3(*est) + vec
    for cs, (idx, sign) in zip(cs_rows, tables):
        cs.index_add_(1, idx, sign * u)


# --------------------------------------------------------------------------
# PowerSGD helpers
# --------------------------------------------------------------------------
def should_compress(n: int, m: int, rank: int, min_rate: float):
    """(compress?, numel before, numel after) as in powerSGD_hook.py:46-70."""
    before = n * m
    after = (n + m) * rank
    return (after * min_rate < before, before, after)


def gram_schmidt_ref(mat: torch.Tensor, eps: float = 0.0) -> None:
    """Column-by-column Gram-Schmidt in place (powerSGD_hook.py:12-43)."""
    ncol = mat.shape[1]
    for i in range(ncol):
        col = mat[:, i : i + 1]
        if eps == 0:
            col /= torch.norm(col)
        else:
            col /= torch.norm(col) + eps
        if i + 1 < ncol:
            rest = mat[:, i + 1 :]
            rest -= torch.sum(col * rest, dim=0) * col


ORTH_SHIFT, ORTH_SHIFT_FINAL = 1e-5, 1e-7


def shifted_cholesky_qr2_(mat: torch.Tensor, eps: float = 0.0) -> None:
    """What the native orthogonalisation computes (csrc/orth.cu), restated in the matrix's own
    precision: two rounds of ``A <- A R^-1`` with ``R`` the Cholesky factor of ``A^T A``, a pivot
    never taken below ``shift`` times its column's squared norm, exactly-zero columns left zero
    (the kernel refills those with pseudo-random values in its last round).  In exact arithmetic
    and without shifts this is the Gram-Schmidt result of :func:`gram_schmidt_ref`."""
    r = mat.shape[1]
    for rnd, shift in enumerate((ORTH_SHIFT, ORTH_SHIFT_FINAL)):
        G = mat.t() @ mat
        R = torch.zeros_like(G)
        for j in range(r):
            if not bool(G[j, j] > 0):
                continue
            d = G[j, j] - (R[:j, j] ** 2).sum()
            d = torch.maximum(d, shift * G[j, j])
            R[j, j] = d.sqrt()
            if j + 1 < r:
                R[j, j + 1:] = (G[j, j + 1:] - R[:j, j] @ R[:j, j + 1:]) / R[j, j]
        Ri = torch.zeros_like(R)
        for c in range(r):
            if not bool(R[c, c] > 0):
                continue
            for i in range(c, -1, -1):
                if not bool(R[i, i] > 0):
                    continue
                v = (1.0 if i == c else 0.0) - R[i, i + 1:c + 1] @ Ri[i + 1:c + 1, c]
                Ri[i, c] = v / (R[i, i] + (eps if rnd == 0 else 0.0))
        mat.copy_(mat @ Ri)


def topk_keep_(err: torch.Tensor, topk_ratio: float) -> None:
    """Keep the ``max(1, int(0.5*ratio*numel))`` largest-magnitude entries."""
    flat = err.view(-1)
    k = max(1, int(0.5 * topk_ratio * flat.numel()))
    _, pos = torch.topk(flat.abs(), k, sorted=False)
    vals = flat[pos].clone()
    flat.zero_()
    flat[pos] = vals


# --------------------------------------------------------------------------
# random block selection
# --------------------------------------------------------------------------
def block_bounds(numel: int, ratio: float, start: int):
    """(block, first_len, rest) of a wrap-around block starting at ``start``."""
    block = max(1, int(ratio * numel))
    end = min(start + block, numel)
    first = end - start
    return block, first, block - first


def block_mask(numel: int, ratio: float, start: int, device="cpu") -> torch.Tensor:
    block, first, rest = block_bounds(numel, ratio, start)
    mask = torch.zeros(numel, dtype=torch.bool, device=device)
    mask[start : start + first] = True
    if rest > 0:
        mask[:rest] = True
    return mask


# --------------------------------------------------------------------------
# 8-bit group quantisation
# --------------------------------------------------------------------------
QUANT_GROUP = 256


def quant8_encode_ref(x: torch.Tensor):
    """Symmetric int8 per group of 256 consecutive elements -> (codes, scales)."""
    flat = x.reshape(-1).float()
    n = flat.numel()
    groups = (n + QUANT_GROUP - 1) // QUANT_GROUP
    pad = groups * QUANT_GROUP - n
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    g = flat.view(groups, QUANT_GROUP)
    scale = g.abs().amax(dim=1) / 127.0
    inv = torch.where(scale > 0, 1.0 / scale, torch.zeros_like(scale))
    q = torch.clamp(torch.round(g * inv[:, None]), -127, 127).to(torch.int8)
    return q.view(-1)[:n].contiguous(), scale.contiguous()


def quant8_decode_ref(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    n = codes.numel()
    gidx = torch.arange(n, device=codes.device) // QUANT_GROUP
    return codes.float() * scale[gidx]


# --------------------------------------------------------------------------
# LAMB (one tensor)
# --------------------------------------------------------------------------
def lamb_step_ref(p, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale=1.0,
                  bias_correction=True, max_trust=None):
    """One LAMB update on a single tensor, fp32 (You et al. 2019, as in apex FusedLAMB)."""
    g = g.float() / grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    if bias_correction:
        mh = m / (1 - beta1 ** step)
        vh = v / (1 - beta2 ** step)
    else:
        mh, vh = m, v
    upd = mh / (vh.sqrt() + eps) + wd * p
    wn = p.norm()
    un = upd.norm()
    trust = torch.where((wn > 0) & (un > 0), wn / un, torch.ones_like(wn))
    if max_trust is not None:
        trust = trust.clamp(max=max_trust)
    p.add_(upd * trust, alpha=-lr)

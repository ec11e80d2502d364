"""Runs the reference's two count-sketch kernels (``communication/compressors/CountSketch.py:27-98``,
compiled from the reference's own source string through the stand-in loader) on one small matrix
and compares them with a NumPy restatement of the same arithmetic.  One GPU; prints ``ok``.

    python baseline/check_reference_kernels.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
sys.path[:] = [p for p in sys.path if os.path.abspath(p or os.getcwd()) != REPO]
sys.path.insert(0, HERE)


def _hash(v, rng, a, b):
    """CountSketch.py:7-18 on wrapping signed 32-bit integers (arithmetic right shifts)."""
    h = (np.int64(a) * v.astype(np.int64) + b).astype(np.int32)
    h = h ^ (h >> 16)
    h = (h.astype(np.int64) * 0x85EBCA6B).astype(np.int32)
    h = h ^ (h >> 13)
    h = (h.astype(np.int64) * 0xC2B2AE35).astype(np.int32)
    h = h ^ (h >> 16)
    return np.fmod(h, np.int32(rng))


def main():
    from compat import install

    install.install()
    import torch
    from communication.compressors.CountSketch import DenseCS

    torch.manual_seed(0)
    N, D, frac, beta = 6, 700, 0.1, 0.9
    cs = DenseCS(N, D, frac)
    W = cs.range
    cols = np.arange(D, dtype=np.int32)
    idx = _hash(cols, W, 994443, 609478)
    sign = np.where(_hash(cols, W, 994443 + 2, 609478 + 3) & 1, 1.0, -1.0).astype(np.float32)
    assert idx.min() >= 0 and idx.max() < W

    S = np.zeros((N, W), np.float32)
    for it in range(3):
        vec = torch.randn(N, D, device="cuda")
        v = vec.cpu().numpy()
        cs.update(vec, beta)
        old = S.copy()
        for j in range(D):
            S[:, idx[j]] += sign[j] * v[:, j] - (1 - beta) * old[:, idx[j]]
        torch.cuda.synchronize()
        got = cs.cs.cpu().numpy()
        assert np.allclose(got, S, rtol=1e-4, atol=1e-4), f"update {it}: max diff {np.abs(got - S).max()}"
        S = got.copy()                       # atomics sum in another order: follow the device copy

    grad = torch.randn(N, D, device="cuda")
    g = grad.cpu().numpy()
    cs.query(grad, 1 - beta)
    torch.cuda.synchronize()
    want = g + (1 - beta) * sign[None, :] * S[:, idx]
    assert np.allclose(grad.cpu().numpy(), want, rtol=1e-5, atol=1e-5), np.abs(grad.cpu().numpy() - want).max()
    print("ok")


if __name__ == "__main__":
    main()

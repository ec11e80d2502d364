"""Hash emulation, sketch algebra and persistence (CPU)."""
import ctypes as C
import pickle

import numpy as np
import pytest
import torch

from conef_b200.compressors import DenseCS, DenseCSHash3, HalfDenseCS, LowRankError, Quant8Error, TopKError
from conef_b200.ops import native
from conef_b200.ops import reference as ref


def _hash_c_semantics(v, rng, a, b):
    """Independent emulation with Python ints of signed-int32 C arithmetic."""
    def wrap(x):
        x &= 0xFFFFFFFF
        return x - (1 << 32) if x >= (1 << 31) else x
    h = wrap(a * v + b)
    h = wrap(h ^ (h >> 16))      # Python >> on negative ints is arithmetic
    h = wrap(h * 0x85EBCA6B)
    h = wrap(h ^ (h >> 13))
    h = wrap(h * 0xC2B2AE35)
    h = wrap(h ^ (h >> 16))
    assert h >= 0
    return h % rng


@pytest.mark.parametrize("D,W,a,b", [(5760, 576, 994443, 609478), (650, 65, 4113759, 2949676), (37, 1, 9171025, 2171464)])
def test_hash_matches_int32_emulation(D, W, a, b):
    got = ref.hash32(np.arange(D), W, a, b)
    want = np.array([_hash_c_semantics(j, W, a, b) for j in range(D)])
    assert np.array_equal(got, want)
    assert got.min() >= 0 and got.max() < W


@pytest.mark.parametrize("D,W", [(5760, 576), (650, 65), (1024, 102), (70, 64), (33278, 3327)])
def test_block_layout_of_the_hash(D, W):
    """Block layout: columns hashed in aligned groups of 32, one group per cell block and window.  The
    regrouped records must describe the same map as the column table, columns of one window never
    share a cell, and every cell block receives the same number of groups (give or take the last
    window)."""
    idx, sign = ref.hash_table(D, W, layout="block")
    idx, sign = idx.numpy(), sign.numpy()
    nb, ng = W // 32, (D + 31) // 32
    S = (ng + nb - 1) // nb
    assert idx.min() >= 0 and idx.max() < 32 * nb
    # inside an aligned group the 32 columns take 32 different lanes of ONE cell block
    for g in (0, ng // 2, ng - 1):
        cols = np.arange(32 * g, min(32 * g + 32, D))
        assert len(set(idx[cols] // 32)) == 1 and len(set(idx[cols] % 32)) == len(cols)
    # inside a window no two columns share a cell
    for s in (0, S - 1):
        cols = np.arange(32 * nb * s, min(32 * nb * (s + 1), D))
        assert len(set(idx[cols])) == len(cols)
    counts = np.bincount(idx, minlength=W)
    assert counts[:32 * nb].max() - counts[:32 * nb].min() <= 1 and counts[32 * nb:].sum() == 0
    rec = ref.block_csr(D, W, ref.DEFAULT_A, ref.DEFAULT_B).view(np.uint32).reshape(S, nb, 2)
    seen = np.zeros(D, dtype=bool)
    for s in range(S):
        for c in range(nb):
            word, bits = int(rec[s, c, 0]), int(rec[s, c, 1])
            g, x = word & ref.NO_GROUP, word >> 27
            if g == ref.NO_GROUP:
                continue
            assert s * nb <= g < (s + 1) * nb
            lanes = np.arange(32)
            cols = 32 * g + (lanes ^ x)
            ok = cols < D
            assert np.array_equal(idx[cols[ok]], 32 * c + lanes[ok])
            assert np.array_equal(sign[cols[ok]] > 0, ((bits >> (lanes[ok] ^ x)) & 1).astype(bool))
            seen[cols[ok]] = True
    assert seen.all()


def test_block_layout_is_an_unbiased_sketch(monkeypatch):
    """Query after update returns the vector plus zero-mean noise whose energy matches the count-sketch
    bound (each cell holds about D / W columns)."""
    monkeypatch.setenv("CONEF_HASH", "block")
    N, D = 64, 2048
    torch.manual_seed(0)
    v = torch.randn(N, D)
    cs = DenseCS(N, D, 0.125, device="cpu")
    assert cs.range == 256
    cs.update(v.clone(), 1.0)
    est = torch.zeros(N, D)
    cs.query(est, 1.0)
    err = est - v
    assert abs(float(err.mean())) < 0.05
    # per-element noise variance = (colliders per cell) * var(v) = (D / W - 1) = 7
    assert 5.5 < float(err.var()) < 8.5
    monkeypatch.setenv("CONEF_HASH", "universal")
    cs2 = DenseCS(N, D, 0.125, device="cpu")
    cs2.update(v.clone(), 1.0)
    est2 = torch.zeros(N, D)
    cs2.query(est2, 1.0)
    assert float((est2 - v).var()) > 0.9 * float(err.var())      # the block layout is not noisier


def test_sign_split_reference_config():
    idx, sign = ref.hash_table(5760, 576)
    assert idx.min() == 0 and idx.max() == 575
    assert abs(float((sign > 0).float().mean()) - 0.509) < 5e-3


@pytest.mark.skipif(not native.available(), reason="native library not built")
@pytest.mark.parametrize("layout", ["universal", "block"])
def test_cpp_hash_table_matches_python(layout):
    D, W = 1000, 77
    tab = np.zeros(D, dtype=np.int32)
    cnt = np.zeros(W, dtype=np.int32)
    native.lib().conef_cpu_hash_table(tab.ctypes.data, cnt.ctypes.data, D, W, ref.DEFAULT_A, ref.DEFAULT_B, 2, 3,
                                      int(layout == "block"))
    assert np.array_equal(tab, ref.packed_hash_table(D, W, ref.DEFAULT_A, ref.DEFAULT_B, layout=layout))
    idx, _ = ref.hash_table(D, W, layout=layout)
    assert np.array_equal(cnt, np.bincount(idx.numpy(), minlength=W))


@pytest.mark.skipif(not native.available(), reason="native library not built")
def test_cpp_sketch_matches_torch():
    N, D, W = 5, 300, 30
    torch.manual_seed(0)
    cs = DenseCS(N, D, 0.1, device="cpu")
    v = torch.randn(N, D)
    cs.update(v.clone(), 0.9)
    cs.update(torch.randn(N, D), 0.9)
    idx, sign = ref.hash_table(D, W)
    packed = ref.packed_hash_table(D, W, ref.DEFAULT_A, ref.DEFAULT_B).copy()
    counts = np.bincount(idx.numpy(), minlength=W).astype(np.int32)
    c2 = np.zeros((N, W), dtype=np.float32)
    lib = native.lib()
    torch.manual_seed(0)
    v1 = torch.randn(N, D).numpy().copy()
    lib.conef_cpu_sketch_update(v1.ctypes.data, c2.ctypes.data, packed.ctypes.data, counts.ctypes.data, N, D, W, 0.9)
    v2 = torch.randn(N, D).numpy().copy()
    lib.conef_cpu_sketch_update(v2.ctypes.data, c2.ctypes.data, packed.ctypes.data, counts.ctypes.data, N, D, W, 0.9)
    np.testing.assert_allclose(c2, cs.cs.numpy(), rtol=1e-5, atol=1e-5)
    m1 = torch.randn(N, D)
    m2 = m1.numpy().copy()
    cs.query(m1, 0.1)
    lib.conef_cpu_sketch_query(m2.ctypes.data, c2.ctypes.data, packed.ctypes.data, N, D, W, 0.1)
    np.testing.assert_allclose(m2, m1.numpy(), rtol=1e-5, atol=1e-5)


def test_sketch_linearity_and_decay():
    N, D = 4, 200
    a, b = torch.randn(N, D), torch.randn(N, D)
    s1, s2, s3 = (DenseCS(N, D, 0.2, device="cpu") for _ in range(3))
    s1.update(a, 1.0); s1.update(b, 1.0)       # beta = 1: pure accumulation
    s3.update(a + b, 1.0)
    torch.testing.assert_close(s1.cs, s3.cs)
    # update semantics: cs <- cs (1 - (1-beta) k_h) + sketch(v), as the reference kernel
    idx, sign = ref.hash_table(D, s2.range)
    s2.update(a, 1.0)
    old = s2.cs.clone()
    s2.update(b, 0.9)
    cnt = torch.bincount(idx, minlength=s2.range).float()
    want = old * (1 - 0.1 * cnt)
    want.index_add_(1, idx, b * sign)
    torch.testing.assert_close(s2.cs, want)


def test_query_is_transpose_of_sketch():
    N, D = 3, 64
    cs = DenseCS(N, D, 0.25, device="cpu")
    cs.cs.normal_()
    idx, sign = ref.hash_table(D, cs.range)
    g = torch.zeros(N, D)
    cs.query(g, 0.5)
    torch.testing.assert_close(g, 0.5 * cs.cs[:, idx] * sign)
    # exact per-element reference formula
    for j in (0, 17, 63):
        assert torch.allclose(g[:, j], 0.5 * sign[j] * cs.cs[:, idx[j]])


def test_width_one_and_small():
    cs = DenseCS(2, 5, 0.01, device="cpu")
    assert cs.range == 1
    v = torch.randn(2, 5)
    cs.update(v, 1.0)
    _, sign = ref.hash_table(5, 1)
    torch.testing.assert_close(cs.cs[:, 0], (v * sign).sum(1))


def test_half_sketch_tracks_fp32():
    N, D = 4, 128
    v = torch.randn(N, D)
    a, b = DenseCS(N, D, 0.25, device="cpu"), HalfDenseCS(N, D, 0.25, device="cpu")
    a.update(v, 0.9); b.update(v, 0.9)
    assert b.cs.dtype == torch.float16 and b.nbytes() * 2 == a.nbytes()
    torch.testing.assert_close(b.cs.float(), a.cs, rtol=2e-3, atol=2e-3)


def test_hash3_median_and_consistent_sign_hash():
    N, D = 3, 90
    cs = DenseCSHash3(N, D, 0.5, device="cpu")
    v = torch.randn(N, D)
    cs.update(v, 1.0)
    g = torch.zeros(N, D)
    cs.query(g, 1.0)
    tabs = cs._tables()
    est = [c[:, t[0]] * t[1] for c, t in zip(cs._rows(), tabs)]
    torch.testing.assert_close(g, ref.median3(*est))
    # with a wide sketch most coordinates are recovered exactly by the median
    big = DenseCSHash3(N, D, 4.0, device="cpu")
    big.update(v, 1.0)
    g2 = torch.zeros(N, D)
    big.query(g2, 1.0)
    assert (g2 - v).abs().lt(1e-5).float().mean() > 0.8


@pytest.mark.parametrize("cls", [DenseCS, HalfDenseCS, DenseCSHash3])
def test_sketch_state_roundtrip(cls):
    cs = cls(6, 50, 0.2, device="cpu", seed=11)
    cs.update(torch.randn(6, 50), 0.9)
    blob = pickle.dumps(cs)
    other = pickle.loads(blob)
    g1, g2 = torch.zeros(6, 50), torch.zeros(6, 50)
    cs.query(g1, 0.3); other.query(g2, 0.3)     # needs the hash seeds: the reference loses them
    assert torch.equal(g1, g2)
    sd = cs.state_dict()
    assert {"N", "D", "blk_size", "range"} <= set(sd)
    third = cls(6, 50, 0.2, device="cpu", seed=11)
    third.load_state_dict(sd)
    g3 = torch.zeros(6, 50)
    third.query(g3, 0.3)
    assert torch.equal(g1, g3)


def test_quant8_roundtrip_and_contract():
    x = torch.randn(3, 300)
    q = Quant8Error(3, 300, device="cpu")
    q.update(x, 0.0)
    back = torch.zeros(3, 300)
    q.query(back, 1.0)
    # error bounded by half a quantisation step of each 256-element group
    flat, bflat = x.view(-1), back.view(-1)
    for gidx in range(q.scales.numel()):
        sl = slice(gidx * 256, min((gidx + 1) * 256, flat.numel()))
        assert (flat[sl] - bflat[sl]).abs().max() <= q.scales[gidx] * 0.5 + 1e-7
    assert q.nbytes() == 900 + 4 * 4
    # beta keeps a fraction of the old error
    q.update(torch.zeros(3, 300), 0.5)
    half = torch.zeros(3, 300)
    q.query(half, 1.0)
    torch.testing.assert_close(half, 0.5 * back, atol=2e-2, rtol=0)


def test_topk_keeps_largest():
    t = TopKError(4, 25, topk_ratio=0.4, device="cpu")
    v = torch.randn(4, 25)
    t.update(v, 0.0)
    k = max(1, int(0.5 * 0.4 * 100))
    assert int((t.err != 0).sum()) == k
    thresh = v.abs().view(-1).topk(k).values.min()
    assert t.err[t.err != 0].abs().min() >= thresh


def test_lowrank_recovers_lowrank_error():
    torch.manual_seed(1)
    u, v = torch.randn(40, 2), torch.randn(30, 2)
    target = u @ v.t()
    lr = LowRankError(40, 30, rank=2, device="cpu")
    for _ in range(4):
        lr.update(target, 0.0)
    out = torch.zeros(40, 30)
    lr.query(out, 1.0)
    torch.testing.assert_close(out, target, rtol=1e-3, atol=1e-3)
    assert lr.nbytes() == (40 + 30) * 2 * 4




def test_dense_cs_on_cpu_host_loops_equal_the_pytorch_ops(monkeypatch):
    """CPU tensors go through the library's host loops when it is built; ``CONEF_BACKEND=torch`` keeps the
    PyTorch ops.  Both must give the same sketch and the same query."""
    from conef_b200.compressors import DenseCS
    from conef_b200.ops import native
    if not native.available():
        pytest.skip("native library not built")
    torch.manual_seed(0)
    v1, v2, g = torch.randn(5, 301), torch.randn(5, 301), torch.randn(5, 301)

    def run(backend):
        monkeypatch.setenv("CONEF_BACKEND", backend)
        cs = DenseCS(5, 301, 0.1, device="cpu", seed=3)
        cs.update(v1.clone(), 0.9)
        cs.update(v2.clone(), 0.9)
        out = g.clone()
        cs.query(out, 0.5)
        return cs.cs.clone(), out
    (c_host, q_host), (c_torch, q_torch) = run("native"), run("torch")
    torch.testing.assert_close(c_host, c_torch, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(q_host, q_torch, rtol=1e-5, atol=1e-5)
    assert not torch.equal(q_host, g)

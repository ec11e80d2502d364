"""The allocation-free LAMB entry point, called through its exported C symbol.

Some users of this library run the optimizer where device memory may not be
allocated (memory handed out once by an external pool, or a C/C++ embedder with no
caching allocator).  ``conef_lamb_step_noalloc`` serves them by keeping its norm
scratch in static device memory.  This test loads the shared object with plain
``ctypes`` (not the package's binding), runs the new entry point and the regular
``conef_lamb_step`` on identical copies of the same tensors for two steps in a row
— the second call reuses the scratch the first one dirtied — and expects the same
parameters and moments.  The file name sorts last so that a ``-x`` run has already
executed every other test when this one starts.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from conef_b200.ops import native

pytestmark = pytest.mark.gpu
CHUNK = 65536
MAX_TENSORS = 4096


def _load():
    lib = C.CDLL(str(native.so_path()))
    vp, f, i = C.c_void_p, C.c_float, C.c_int
    lib.conef_lamb_step_noalloc.argtypes = [vp, i, vp, i, i, f, f, f, f, i, i, f, f, vp]
    lib.conef_lamb_step_noalloc.restype = i
    lib.conef_lamb_step.argtypes = [vp, i, vp, i, i, vp, f, f, f, f, i, i, f, f, vp]
    lib.conef_lamb_step.restype = i
    lib.conef_last_error.restype = C.c_char_p
    return lib


def _tables(params, grads, ms, vs, wd, dev):
    rec = np.zeros(len(params), dtype=native.LAMB_DTYPE)
    chunks = []
    for t, (p, g, m, v) in enumerate(zip(params, grads, ms, vs)):
        rec[t] = (p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), wd, 0)
        chunks += [(t, c) for c in range((p.numel() + CHUNK - 1) // CHUNK)]
    return (native.upload_struct_array(rec, dev), torch.from_numpy(np.asarray(chunks, dtype=np.int32)).to(dev),
            len(chunks))


def test_noalloc_lamb_matches_regular_entry_point_twice():
    lib = _load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(7)
    shapes = [(513, 77), (77,), (3, 3, 3), (150001,)]

    def fresh():
        g = torch.Generator().manual_seed(1)
        ps = [torch.randn(s, generator=g).to(dev) for s in shapes]
        return ps, [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
    pa, ma, va = fresh()
    pb, mb, vb = fresh()
    norms = torch.zeros(1 + 2 * len(shapes), device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    for step in (1, 2):                       # two calls in a row: the second reuses dirtied scratch
        gen = torch.Generator().manual_seed(100 + step)
        grads = [torch.randn(s, generator=gen) * 2 for s in shapes]
        ga = [x.clone().to(dev) for x in grads]
        gb = [x.clone().to(dev) for x in grads]
        ta, ca, na = _tables(pa, ga, ma, va, 0.01, dev)
        tb, cb_, nb = _tables(pb, gb, mb, vb, 0.01, dev)
        rc = lib.conef_lamb_step_noalloc(ta.data_ptr(), len(shapes), ca.data_ptr(), na, CHUNK, 1e-2, 0.9, 0.999, 1e-6,
                                         step, 1, 1.0, 1.0, stream)
        assert rc == 0, lib.conef_last_error()
        rc = lib.conef_lamb_step(tb.data_ptr(), len(shapes), cb_.data_ptr(), nb, CHUNK, norms.data_ptr(), 1e-2, 0.9,
                                 0.999, 1e-6, step, 1, 1.0, 1.0, stream)
        assert rc == 0, lib.conef_last_error()
        torch.cuda.synchronize()
        for a, b in zip(pa + ma + va, pb + mb + vb):
            torch.testing.assert_close(a, b, rtol=2e-4, atol=2e-5)
    assert all(torch.isfinite(p).all() for p in pa)


def test_noalloc_lamb_rejects_oversized_request():
    lib = _load()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    dummy = torch.zeros(16, device="cuda")
    rc = lib.conef_lamb_step_noalloc(dummy.data_ptr(), MAX_TENSORS + 1, dummy.data_ptr(), 1, CHUNK, 1e-2, 0.9, 0.999,
                                     1e-6, 1, 1, 1.0, 1.0, stream)
    assert rc != 0
    assert b"exceed" in lib.conef_last_error()

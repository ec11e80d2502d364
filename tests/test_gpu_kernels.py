"""Numerics of every CUDA kernel against the plain PyTorch fp32 reference (needs a B200)."""
import ctypes as C

import numpy as np
import pytest
import torch

import conef_b200 as cb
from conef_b200.compressors import DenseCS, DenseCSHash3, HalfDenseCS, Quant8Error
from conef_b200.ops import native
from conef_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _st():
    return native.stream_ptr(torch.device(DEV))


def test_native_library_is_loaded():
    assert native.lib().conef_version() >= 100


@pytest.mark.parametrize("layout", ["universal", "block"])
@pytest.mark.parametrize("D,W", [(5760, 576), (650, 65), (33, 1), (1024, 409)])
def test_hash_table_kernel(D, W, layout):
    tab = torch.zeros(D, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(W, dtype=torch.int32, device=DEV)
    native.check(native.lib().conef_build_hash_table(tab.data_ptr(), cnt.data_ptr(), D, W, ref.DEFAULT_A,
                                                     ref.DEFAULT_B, 2, 3, int(layout == "block"), _st()))
    want = ref.packed_hash_table(D, W, ref.DEFAULT_A, ref.DEFAULT_B, layout=layout)
    assert np.array_equal(tab.cpu().numpy(), want)
    idx, _ = ref.hash_table(D, W, layout=layout)
    assert np.array_equal(cnt.cpu().numpy(), np.bincount(idx.numpy(), minlength=W))


@pytest.mark.parametrize("cls", [DenseCS, HalfDenseCS, DenseCSHash3])
@pytest.mark.parametrize("N,D,size", [(7, 333, 0.1), (64, 576, 0.1), (3, 50, 0.01), (130, 1030, 0.5)])
def test_sketch_kernels_match_reference(cls, N, D, size):
    torch.manual_seed(0)
    g, c = cls(N, D, size, device=DEV), cls(N, D, size, device="cpu")
    tol = dict(rtol=2e-3, atol=2e-3) if cls is HalfDenseCS else dict(rtol=1e-4, atol=1e-4)
    for step in range(3):
        v = torch.randn(N, D)
        g.update(v.to(DEV), 0.9)
        c.update(v.clone(), 0.9)
        m = torch.randn(N, D)
        mg = m.to(DEV)
        g.query(mg, 0.1)
        c.query(m, 0.1)
        torch.testing.assert_close(mg.cpu(), m, **tol)
    rows_g = g._rows() if cls is DenseCSHash3 else (g.cs,)
    rows_c = c._rows() if cls is DenseCSHash3 else (c.cs,)
    for a, b in zip(rows_g, rows_c):
        torch.testing.assert_close(a.float().cpu(), b.float(), **tol)


def test_quant8_kernels_match_reference():
    torch.manual_seed(1)
    g, c = Quant8Error(5, 1000, device=DEV), Quant8Error(5, 1000, device="cpu")
    for _ in range(3):
        v = torch.randn(5, 1000)
        g.update(v.to(DEV), 0.5)
        c.update(v.clone(), 0.5)
    # codes may differ by one step where a value sits on a rounding boundary
    assert (g.codes.cpu().int() - c.codes.int()).abs().max() <= 1
    torch.testing.assert_close(g.scales.cpu(), c.scales, rtol=1e-5, atol=1e-7)
    x = torch.randn(5, 1000)
    xg = x.to(DEV)
    g.query(xg, 0.7)
    c.query(x, 0.7)
    torch.testing.assert_close(xg.cpu(), x, rtol=0, atol=float(c.scales.max()) * 0.8)


def test_fill_normal_is_deterministic_and_normal():
    a = torch.empty(1_000_003, device=DEV)
    b = torch.empty(1_000_003, device=DEV)
    lib = native.lib()
    native.check(lib.conef_fill_normal(a.data_ptr(), a.numel(), 12345, _st()))
    native.check(lib.conef_fill_normal(b.data_ptr(), b.numel(), 12345, _st()))
    assert torch.equal(a, b)
    native.check(lib.conef_fill_normal(b.data_ptr(), b.numel(), 12346, _st()))
    assert not torch.equal(a, b)
    assert abs(float(a.mean())) < 5e-3 and abs(float(a.std()) - 1) < 5e-3
    assert torch.isfinite(a).all()


def test_lamb_kernel_matches_reference():
    from conef_b200.optim import FusedLAMB

    torch.manual_seed(2)
    shapes = [(300, 70), (70,), (1, 5), (200000,)]
    pg = [torch.nn.Parameter(torch.randn(s, device=DEV)) for s in shapes]
    pc = [torch.nn.Parameter(p.detach().cpu().clone()) for p in pg]
    og = FusedLAMB([{"params": pg[:2], "weight_decay": 0.01}, {"params": pg[2:], "weight_decay": 0.0}], lr=1e-2)
    oc = FusedLAMB([{"params": pc[:2], "weight_decay": 0.01}, {"params": pc[2:], "weight_decay": 0.0}], lr=1e-2)
    for _ in range(3):
        for a, b in zip(pg, pc):
            g = torch.randn(a.shape) * 3
            a.grad, b.grad = g.to(DEV), g.clone()
        og.step()
        oc.step()
    for a, b in zip(pg, pc):
        torch.testing.assert_close(a.detach().cpu(), b.detach(), rtol=2e-4, atol=2e-5)


def test_bounded_wait_gives_up_and_process_survives():
    """A wait on a flag nobody sets returns an error status instead of hanging."""
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    native.check(native.lib().conef_wait_flags(flags.data_ptr(), 2, 5, status.data_ptr(), 2000, _st()))
    torch.cuda.synchronize()
    assert int(status[0]) == 1
    # the context is still usable
    assert float(torch.ones(4, device=DEV).sum()) == 4.0


def test_oneshot_allreduce_math_with_preset_flags():
    """Two 'ranks' emulated as two buffers on one GPU with the flags already published."""
    n = 10_007
    a, b = torch.randn(n, device=DEV), torch.randn(n, device=DEV)
    out = torch.empty(n, device=DEV)
    ptrs = torch.tensor([a.data_ptr(), b.data_ptr()], dtype=torch.int64, device=DEV)
    flags = torch.full((8,), 3, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    native.check(native.lib().conef_allreduce_oneshot(out.data_ptr(), ptrs.data_ptr(), 0, flags.data_ptr(), 2, 0, 3,
                                                      n, 0.5, status.data_ptr(), 1000, _st()))
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    torch.testing.assert_close(out, (a + b) * 0.5)


def test_orthogonalize_kernel():
    """Row-parallel Gram-Schmidt (Gram matrix, applied twice) against the column-by-column oracle."""
    torch.manual_seed(3)
    shapes = [(1000, 4), (37, 3), (5000, 8), (9, 1), (30528, 8), (700, 20)]
    mats = np.zeros(len(shapes), dtype=native.MAT_DTYPE)
    off, tiles = 0, []
    for k, (n, r) in enumerate(shapes):
        mats[k]["n"], mats[k]["m"], mats[k]["r"], mats[k]["p_off"] = n, 1, r, off
        off += n * r
        tiles += [(k, c) for c in range((n + 511) // 512)]
    flat = torch.randn(off)
    dev = flat.to(DEV)
    md = native.upload_struct_array(mats, torch.device(DEV))
    td = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    gram = torch.zeros(2 * len(tiles) * 1024, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    native.check(native.lib().conef_orthogonalize_packed(md.data_ptr(), td.data_ptr(), len(tiles), len(shapes), 0,
                                                         dev.data_ptr(), 0.0, 0, 0, 1, 0, status.data_ptr(), 0, 0, 16,
                                                         gram.data_ptr(), _st()))
    got = dev.cpu()
    off = 0
    for n, r in shapes:
        want = flat[off : off + n * r].view(n, r).clone()
        ref.gram_schmidt_ref(want)
        g = got[off : off + n * r].view(n, r)
        torch.testing.assert_close(g, want, rtol=1e-3, atol=1e-4)
        torch.testing.assert_close(g.t() @ g, torch.eye(r), rtol=0, atol=1e-4)
        off += n * r


def _orth_on_device(blocks, eps=0.0, which=0, one_launch=False, cluster=False):
    """Runs the native orthogonalisation on a list of (n x r) CPU blocks; returns the results.
    ``one_launch``: the single-kernel form with two barriers among its CTAs; ``cluster``: one
    thread-block cluster per block (Gram partials through distributed shared memory)."""
    mats = np.zeros(len(blocks), dtype=native.MAT_DTYPE)
    off, tiles = 0, []
    for k, b in enumerate(blocks):
        n, r = b.shape
        mats[k]["n"], mats[k]["m"], mats[k]["r"], mats[k]["p_off"] = n, 1, r, off
        off += n * r
        tiles += [(k, c) for c in range((n + 511) // 512)]
    dev = torch.cat([b.reshape(-1) for b in blocks]).float().to(DEV)
    md = native.upload_struct_array(mats, torch.device(DEV))
    td = torch.tensor(tiles + [(k, b.shape[0]) for k, b in enumerate(blocks)], dtype=torch.int32, device=DEV)
    gram = torch.zeros(2 * len(tiles) * 1024, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    if cluster:
        extra = native.OrthExtra()
        extra.max_rank = max(b.shape[1] for b in blocks)
        extra.cl_list, extra.cl_nmat = td.data_ptr() + 8 * len(tiles), len(blocks)
        extra.cl_max_rows = max(b.shape[0] for b in blocks)
        native.check(native.lib().conef_orthogonalize_fused(md.data_ptr(), td.data_ptr(), len(tiles), which,
                                                            dev.data_ptr(), eps, 0, 0, 1, 0, status.data_ptr(), 0, 0, 16,
                                                            gram.data_ptr(), 0, C.byref(extra), _st()))
        torch.cuda.synchronize()
        # blocks taller than 8 x 1024 rows go to the chunked forms (here, without barrier words: three launches)
        want_launches = 1 if extra.cl_max_rows <= 8 * 1024 else 3
        assert native.lib().conef_orth_last_launches() == want_launches, "unexpected form"
        assert int(status[0]) == 0
    elif one_launch:
        bar = torch.zeros(2, dtype=torch.int32, device=DEV)
        extra = native.OrthExtra()
        extra.bar, extra.max_rank = bar.data_ptr(), max(b.shape[1] for b in blocks)
        native.check(native.lib().conef_orthogonalize_fused(md.data_ptr(), td.data_ptr(), len(tiles), which,
                                                            dev.data_ptr(), eps, 0, 0, 1, 0, status.data_ptr(), 0, 0, 16,
                                                            gram.data_ptr(), 0, C.byref(extra), _st()))
        torch.cuda.synchronize()
        assert native.lib().conef_orth_last_launches() == 1, "the one-launch form was not taken"
        assert int(status[0]) == 0 and int(bar[0]) == 0 and int(bar[1]) == 2      # two barriers passed
    else:
        native.check(native.lib().conef_orthogonalize_packed(md.data_ptr(), td.data_ptr(), len(tiles), len(blocks),
                                                             which, dev.data_ptr(), eps, 0, 0, 1, 0, status.data_ptr(),
                                                             0, 0, 16, gram.data_ptr(), _st()))
    got, out, off = dev.cpu(), [], 0
    for b in blocks:
        out.append(got[off : off + b.numel()].view_as(b))
        off += b.numel()
    return out


@pytest.mark.parametrize("shapes", [[(1000, 4), (37, 3), (5000, 8), (9, 1), (30528, 8)], [(700, 20), (2000, 16)],
                                    [(1500, 32), (600, 27)]], ids=["r<=8", "r<=32a", "r<=32b"])
@pytest.mark.parametrize("form", ["one_launch", "cluster"])
def test_orthogonalize_one_launch_matches_three_kernels(shapes, form):
    """The single-launch forms (rows kept in shared memory; two barriers among all CTAs, or one
    thread-block cluster per block with Gram partials read through distributed shared memory) against
    the three-kernel form and the column-by-column oracle, including a zero column and blocks with
    fewer rows than a cluster has CTAs."""
    torch.manual_seed(7)
    blocks = [torch.randn(n, r) for n, r in shapes]
    blocks[0][:, -1] = 0
    one = _orth_on_device([b.clone() for b in blocks], one_launch=form == "one_launch", cluster=form == "cluster")
    three = _orth_on_device([b.clone() for b in blocks], one_launch=False)
    for k, (b, x, y) in enumerate(zip(blocks, one, three)):
        torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-5)
        r = b.shape[1]
        keep = list(range(r - 1)) if k == 0 else list(range(r))
        if keep:
            want = b[:, keep].clone()
            ref.gram_schmidt_ref(want)
            torch.testing.assert_close(x[:, keep], want, rtol=2e-3, atol=2e-4)
            torch.testing.assert_close(x[:, keep].t() @ x[:, keep], torch.eye(len(keep)), rtol=0, atol=1e-4)
    assert 0.8 < float(one[0][:, -1].norm()) < 1.2            # the zero column was refilled


@pytest.mark.parametrize("relres", [1e-3, 1e-4, 1e-5, 1e-6])
def test_orthogonalize_kernel_keeps_nearly_dependent_columns(relres):
    """Columns within ``relres`` of the span of earlier ones stay alive, come out orthonormal and
    agree with the CPU restatement of the same algorithm."""
    g = torch.Generator().manual_seed(11)
    blocks = []
    for n in (2000, 30528):
        a = torch.randn(n, 8, generator=g, dtype=torch.float64)
        a[:, 3] = 0.7 * a[:, 0] - 1.3 * a[:, 1] + relres * torch.randn(n, generator=g, dtype=torch.float64)
        a[:, 6] = a[:, 2] + a[:, 5] + relres * torch.randn(n, generator=g, dtype=torch.float64)
        blocks.append(a.float())
    for a, q in zip(blocks * 3, _orth_on_device(blocks) + _orth_on_device(blocks, one_launch=True)
                    + _orth_on_device(blocks, cluster=True)):
        q = q.double()
        assert bool((q.norm(dim=0) > 0.99).all()), q.norm(dim=0)
        torch.testing.assert_close(q.t() @ q, torch.eye(8, dtype=torch.float64), rtol=0, atol=1e-4)
        want = a.double()
        ref.gram_schmidt_ref(want)
        resid = want - q @ (q.t() @ want)
        assert float(resid.norm(dim=0).max()) < 2e-7 / relres + 1e-4


def test_orthogonalize_kernel_refills_a_zero_column():
    """An all-zero column has no direction to keep: it is replaced by fixed pseudo-random values of
    about unit norm (identical in every call, hence on every rank), the others are untouched."""
    torch.manual_seed(2)
    a = torch.randn(3000, 4)
    a[:, 2] = 0
    q1, = _orth_on_device([a.clone()])
    q2, = _orth_on_device([a.clone()])
    assert torch.equal(q1, q2)
    assert 0.9 < float(q1[:, 2].norm()) < 1.1
    keep = [0, 1, 3]
    want = a[:, keep].clone()
    ref.gram_schmidt_ref(want)
    torch.testing.assert_close(q1[:, keep], want, rtol=1e-3, atol=1e-4)
    assert float((q1[:, keep].t() @ q1[:, 2]).abs().max()) < 0.1


def test_hook_path_sees_a_wait_that_gave_up_without_a_host_sync():
    """The status word is copied to pinned memory behind a step's kernels; a later hook call raises."""
    import conef_b200 as cb

    state = cb.PowerSGDState(None, start_powerSGD_iter=2)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream()
    state.post_status(status, stream)
    torch.cuda.synchronize()
    state.poll_status()                               # clean word: nothing happens
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    native.check(native.lib().conef_wait_flags(flags.data_ptr(), 2, 5, status.data_ptr(), 2000, _st()))
    state.post_status(status, stream)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="wait gave up"):
        state.poll_status()
    assert int(status[0]) == 0                        # cleared for the next step
    state.poll_status()


def test_runtime_compiled_kernel_loader():
    """A CUDA source string compiled at run time for the device's architecture and launched on torch's stream."""
    from conef_b200.ops.jit import JitKernel

    src = r'''
    extern "C" __global__ void axpy(float* y, const float* x, float a, int n) {
      int i = blockIdx.x * blockDim.x + threadIdx.x;
      if (i < n) y[i] += a * x[i];
    }'''
    k = JitKernel(src, "axpy")
    assert JitKernel.compute_arch().startswith("sm_")
    x, y = torch.randn(1000, device=DEV), torch.randn(1000, device=DEV)
    want = y + 2.5 * x
    k(grid=(4, 1, 1), block=(256, 1, 1), args=[y, x, 2.5, 1000])
    torch.cuda.synchronize()
    torch.testing.assert_close(y, want)


def test_grouped_topk_matches_torch_topk():
    """Radix select over several matrices at once against torch.topk per matrix."""
    import math
    shapes = [(300, 257), (1, 1), (7, 3), (2048, 513), (64, 64)]
    ratio = 0.4
    lib = native.lib()
    mats = np.zeros(len(shapes), dtype=native.MAT_DTYPE)
    off, chunks = 3, []          # an odd start: the kernels may not assume alignment
    ch = lib.conef_topk_chunk()
    for k, (n, m) in enumerate(shapes):
        mats[k]["g_off"], mats[k]["n"], mats[k]["m"] = off, n, m
        chunks += [(k, c) for c in range(math.ceil(n * m / ch))]
        off += n * m + 5
    g = torch.Generator().manual_seed(3)
    err = torch.randn(off, generator=g).to(DEV)
    n4, m4 = shapes[4]
    o4 = int(mats[4]["g_off"])
    err[o4 : o4 + n4 * m4][::2] = 0.0          # half zeros: the threshold lands among real values
    want = err.clone()
    for k, (n, m) in enumerate(shapes):
        o = int(mats[k]["g_off"])
        ref.topk_keep_(want[o : o + n * m].view(n, m), ratio)
    guard = err.clone()
    tiles = torch.from_numpy(np.asarray(chunks, dtype=np.int32)).to(DEV)
    scratch = torch.zeros(len(shapes) * 2050, dtype=torch.int32, device=DEV)
    mats_dev = native.upload_struct_array(mats, DEV)
    for _ in range(2):                          # the second call must find its scratch clean
        got = err.clone()
        native.check(lib.conef_topk_keep(mats_dev.data_ptr(), len(shapes), tiles.data_ptr(), len(chunks),
                                         got.data_ptr(), ratio, scratch.data_ptr(), native.stream_ptr()))
        torch.cuda.synchronize()
        for k, (n, m) in enumerate(shapes):
            o = int(mats[k]["g_off"])
            a, b = got[o : o + n * m], want[o : o + n * m]
            assert int((a != 0).sum()) == int((b != 0).sum()) == min(
                max(1, int(0.5 * ratio * n * m)), int((err[o : o + n * m] != 0).sum()))
            torch.testing.assert_close(a, b, rtol=0, atol=0)
        # the gaps between the matrices are untouched
        mask = torch.ones(off, dtype=torch.bool, device=DEV)
        for k, (n, m) in enumerate(shapes):
            o = int(mats[k]["g_off"])
            mask[o : o + n * m] = False
        assert torch.equal(got[mask], guard[mask])
    assert int(scratch[: len(shapes) * 2048].abs().sum()) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(128, 160, 32, 32), (7, 16, 5, 3), (33, 640, 8, 8), (3, 2048, 2, 2), (5, 24, 1, 1)])
def test_channel_sum_kernel(shape, dtype):
    """Column sums of a channels-last gradient (the bias gradient of a convolution) against an fp32 sum."""
    from conef_b200.ops.colsum import channel_sum
    torch.manual_seed(0)
    t = torch.randn(shape, device=DEV).to(dtype).contiguous(memory_format=torch.channels_last)
    before = native.reset_launch_count()
    got = channel_sum(t)
    assert native.reset_launch_count() >= 1, "the native kernel did not run"
    want = t.float().sum(dim=(0, 2, 3))
    scale = float(t.float().abs().sum(dim=(0, 2, 3)).max())
    assert got.dtype == torch.float32 and got.shape == want.shape
    assert float((got - want).abs().max()) <= 2e-6 * scale + 1e-5
    # shapes the kernel does not take go through the library sum
    odd = torch.randn(4, 6, 3, 3, device=DEV).contiguous(memory_format=torch.channels_last)
    torch.testing.assert_close(channel_sum(odd), odd.sum(dim=(0, 2, 3)))


def test_conv_layer_bias_gradient_matches_torch():
    """``models.layers.Conv2d`` against ``nn.Conv2d``: same outputs, same input / weight gradients, bias
    gradient from the column-sum kernel (bf16 autocast, channels-last, strides and 1x1 kernels)."""
    from conef_b200.models.layers import Conv2d
    torch.manual_seed(1)
    for cin, cout, k, stride in ((16, 32, 3, 1), (32, 64, 3, 2), (24, 40, 1, 2)):
        ref_conv = torch.nn.Conv2d(cin, cout, k, stride=stride, padding=k // 2).to(DEV).to(memory_format=torch.channels_last)
        own = Conv2d(cin, cout, k, stride=stride, padding=k // 2).to(DEV).to(memory_format=torch.channels_last)
        own.load_state_dict(ref_conv.state_dict())
        x = torch.randn(8, cin, 12, 12, device=DEV).contiguous(memory_format=torch.channels_last)
        outs = []
        for conv in (ref_conv, own):
            xi = x.clone().requires_grad_(True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = conv(xi)
                loss = (y.float() * torch.linspace(-1, 1, y.numel(), device=DEV).view_as(y)).sum()
            loss.backward()
            outs.append((y.detach().float(), xi.grad.float(), conv.weight.grad.float(), conv.bias.grad.float()))
        for a, b in zip(*outs):
            torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-2)
        # the bias gradient is an fp32 sum of the bf16 output gradient: tighter than bf16 accumulation
        assert outs[1][3].dtype == torch.float32


@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_batch_norm_layer_matches_torch(dtype, relu):
    """``models.layers.BatchNorm2d`` (statistics, normalisation (+ ReLU), backward sums and input gradient
    on the column kernels) against ``nn.BatchNorm2d`` (+ ``F.relu``) in training mode: outputs, gradients
    and running statistics, with a mean far from zero (the shifted sums must not lose the variance) and a
    channel count of every slab layout."""
    from conef_b200.models.layers import BatchNorm2d
    torch.manual_seed(3)
    for n, c, h, w in ((16, 160, 8, 8), (4, 16, 7, 5), (9, 640, 3, 3)):
        ref_bn = torch.nn.BatchNorm2d(c, momentum=0.9).to(DEV)
        own = BatchNorm2d(c, momentum=0.9).to(DEV)
        with torch.no_grad():
            ref_bn.weight.uniform_(0.5, 1.5)
            ref_bn.bias.uniform_(-1, 1)
        own.load_state_dict(ref_bn.state_dict())
        x = (torch.randn(n, c, h, w, device=DEV) * 0.5 + 30.0).to(dtype).contiguous(memory_format=torch.channels_last)
        g = torch.randn(n, c, h, w, device=DEV).to(dtype).contiguous(memory_format=torch.channels_last)
        res = []
        for bn in (ref_bn, own):
            xi = x.clone().requires_grad_(True)
            native.reset_launch_count()
            y = bn(xi, relu=relu) if bn is own else (torch.relu(bn(xi)) if relu else bn(xi))
            y.backward(g)
            launches = native.reset_launch_count()
            res.append((y.detach().float(), xi.grad.float(), bn.weight.grad.float(), bn.bias.grad.float(),
                        bn.running_mean.clone(), bn.running_var.clone()))
        assert launches >= 4, "the native kernels did not run"
        tol = dict(rtol=3e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=2e-3, atol=2e-3)
        for k, (a, b) in enumerate(zip(*res)):
            if relu and k in (1, 2, 3):
                # an activation within rounding of zero may fall on the other side of the ReLU
                assert (a - b).norm() <= (3e-2 if dtype == torch.bfloat16 else 1e-2) * b.norm() + 1e-3
            else:
                torch.testing.assert_close(a, b, **tol)
        assert int(own.num_batches_tracked) == 1
    # evaluation mode takes the library path
    own.eval()
    want = ref_bn.eval()(x)
    torch.testing.assert_close(own(x, relu=relu), torch.relu(want) if relu else want, rtol=1e-4, atol=1e-3)


def test_linear_and_layer_norm_layers_match_torch():
    """``models.layers.Linear`` (bias gradient on the column-sum kernel) and ``models.layers.LayerNorm`` (weight
    and bias gradients on the column kernel) against ``torch.nn`` under bf16 autocast and in fp32."""
    from conef_b200.models.layers import LayerNorm, Linear
    torch.manual_seed(5)
    for autocast in (True, False):
        ref_lin, own_lin = torch.nn.Linear(256, 512).to(DEV), Linear(256, 512).to(DEV)
        ref_ln, own_ln = torch.nn.LayerNorm(512, eps=1e-12).to(DEV), LayerNorm(512, eps=1e-12).to(DEV)
        with torch.no_grad():
            ref_ln.weight.uniform_(0.5, 1.5)
            ref_ln.bias.uniform_(-1, 1)
        own_lin.load_state_dict(ref_lin.state_dict())
        own_ln.load_state_dict(ref_ln.state_dict())
        x = torch.randn(6, 37, 256, device=DEV)
        g = torch.randn(6, 37, 512, device=DEV)
        res = []
        for lin, ln in ((ref_lin, ref_ln), (own_lin, own_ln)):
            xi = x.clone().requires_grad_(True)
            native.reset_launch_count()
            with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
                y = ln(lin(xi) * 3.0 + 20.0)
            y.backward(g.to(y.dtype))
            launches = native.reset_launch_count()
            res.append((y.detach().float(), xi.grad, lin.weight.grad, lin.bias.grad, ln.weight.grad, ln.bias.grad))
        assert launches >= 2, "the native kernels did not run"
        tol = dict(rtol=3e-2, atol=3e-2) if autocast else dict(rtol=2e-4, atol=2e-4)
        for a, b in zip(*res):
            assert a.dtype == b.dtype and a.shape == b.shape
            assert (a.float() - b.float()).norm() <= tol["rtol"] * b.float().norm() + tol["atol"]


@pytest.mark.parametrize("kw", [dict(momentum=0.9, nesterov=True, weight_decay=5e-4), dict(momentum=0.9, dampening=0.1),
                                dict(weight_decay=1e-2)])
def test_fused_sgd_kernel_matches_torch_sgd(kw):
    """One multi-tensor launch per step against torch.optim.SGD (ragged sizes, an unaligned view)."""
    from conef_b200.optim import FusedSGD
    torch.manual_seed(0)
    base = torch.randn(70001, device=DEV)
    shapes = [(640, 1441), (17,), (3, 5, 7), (65536 + 3,)]
    ref_p = [torch.nn.Parameter(torch.randn(s, device=DEV)) for s in shapes] + [torch.nn.Parameter(base[1:].clone())]
    own_p = [torch.nn.Parameter(p.detach().clone()) for p in ref_p]
    ref_opt, own_opt = torch.optim.SGD(ref_p, lr=0.1, **kw), FusedSGD(own_p, lr=0.1, **kw)
    for step in range(4):
        for a, b in zip(ref_p, own_p):
            g = torch.randn_like(a)
            a.grad, b.grad = g.clone(), g.clone()
        native.reset_launch_count()
        ref_opt.step()
        own_opt.step()
        assert native.reset_launch_count() == 1
    for a, b in zip(ref_p, own_p):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
def test_fused_sgd_takes_channels_last_and_mixed_groups():
    """Channels-last convolution weights go through the kernel (it walks the storage); a strided view in the
    same group runs as PyTorch ops beside it; zero_grad keeps the gradient tensors and clears them."""
    from conef_b200.optim import FusedSGD
    torch.manual_seed(1)
    kw = dict(lr=0.05, momentum=0.9, weight_decay=5e-4)
    w = torch.randn(64, 32, 3, 3, device=DEV).contiguous(memory_format=torch.channels_last)
    wide = torch.randn(40, 12, device=DEV)
    ref_p = [torch.nn.Parameter(w.clone(memory_format=torch.preserve_format)), torch.nn.Parameter(torch.randn(33, device=DEV)),
             torch.nn.Parameter(wide.clone())]
    own_p = [torch.nn.Parameter(p.detach().clone(memory_format=torch.preserve_format)) for p in ref_p]
    assert not own_p[0].is_contiguous() and own_p[0].stride() == ref_p[0].stride()
    ref_opt, own_opt = torch.optim.SGD(ref_p, **kw), FusedSGD(own_p, **kw)
    for step in range(3):
        for i, (a, b) in enumerate(zip(ref_p, own_p)):
            g = torch.randn_like(a)                      # keeps the parameter's strides
            a.grad = g.clone(memory_format=torch.preserve_format)
            b.grad = g.clone(memory_format=torch.preserve_format) if i < 2 else g.t().contiguous().t()   # transposed strides
        native.reset_launch_count()
        ref_opt.step()
        own_opt.step()
        assert native.reset_launch_count() == 1          # the two dense parameters; the third took the PyTorch path
    for a, b in zip(ref_p, own_p):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    # a momentum buffer that comes back from a checkpoint in another memory format is re-laid, not a reason to fall back
    own_opt.state[own_p[0]]["momentum_buffer"] = own_opt.state[own_p[0]]["momentum_buffer"].contiguous()
    assert own_opt.state[own_p[0]]["momentum_buffer"].stride() != own_p[0].stride()
    for i, (a, b) in enumerate(zip(ref_p, own_p)):
        g = torch.randn_like(a)
        a.grad = g.clone(memory_format=torch.preserve_format)
        b.grad = g.clone(memory_format=torch.preserve_format) if i < 2 else g.t().contiguous().t()
    native.reset_launch_count()
    ref_opt.step()
    own_opt.step()
    assert native.reset_launch_count() == 1
    assert own_opt.state[own_p[0]]["momentum_buffer"].stride() == own_p[0].stride()
    for a, b in zip(ref_p, own_p):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    ptrs = [p.grad.data_ptr() for p in own_p]
    own_opt.zero_grad(set_to_none=False)
    assert [p.grad.data_ptr() for p in own_p] == ptrs and all(float(p.grad.abs().max()) == 0 for p in own_p)
    own_opt.zero_grad()
    assert all(p.grad is None for p in own_p)

"""HSTU attention forward kernel (tcgen05) vs the fp32 PyTorch statement of the reference golden."""
import pytest
import torch

from recsdk_b200.ops import _lib
from recsdk_b200.ops import hstu_attention as HA

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _jagged(lens, H, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    T = sum(lens)
    mk = lambda: (torch.randn(T, H, D, generator=g, device=DEV) * 0.5).bfloat16()  # noqa: E731
    off = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=DEV)
    return mk(), mk(), mk(), off


def _close(a, b, tol=5e-3):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err <= tol * scale + tol, "max err %g vs scale %g" % (err, scale)


@pytest.mark.parametrize("lens,H,D", [([128], 1, 64), ([200, 37, 513, 1], 2, 64), ([300, 129], 2, 128), ([1000, 64, 700], 4, 64)])
@pytest.mark.parametrize("bias", [False, True])
def test_fwd_causal(lens, H, D, bias):
    q, k, v, off = _jagged(lens, H, D, 1)
    kw = {}
    if bias:
        g = torch.Generator().manual_seed(2)
        ts = torch.cat([torch.cumsum(torch.randint(1, 5000, (n,), generator=g), 0) for n in lens]).float().to(DEV)
        kw = dict(ts=ts, ts_w=(torch.randn(65, generator=g) * 0.5).to(DEV), ts_divisor=0.301,
                  pos_w=(torch.randn(512, generator=g) * 0.5).to(DEV))
    alpha, scale = 1.0 / D ** 0.5, 1.0 / max(lens)
    out = HA.hstu_attn_fwd(q, k, v, off, off, max(lens), alpha, scale, True, **kw)
    ref = HA.hstu_attention_ref(q, k, v, off, off, alpha, scale, True, **kw)
    torch.cuda.synchronize()
    _lib.check_status()
    _close(out, ref)


def test_fwd_context_targets_noncausal_and_delta():
    lens = [400, 260, 129]
    q, k, v, off = _jagged(lens, 2, 64, 3)
    alpha, scale = 0.125, 1.0 / 400
    nc = torch.tensor([10, 0, 3], device=DEV)
    nt = torch.tensor([100, 130, 5], device=DEV)
    for gs in (1, 7):
        out = HA.hstu_attn_fwd(q, k, v, off, off, 400, alpha, scale, True, nc, nt, gs)
        ref = HA.hstu_attention_ref(q, k, v, off, off, alpha, scale, True, nc, nt, gs)
        _close(out, ref)
    out = HA.hstu_attn_fwd(q, k, v, off, off, 400, alpha, scale, False)
    _close(out, HA.hstu_attention_ref(q, k, v, off, off, alpha, scale, False))
    # delta: queries are the last rows of every sequence
    qlens = [50, 260, 1]
    qoff = torch.tensor([0, 50, 310, 311], device=DEV)
    qs = torch.cat([q[off[b + 1] - qlens[b]:off[b + 1]] for b in range(3)])
    out = HA.hstu_attn_fwd(qs, k, v, qoff, off, 260, alpha, scale, True)
    ref_full = HA.hstu_attention_ref(q, k, v, off, off, alpha, scale, True)
    ref = torch.cat([ref_full[off[b + 1] - qlens[b]:off[b + 1]] for b in range(3)])
    _close(out, ref)
    torch.cuda.synchronize()
    _lib.check_status()


def test_fwd_paged_matches_jagged():
    H, D, page = 2, 64, 64
    lens = [300, 64, 130]
    qlens = [172, 64, 2]
    q, k, v, off = _jagged(lens, H, D, 5)
    n_pages = sum((n + page - 1) // page for n in lens) + 3
    cache = torch.zeros(n_pages, 2, page, H, D, dtype=torch.bfloat16, device=DEV)
    perm = torch.randperm(n_pages).tolist()
    page_ids, indptr, cur = [], [0], 0
    for b, n in enumerate(lens):
        for pg in range((n + page - 1) // page):
            pid = perm[cur]; cur += 1
            page_ids.append(pid)
            lo, hi = pg * page, min(n, (pg + 1) * page)
            cache[pid, 0, : hi - lo] = k[off[b] + lo: off[b] + hi]
            cache[pid, 1, : hi - lo] = v[off[b] + lo: off[b] + hi]
        indptr.append(len(page_ids))
    qoff = torch.tensor([0, 172, 236, 238], device=DEV)
    qs = torch.cat([q[off[b + 1] - qlens[b]:off[b + 1]] for b in range(3)])
    nt = torch.tensor([100, 0, 1], device=DEV)
    out = HA.hstu_attention_paged(qs, cache, qoff, off, torch.tensor(page_ids, device=DEV), torch.tensor(indptr, device=DEV),
                                  page, 172, 0.125, 1 / 300, nt, 1)
    ref_full = HA.hstu_attention_ref(q, k, v, off, off, 0.125, 1 / 300, True, None, nt, 1)
    ref = torch.cat([ref_full[off[b + 1] - qlens[b]:off[b + 1]] for b in range(3)])
    torch.cuda.synchronize()
    _lib.check_status()
    _close(out, ref)


@pytest.mark.parametrize("lens,H", [([128], 1), ([200, 37, 513, 1], 2), ([700, 300], 4)])
@pytest.mark.parametrize("bias", [False, True])
def test_bwd_matches_reference(lens, H, bias):
    from recsdk_b200.ops.hstu_attention_bwd import hstu_attn_bwd, hstu_attn_bwd_ref

    q, k, v, off = _jagged(lens, H, 64, 11)
    dout = (torch.randn_like(q.float()) * 0.5).bfloat16()
    kw = dict(ts=None, ts_w=None, ts_divisor=0.301, pos_w=None)
    if bias:
        g = torch.Generator().manual_seed(2)
        ts = torch.cat([torch.cumsum(torch.randint(1, 5000, (n,), generator=g), 0) for n in lens]).float().to(DEV)
        kw = dict(ts=ts, ts_w=(torch.randn(65, generator=g) * 0.5).to(DEV), ts_divisor=0.301,
                  pos_w=(torch.randn(512, generator=g) * 0.5).to(DEV))
    alpha, scale = 0.125, 1.0 / max(lens)
    got = hstu_attn_bwd(dout, q, k, v, off, off, alpha, scale, True, None, None, 0, **kw)
    ref = hstu_attn_bwd_ref(dout, q, k, v, off, off, alpha, scale, True, None, None, 0, **kw)
    torch.cuda.synchronize()
    _lib.check_status()
    for name, a, b in zip(("dq", "dk", "dv", "dts_w", "dpos_w"), got, ref):
        if b is None:
            continue
        _close(a, b, tol=2e-2)


def test_bwd_targets_and_autograd():
    lens = [400, 260]
    q, k, v, off = _jagged(lens, 2, 64, 13)
    nc = torch.tensor([10, 0], device=DEV)
    nt = torch.tensor([100, 130], device=DEV)
    from recsdk_b200.ops.hstu_attention_bwd import hstu_attn_bwd, hstu_attn_bwd_ref

    dout = (torch.randn_like(q.float()) * 0.5).bfloat16()
    got = hstu_attn_bwd(dout, q, k, v, off, off, 0.125, 1 / 400, True, nc, nt, 3, None, None, 0.301, None)
    ref = hstu_attn_bwd_ref(dout, q, k, v, off, off, 0.125, 1 / 400, True, nc, nt, 3, None, None, 0.301, None)
    for a, b in zip(got[:3], ref[:3]):
        _close(a, b, tol=2e-2)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    pw = (torch.randn(256, device=DEV) * 0.1).requires_grad_()
    out = HA.hstu_attention(q, k, v, off, alpha=0.125, pos_w=pw)
    out.float().square().sum().backward()
    assert q.grad is not None and k.grad.abs().sum() > 0 and pw.grad.abs().sum() > 0
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("D,S,heads_in_bias,mask_type", [(64, 200, True, 0), (128, 256, False, 0), (64, 333, True, 3), (64, 128, False, 2)])
def test_dense_attn_bias_and_custom_mask_on_the_kernel(D, S, heads_in_bias, mask_type):
    """The reference's main calling convention - relative bias passed as a dense ``attn_bias`` [B,N,S,S], optionally a custom
    0/1 mask (mask_type 3) - runs on the tcgen05 forward kernel; per-row relative error against the fp32 statement, and
    gradients (q, k, v, attn_bias) through the op."""
    import torch

    from recsdk_b200.ops import mxrec  # noqa: F401  (registers torch.ops.mxrec)
    from recsdk_b200.ops.mxrec import _dense_ref

    dev = torch.device("cuda", 0)
    B, N = 2, 4
    g = torch.Generator().manual_seed(S + D)
    q, k, v = (torch.randn(B, S, N, D, generator=g).mul_(0.5).to(dev, torch.bfloat16).requires_grad_() for _ in range(3))
    bias = (torch.randn(B, N if heads_in_bias else 1, S, S, generator=g) * 0.5).to(dev, torch.bfloat16).requires_grad_()
    mask = None
    if mask_type == 3:
        mask = (torch.rand(B, 1, S, S, generator=g) < 0.6).to(dev)
    out = torch.ops.mxrec.hstu_dense(q, k, v, mask, bias, mask_type, S, 1.0 / S)
    ref_in = [t.detach().float().requires_grad_() for t in (q, k, v, bias)]
    want = _dense_ref(ref_in[0], ref_in[1], ref_in[2], mask, ref_in[3], mask_type, 1.0 / S)
    err = (out.float() - want).abs().amax(dim=(-1,))                       # per (batch, row, head)
    scale = want.abs().amax(dim=(-1,)).clamp_min(1e-3)
    assert float((err / scale).max()) < 3e-2, float((err / scale).max())
    w = torch.randn(out.shape, generator=g).to(dev)
    (out.float() * w).sum().backward()
    (want * w).sum().backward()
    for got, ref in zip((q, k, v, bias), ref_in):
        rel = (got.grad.float() - ref.grad).abs().max() / ref.grad.abs().max().clamp_min(1e-6)
        assert float(rel) < 3e-2, float(rel)


def test_jagged_attn_bias_on_the_kernel():
    import torch

    from recsdk_b200.ops import mxrec  # noqa: F401
    from recsdk_b200.ops.mxrec import _jagged_ref_bias

    dev = torch.device("cuda", 0)
    lens, N, D, Smax = [70, 300, 129], 2, 64, 320
    offs = torch.tensor([0, 70, 370, 499], dtype=torch.int32, device=dev)
    T = int(offs[-1])
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(T, N, D, generator=g).mul_(0.5).to(dev, torch.bfloat16) for _ in range(3))
    bias = (torch.randn(len(lens), N, Smax, Smax, generator=g) * 0.5).to(dev, torch.bfloat16)
    out = torch.ops.mxrec.hstu_jagged.equal(q, k, v, None, bias, 0, Smax, 1.0 / Smax, offs, None, None, 0, 1.0, False)
    want = _jagged_ref_bias(q, k, v, None, bias, 0, 1.0 / Smax, offs, offs, None, None, 0, 1.0)
    err = (out.float() - want.float()).abs().amax(dim=-1)
    scale = want.float().abs().amax(dim=-1).clamp_min(1e-3)
    assert float((err / scale).max()) < 3e-2


@pytest.mark.parametrize("mask_type,layout", [(0, "jagged"), (3, "jagged"), (2, "normal"), (0, "normal")])
def test_fuxi_variant_on_the_kernels(mask_type, layout):
    """``hstu_fuxi`` (SiLU attention + two bias-times-V parts) through the tcgen05 attention and GEMM kernels against the
    fp32 statement, forward and gradients."""
    import torch

    from recsdk_b200.ops import mxrec  # noqa: F401
    from recsdk_b200.ops.mxrec import _fuxi_ref

    dev = torch.device("cuda", 0)
    N, D, S = 2, 64, 160
    g = torch.Generator().manual_seed(3 + mask_type)
    if layout == "jagged":
        offs = [0, 70, 229, 330]                                   # lengths 70, 159, 101 (not multiples of 8)
        T, nb = offs[-1], 3
        shape = (T, N, D)
    else:
        offs, nb = None, 2
        shape = (nb, S, N, D)
    q, k, v = ((torch.randn(*shape, generator=g) * 0.5).to(dev, torch.bfloat16).requires_grad_() for _ in range(3))
    tsb = (torch.randn(nb, S, S, generator=g) * 0.3).to(dev, torch.bfloat16).requires_grad_()
    pob = (torch.randn(1, S, S, generator=g) * 0.3).to(dev, torch.bfloat16).requires_grad_()
    mask = (torch.rand(nb, N, S, S, generator=g) < 0.5).to(dev, torch.bfloat16) if mask_type == 3 else None
    out = torch.ops.mxrec.hstu_fuxi(q, k, v, tsb, pob, mask, mask_type, S, 0.0, layout, offs)
    refs = [t.detach().float().requires_grad_() for t in (q, k, v, tsb, pob)]
    want = _fuxi_ref(*refs, mask, mask_type, 1.0 / S, layout, offs)
    assert out.shape == want.shape and out.shape[-1] == 3 * D
    err = (out.float() - want).abs().amax(dim=-1)
    scale = want.abs().amax(dim=-1).clamp_min(1e-2)
    assert float((err / scale).max()) < 4e-2, float((err / scale).max())
    w = torch.randn(out.shape, generator=g).to(dev)
    (out.float() * w).sum().backward()
    (want * w).sum().backward()
    for got, ref in zip((q, k, v, tsb, pob), refs):
        rel = (got.grad.float() - ref.grad).abs().max() / ref.grad.abs().max().clamp_min(1e-6)
        assert float(rel) < 3e-2, float(rel)

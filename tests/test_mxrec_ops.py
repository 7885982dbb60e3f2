"""``torch.ops.mxrec.*`` registrations: names resolve, argument orders work, results match direct math (CPU)."""
import torch

import recsdk_b200.ops.mxrec  # noqa: F401  (registers the operators)
from recsdk_b200.ops.hstu_attention import hstu_attention_ref


def test_hstu_dense_and_backward():
    torch.manual_seed(0)
    B, S, N, D = 2, 12, 2, 16
    q, k, v = (torch.randn(B, S, N, D) * 0.5 for _ in range(3))
    out = torch.ops.mxrec.hstu_dense(q, k, v, None, None, 0, S, 0.0)
    offs = torch.arange(0, (B + 1) * S, S)
    ref = hstu_attention_ref(q.reshape(B * S, N, D), k.reshape(B * S, N, D), v.reshape(B * S, N, D), offs, offs, 1.0, 1.0 / S)
    assert torch.allclose(out.reshape(B * S, N, D), ref, atol=1e-5)
    bias = torch.randn(B, N, S, S) * 0.1
    g = torch.randn_like(out)
    dq, dk, dv, db = torch.ops.mxrec.hstu_dense_backward(g, q, k, v, None, bias, 0, S, 0.0)
    qq, bb = q.clone().requires_grad_(True), bias.clone().requires_grad_(True)
    o2 = torch.ops.mxrec.hstu_dense(qq, k, v, None, bb, 0, S, 0.0)
    o2.backward(g)
    assert torch.allclose(dq, qq.grad, atol=1e-5) and torch.allclose(db, bb.grad, atol=1e-5)


def test_hstu_jagged_overloads_and_paged():
    torch.manual_seed(1)
    N, D = 2, 16
    qo = torch.tensor([0, 5, 9])
    ko = torch.tensor([0, 8, 15])
    q = torch.randn(9, N, D) * 0.5
    k, v = torch.randn(15, N, D) * 0.5, torch.randn(15, N, D) * 0.5
    nt = torch.tensor([2, 1])
    out = torch.ops.mxrec.hstu_jagged.delta(q, k, v, None, None, 0, 5, 8, 0.1, qo, ko, None, nt, 1, 0.5, False)
    ref = hstu_attention_ref(q, k, v, qo, ko, 0.5, 0.1, True, None, nt, 1)
    assert torch.allclose(out, ref, atol=1e-5)
    eq = torch.ops.mxrec.hstu_jagged.equal(k, k, v, None, None, 0, 8, 0.1, ko, None, None, 0, 1.0, False)
    assert torch.allclose(eq, hstu_attention_ref(k, k, v, ko, ko, 1.0, 0.1), atol=1e-5)
    g = torch.randn_like(out)
    dq, dk, dv, _ = torch.ops.mxrec.hstu_jagged_backward.delta(g, q, k, v, None, None, 0, 5, 8, 0.1, qo, ko, None, nt, 1, 0.5, False)
    qq = q.clone().requires_grad_(True)
    hstu_attention_ref(qq, k, v, qo, ko, 0.5, 0.1, True, None, nt, 1).backward(g)
    assert torch.allclose(dq, qq.grad, atol=1e-4)
    # paged: history in the cache, the op appends the new tokens and attends
    page = 4
    cache = torch.zeros(8, 2, page, N, D)
    page_ids = torch.tensor([0, 1, 5, 6])
    page_off = torch.tensor([0, 2, 4])
    hist = [3, 3]
    for b in range(2):
        for t in range(hist[b]):
            pg = page_ids[page_off[b] + t // page]
            cache[pg, 0, t % page] = k[ko[b] + t]
            cache[pg, 1, t % page] = v[ko[b] + t]
    ko2 = torch.tensor([0, 8, 7 + 8]) if False else torch.tensor([0, 8, 8 + 7])
    newk = torch.cat([k[3:8], k[11:15]])
    newv = torch.cat([v[3:8], v[11:15]])
    qn = torch.randn(9, N, D)
    out = torch.ops.mxrec.hstu_paged(qn, newk, newv, cache, None, None, 0, 5, 8, 0.1, qo, ko2, None, page_off, page_ids, None, None, 0,
                                     1.0, False)
    ref = hstu_attention_ref(qn, k, v, qo, ko2, 1.0, 0.1)
    assert torch.allclose(out, ref, atol=1e-5)


def test_in_linear_silu_and_small_ops():
    torch.manual_seed(2)
    x, w, b = torch.randn(7, 12), torch.randn(20, 12), torch.randn(20)
    outs = torch.ops.mxrec.in_linear_silu(x, w, b, [4, 6, 5, 5])
    z = x @ w.t() + b
    assert [o.shape[1] for o in outs] == [4, 6, 5, 5] and torch.allclose(torch.cat(outs, 1), torch.nn.functional.silu(z), atol=1e-5)
    gs = [torch.randn_like(o) for o in outs]
    dx, dw, db = torch.ops.mxrec.in_linear_silu_backward(x, w, b, gs[0], gs[1], gs[2], gs[3], z, [4, 6, 5, 5])
    xx, ww, bb = (t.clone().requires_grad_(True) for t in (x, w, b))
    torch.nn.functional.silu(xx @ ww.t() + bb).backward(torch.cat(gs, 1))
    assert torch.allclose(dx, xx.grad, atol=1e-4) and torch.allclose(dw, ww.grad, atol=1e-4) and torch.allclose(db, bb.grad, atol=1e-4)
    ts = torch.sort(torch.randint(0, 10000, (2, 6))).values
    tw = torch.randn(3, 9)
    rab, idx = torch.ops.mxrec.relative_attn_bias_time_with_index(ts, tw, 0.5)
    assert rab.shape == (3, 2, 6, 6) and torch.equal(torch.ops.mxrec.relative_attn_bias_time(ts, tw, 0.5), rab)
    dwt = torch.ops.mxrec.relative_attn_bias_time_backward(torch.ones_like(rab), idx, 8)
    assert dwt.shape == (3, 9) and float(dwt.sum()) == 3 * 2 * 36
    y = torch.ops.mxrec.ln_mul(x, torch.ones_like(x), torch.ones(12), torch.zeros(12))
    assert torch.allclose(y, torch.nn.functional.layer_norm(x, (12,)), atol=1e-5)
    assert torch.equal(torch.ops.mxrec.gather_for_rank1(b, torch.tensor([3, 1])), b[[3, 1]])
    two = torch.ops.mxrec.multislice_concat(x, 2, [2, 1], [0, 5, 3], [2, 3, 4])
    assert len(two) == 2 and torch.equal(two[0], torch.cat([x[:, :2], x[:, 5:8]], 1)) and torch.equal(two[1], x[:, 3:7])
    r = torch.ops.mxrec.reverse_sequence(torch.arange(12.).view(2, 6, 1), torch.tensor([3, 6]))
    assert r[0, :3, 0].tolist() == [2, 1, 0] and r[1, :, 0].tolist() == [11, 10, 9, 8, 7, 6]
    # TBE-compatible lookup over one flat buffer
    wflat = torch.randn(5 * 4 + 3 * 8)
    out = torch.ops.mxrec.split_embedding_codegen_forward_unweighted_cuda(
        wflat, wflat[:0], wflat[:0], torch.zeros(2, dtype=torch.int32), torch.tensor([0, 20]), torch.tensor([0, 4, 12]), 12, 8,
        torch.tensor([0, 4, 1, 2, 2]), torch.tensor([0, 2, 3, 4, 5]), 0, torch.zeros(0, dtype=torch.int32), torch.zeros(0), 0, False,
        None, None, torch.tensor([5, 3]))
    t0, t1 = wflat[:20].view(5, 4), wflat[20:].view(3, 8)
    assert torch.allclose(out[0, :4], t0[0] + t0[4]) and torch.allclose(out[1, 4:], t1[2])


def test_fuxi_and_disentangle():
    torch.manual_seed(3)
    B, S, N, D = 2, 6, 2, 8
    q, k, v = (torch.randn(B, S, N, D) for _ in range(3))
    tb, pb = torch.randn(B, S, S), torch.randn(1, S, S)
    out = torch.ops.mxrec.hstu_fuxi(q, k, v, tb, pb, None, 0, S, 0.0, "normal", None)
    assert out.shape == (B, S, N, 3 * D)
    assert torch.allclose(out[..., :D], torch.ops.mxrec.hstu_dense(q, k, v, None, None, 0, S, 0.0), atol=1e-5)
    m = torch.tril(torch.ones(S, S))
    assert torch.allclose(out[0, :, 1, D:2 * D], (tb[0] * m) @ v[0, :, 1], atol=1e-5)
    jag = torch.ops.mxrec.hstu_fuxi(q.reshape(B * S, N, D), k.reshape(B * S, N, D), v.reshape(B * S, N, D), None, None, None, 0, S, 0.0,
                                    "jagged", [0, S, 2 * S])
    assert torch.allclose(jag.view(B, S, N, D), out[..., :D], atol=1e-5)
    # disentangled attention: with zero position projections it is plain masked softmax attention
    qq, kk, vv = (torch.randn(B, N, S, D) for _ in range(3))
    rel = (torch.arange(S)[:, None] - torch.arange(S)[None, :]).view(1, 1, S, S)
    mask = torch.ones(B, 1, S, S)
    z = torch.zeros(2 * S, N, D)
    o, p, w = torch.ops.mxrec.disentangle_attention(qq, kk, vv, z, z, rel, mask, "c2p|p2c", 0.25)
    ref = torch.softmax(qq @ kk.transpose(-1, -2) * 0.25, -1) @ vv
    assert torch.allclose(o, ref, atol=1e-5) and torch.allclose(p.sum(-1), torch.ones(B, N, S), atol=1e-5)
    pk = torch.randn(2 * S, N, D)
    _, _, w2 = torch.ops.mxrec.disentangle_attention(qq, kk, vv, pk, z, rel, mask, "c2p", 0.25)
    i, j = 4, 1
    exp = (qq[0, 0, i] @ kk[0, 0, j] + qq[0, 0, i] @ pk[i - j + S, 0]) * 0.25
    assert torch.allclose(w2[0, 0, i, j], exp, atol=1e-5)


def test_hstu_ops_accept_the_reference_operator_range():
    """fp32 / fp16 / bf16 inputs, D_qk != D_v, jagged and dense, with gradients (served by the fp32 statement wherever the
    tcgen05 kernels do not apply)."""
    import pytest

    g = torch.Generator().manual_seed(0)
    offs = torch.tensor([0, 5, 12])
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        q = torch.randn(12, 2, 24, generator=g).to(dt).requires_grad_()
        k = torch.randn(12, 2, 24, generator=g).to(dt).requires_grad_()
        v = torch.randn(12, 2, 16, generator=g).to(dt).requires_grad_()
        o = torch.ops.mxrec.hstu_jagged.equal(q, k, v, None, None, 0, 7, 0.0, offs, None, None, 0, 1.0, False)
        assert o.shape == (12, 2, 16) and o.dtype == dt
        o.float().sum().backward()
        assert all(t.grad is not None and torch.isfinite(t.grad.float()).all() for t in (q, k, v))
        od = torch.ops.mxrec.hstu_dense(q[:10].view(2, 5, 2, 24), k[:10].view(2, 5, 2, 24), v[:10].view(2, 5, 2, 16), None, None, 0, 5, 0.0)
        assert od.shape == (2, 5, 2, 16)
        # causal: the first token of every sequence only sees itself
        q0 = q.detach().float()[0]
        want0 = torch.nn.functional.silu((q0 * k.detach().float()[0]).sum(-1)) / 7.0
        assert torch.allclose(o.detach().float()[0], want0[:, None] * v.detach().float()[0], atol=2e-2, rtol=2e-2)
    with pytest.raises(NotImplementedError):
        torch.ops.mxrec.hstu_dense(q[:10].view(2, 5, 2, 24), k[:10].view(2, 5, 2, 24), v[:10].view(2, 5, 2, 16), None, None, 1, 5, 0.0)


def test_fuxi_backward_operator_matches_autograd():
    """``hstu_dense_backward_fuxi`` (jagged layout): gradients of q, k, v and of both biases equal autograd through
    ``hstu_fuxi``; the position bias shared by the batch gets one summed gradient; without biases the last two are empty."""
    torch.manual_seed(0)
    offs, N, D = [0, 5, 9], 2, 8
    q, k, v = (torch.randn(9, N, D, requires_grad=True) for _ in range(3))
    tb, pb = torch.randn(2, 6, 6, requires_grad=True), torch.randn(1, 6, 6, requires_grad=True)
    out = torch.ops.mxrec.hstu_fuxi(q, k, v, tb, pb, None, 0, 6, 0.0, "jagged", offs)
    assert out.shape == (9, N, 3 * D)
    g = torch.randn_like(out)
    want = torch.autograd.grad(out, [q, k, v, pb, tb], g)
    got = torch.ops.mxrec.hstu_dense_backward_fuxi(g, q.detach(), k.detach(), v.detach(), None, pb.detach(), tb.detach(), "jagged", 0, 6,
                                                   0.0, offs)
    for a, b in zip(got, want):
        assert a.shape == b.shape
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    mask = (torch.rand(2, 1, 6, 6) > 0.3).float()
    out = torch.ops.mxrec.hstu_fuxi(q, k, v, None, None, mask, 3, 6, 0.25, "jagged", offs)
    want = torch.autograd.grad(out, [q, k, v], torch.ones_like(out))
    got = torch.ops.mxrec.hstu_dense_backward_fuxi(torch.ones_like(out), q.detach(), k.detach(), v.detach(), mask, None, None, "jagged", 3, 6,
                                                   0.25, offs)
    assert got[3].numel() == 0 and got[4].numel() == 0
    for a, b in zip(got[:3], want):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    import pytest

    with pytest.raises(ValueError):
        torch.ops.mxrec.hstu_dense_backward_fuxi(g, q.detach(), k.detach(), v.detach(), layout="normal", seqOffset=offs)
    with pytest.raises(ValueError):
        torch.ops.mxrec.hstu_dense_backward_fuxi(g[:, :, :D], q.detach(), k.detach(), v.detach(), None, pb.detach(), tb.detach(), "jagged", 0,
                                                 6, 0.0, offs)


def test_jagged_concat_and_split_with_a_prefix_from_the_right():
    """``concat_2d_jagged`` / ``split_2d_jagged`` in the reference's signature: per sample ``[B[:n] | A | B[n:]]`` and back."""
    import pytest

    a = torch.arange(1, 4).float()[:, None].repeat(1, 4)                  # rows 1, 2, 3
    b = torch.arange(4, 8).float()[:, None].repeat(1, 4)                  # rows 4 .. 7
    oa, ob = torch.tensor([0, 1, 2, 3]), torch.tensor([0, 1, 3, 4])
    cat = torch.ops.mxrec.concat_2d_jagged(2, a, b, oa, ob)
    assert cat[:, 0].tolist() == [1, 4, 2, 5, 6, 3, 7]
    sa, sb = torch.ops.mxrec.split_2d_jagged(cat, 2, oa, ob)
    assert torch.equal(sa, a) and torch.equal(sb, b)

    def golden(n):
        rows = []
        for i in range(3):
            bs = list(range(int(ob[i]), int(ob[i + 1])))
            p = min(n, len(bs))
            rows += [b[j] for j in bs[:p]] + [a[j] for j in range(int(oa[i]), int(oa[i + 1]))] + [b[j] for j in bs[p:]]
        return torch.stack(rows)

    for n in (1, 2, 5):
        got = torch.ops.mxrec.concat_2d_jagged(2, a, b, oa, ob, False, n)
        assert torch.equal(got, golden(n))
        ra, rb = torch.ops.mxrec.split_2d_jagged(got, 2, oa, ob, 0, n)
        assert torch.equal(ra, a) and torch.equal(rb, b)
    assert torch.ops.mxrec.concat_2d_jagged(2, a, b, oa, ob, False, 1)[:, 0].tolist() == [4, 1, 5, 2, 6, 7, 3]
    empty_b = torch.ops.mxrec.concat_2d_jagged(1, a, b[:0], oa, torch.zeros(4, dtype=torch.long), False, 3)
    assert torch.equal(empty_b, a)
    ag = a.clone().requires_grad_(True)
    torch.ops.mxrec.concat_2d_jagged(2, ag, b, oa, ob, False, 1).sum().backward()
    assert torch.equal(ag.grad, torch.ones_like(a))
    with pytest.raises(ValueError):
        torch.ops.mxrec.concat_2d_jagged(2, a, b, oa, ob, False, -1)
    x = torch.arange(24.).view(2, 12)
    with pytest.raises(ValueError):
        torch.ops.mxrec.multislice_concat(x, 1, [1], [10], [4])
    with pytest.raises(ValueError):
        torch.ops.mxrec.multislice_concat(x, 2, [1], [0], [4])

"""HSTU helper kernels (relative bias, jagged data movement, fused norm-gate) against the CPU path of the same wrappers."""
import pytest
import torch

from recsdk_b200.ops import hstu_ops as H

pytestmark = pytest.mark.gpu


def _cmp(fn, *args, tol=1e-5, **kw):
    cpu = fn(*args, **kw)
    gpu = fn(*[a.cuda() if isinstance(a, torch.Tensor) else a for a in args], **kw)
    cpu, gpu = (cpu if isinstance(cpu, (tuple, list)) else [cpu]), (gpu if isinstance(gpu, (tuple, list)) else [gpu])
    for c, g in zip(cpu, gpu):
        assert c.shape == g.shape
        assert torch.allclose(c.float(), g.float().cpu(), atol=tol, rtol=tol), (c.float() - g.float().cpu()).abs().max()


def test_relative_bias_kernels():
    g = torch.Generator().manual_seed(0)
    ts = torch.sort(torch.randint(0, 10 ** 6, (3, 70), generator=g)).values.float()
    w = torch.randn(2, 33, generator=g)
    _cmp(H.relative_attn_bias_time, ts, w, 0.301)
    rab, idx = H.relative_attn_bias_time(ts.cuda(), w.cuda(), 0.301, with_index=True)
    _, ridx = H.relative_attn_bias_time(ts, w, 0.301, with_index=True)
    assert (idx.cpu() != ridx).float().mean() < 1e-3                 # bucket edges may round differently
    grad = torch.randn(2, 3, 70, 70, generator=g)
    _cmp(H.relative_attn_bias_time_backward, grad, ridx, 32, tol=1e-3)
    bias = torch.randn(64, 64, generator=g)
    ident = torch.eye(48)
    _cmp(H.relative_attn_bias_pos, bias, ident, [10, 48, 30])


def test_jagged_movement_kernels():
    g = torch.Generator().manual_seed(1)
    lens_a, lens_b = torch.tensor([3, 0, 7, 5]), torch.tensor([2, 4, 0, 1])
    oa = torch.cat([torch.zeros(1, dtype=torch.long), lens_a.cumsum(0)])
    ob = torch.cat([torch.zeros(1, dtype=torch.long), lens_b.cumsum(0)])
    va, vb = torch.randn(15, 24, generator=g), torch.randn(7, 24, generator=g)
    _cmp(H.jagged_to_padded, va, oa, 8)
    padded = H.jagged_to_padded(va, oa, 8)
    _cmp(H.padded_to_jagged, padded, oa, 15)
    _cmp(H.concat_2d_jagged, va, vb, oa, ob)
    cat, oc = H.concat_2d_jagged(va, vb, oa, ob)
    _cmp(H.split_2d_jagged, cat, oa, ob)
    x = torch.randn(4, 9, 16, generator=g)
    _cmp(H.reverse_sequence, x, torch.tensor([9, 1, 4, 0]))
    v = torch.randn(100, generator=g)
    _cmp(H.gather_for_rank1, v, torch.randint(0, 100, (37,), generator=g))
    _cmp(H.multislice_concat, torch.randn(5, 40, generator=g), [0, 10, 32], [4, 8, 8])


def test_ln_mul_and_token_mixing():
    g = torch.Generator().manual_seed(2)
    x, u = torch.randn(50, 512, generator=g), torch.randn(50, 512, generator=g)
    ga, be = torch.randn(512, generator=g), torch.randn(512, generator=g)
    _cmp(H.ln_mul, x, u, ga, be, tol=1e-4)
    _cmp(H.ln_mul, x, None, ga, be, tol=1e-4)
    xg = x.cuda().requires_grad_(True)
    xc = x.clone().requires_grad_(True)
    H.ln_mul(xg, u.cuda(), ga.cuda(), be.cuda()).square().sum().backward()
    H.ln_mul(xc, u, ga, be).square().sum().backward()
    assert torch.allclose(xg.grad.cpu(), xc.grad, atol=2e-3, rtol=2e-3)
    t = torch.randn(3, 32, 32, generator=g)
    _cmp(H.token_mixing, t, torch.ones(32), torch.zeros(32), tol=1e-4)


@pytest.mark.parametrize("C", [256, 512, 384])
@pytest.mark.parametrize("with_u", [True, False])
def test_ln_mul_backward_bf16_all_gradients(C, with_u):
    """bf16 rows of width 256 / 512 take the register-resident vector kernel, 384 the generic one; both against fp32 PyTorch."""
    g = torch.Generator().manual_seed(C + int(with_u))
    rows = 1000
    x = torch.randn(rows, C, generator=g).bfloat16()
    u = torch.randn(rows, C, generator=g).bfloat16() if with_u else None
    ga, be = torch.randn(C, generator=g), torch.randn(C, generator=g)
    dy = torch.randn(rows, C, generator=g).bfloat16()
    leaves_g = [t.cuda().requires_grad_(True) if t is not None else None for t in (x, u, ga, be)]
    leaves_c = [t.float().requires_grad_(True) if t is not None else None for t in (x, u, ga, be)]
    H.ln_mul(*leaves_g).backward(dy.cuda())
    xn = torch.nn.functional.layer_norm(leaves_c[0], (C,), leaves_c[2], leaves_c[3], 1e-5)
    (xn * leaves_c[1] if with_u else xn).backward(dy.float())
    for a, b, tol in zip(leaves_g, leaves_c, (0.05, 0.05, 0.02, 0.02)):
        if a is None:
            continue
        ref = b.grad
        err = (a.grad.float().cpu() - ref).abs().max().item()
        assert err <= tol * max(1.0, ref.abs().max().item()), (err, ref.abs().max().item())

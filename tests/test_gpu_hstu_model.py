"""HSTU model: one layer against a plain PyTorch statement of the same layer, and a short training run."""
import math

import pytest
import torch

from recsdk_b200.models.hstu import HSTUConfig, HSTULayer
from recsdk_b200.models.hstu_bench import build, make_batch
from recsdk_b200.ops import _lib
from recsdk_b200.ops.hstu_attention import hstu_attention_ref
from recsdk_b200.parallel.comm import ShardingEnv

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def test_layer_matches_torch_reference():
    cfg = HSTUConfig(num_layers=1, d_model=256, num_heads=4, head_dim=64, max_seq_len=512, num_time_buckets=64)
    torch.manual_seed(0)
    layer = HSTULayer(cfg, DEV)
    lens = [300, 77, 129]
    off = torch.tensor([0, 300, 377, 506], device=DEV)
    x = (torch.randn(506, 256, device=DEV) * 0.5).bfloat16().requires_grad_()
    ts = torch.cat([torch.cumsum(torch.rand(n) * 3600, 0) for n in lens]).to(DEV)
    y = layer(x, off, 300, ts)
    y.float().square().mean().backward()
    # reference in fp32 torch
    hd = 256
    xr = x.detach().float().requires_grad_()
    xn = torch.nn.functional.layer_norm(xr, (256,), layer.norm_in_w, layer.norm_in_b)
    uvqk = torch.nn.functional.silu(xn.bfloat16().float() @ layer.uvqk.weight(0).bfloat16().float().t() + layer.uvqk.bias(0))
    uvqk = uvqk.bfloat16().float()
    u, v, q, k = uvqk[:, :hd], uvqk[:, hd:2 * hd], uvqk[:, 2 * hd:3 * hd], uvqk[:, 3 * hd:]
    a = hstu_attention_ref(q.view(-1, 4, 64), k.view(-1, 4, 64), v.view(-1, 4, 64), off, off, 1 / 8.0, 1 / 300, True,
                           ts=ts, ts_w=layer.ts_w, ts_divisor=cfg.time_bucket_divisor, pos_w=layer.pos_w)
    yn = torch.nn.functional.layer_norm(a.reshape(-1, hd).float(), (hd,), layer.norm_attn_w, layer.norm_attn_b) * u
    ref = xr + (yn.bfloat16().float() @ layer.out.weight(0).bfloat16().float().t() + layer.out.bias(0))
    torch.cuda.synchronize()
    _lib.check_status()
    err = (y.float() - ref).abs().max().item()
    assert err < 0.06 * ref.abs().max().item(), err
    assert x.grad is not None and torch.isfinite(x.grad.float()).all()
    assert layer.ts_w.grad.abs().sum() > 0 and layer.pos_w.grad.abs().sum() > 0 and layer.uvqk.flat_grad.abs().sum() > 0


def test_hstu_trains():
    from recsdk_b200.models.hstu import HSTUConfig

    cfg = HSTUConfig(num_layers=2, d_model=256, num_heads=4, head_dim=64, max_seq_len=512, num_negatives=64)
    model, opt = build(DEV, ShardingEnv(1, 0), cfg, capacity=1 << 14, lr=3e-3)
    gen = torch.Generator().manual_seed(0)
    k, off, m, ts, T, _keep = make_batch(4, gen, n_items=2000, n_neg=64, max_len=512)
    losses = []
    for _ in range(12):
        opt.zero_grad()
        loss = model(k.to(DEV), off.to(DEV), m, ts.to(DEV))
        loss.backward()
        opt.step()
        losses.append(loss.item())
    torch.cuda.synchronize()
    _lib.check_status()
    assert losses[-1] < losses[0] * 0.9, losses

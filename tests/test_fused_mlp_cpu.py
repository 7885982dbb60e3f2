"""``FusedMLP`` and ``FusedDenseOptimizer`` on their CPU reference path: forward and gradients against an fp32 ``nn.Linear``
stack, the flat parameter / gradient layout, the gradient-ready hook, re-homed gradient buffers, Adam and SGD steps
against ``torch.optim``, and the whole fused DLRM against the unfused one."""
import pytest
import torch

from recsdk_b200.modules.mlp import MLP, FusedMLP
from recsdk_b200.optim import FusedDenseOptimizer, KeyedOptimizerWrapper


def _pair(in_f=13, sizes=(32, 16), final=True):
    torch.manual_seed(0)
    ref = MLP(in_f, list(sizes), final_activation=final)
    fm = FusedMLP(in_f, list(sizes), final_activation=final, device=torch.device("cpu"))
    fm.load_from_linears([m for m in ref.net if isinstance(m, torch.nn.Linear)])
    return ref, fm


def _rel(a, b):
    """Relative error in the Frobenius norm: robust to the few elements whose ReLU flips under bf16 rounding."""
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def _pad(x, fm):
    out = torch.zeros(x.shape[0], fm.in_padded, dtype=torch.bfloat16)
    out[:, : x.shape[1]] = x.to(torch.bfloat16)
    return out


def test_layout_views_and_padding():
    _, fm = _pair()
    assert fm.in_padded == 16 and fm.num_layers == 2 and fm.relu == [True, True]
    assert fm.weight(0).shape == (32, 13) and fm.w32[0].shape == (32, 16) and fm.bias(1).shape == (16,)
    assert torch.all(fm.w32[0][:, 13:] == 0)                               # padded input columns carry zero weights
    assert fm.flat_param.numel() == fm.flat_grad.numel() == fm.flat_shadow.numel() and fm.flat_param.numel() % 64 == 0
    assert fm.flat_shadow.dtype == torch.bfloat16 and torch.equal(fm.w16[0].float(), fm.w32[0].to(torch.bfloat16).float())
    with pytest.raises(ValueError):
        FusedMLP(8, [12, 8])                                               # hidden sizes must be multiples of 8
    with pytest.raises(AssertionError):
        fm(torch.zeros(2, 13, dtype=torch.bfloat16))                       # callers feed the padded width


def _rounded_reference(fm, x):
    """The same network in fp32 autograd with the kernel's rounding points: 16-bit weights, 16-bit activations between
    layers.  -> (output, per-layer weight leaves, per-layer bias leaves, input leaf)."""
    xr = x.detach().float().requires_grad_(True)
    ws = [fm.w32[l].detach().to(torch.bfloat16).float().requires_grad_(True) for l in range(fm.num_layers)]
    bs = [fm.b32[l].detach().clone().requires_grad_(True) for l in range(fm.num_layers)]
    h = xr
    for l in range(fm.num_layers):
        z = h @ ws[l].t() + bs[l]
        h = (torch.relu(z) if fm.relu[l] else z).to(torch.bfloat16).float()
    return h, ws, bs, xr


@pytest.mark.parametrize("final", [True, False])
def test_forward_and_gradients_match_fp32_stack(final):
    _, fm = _pair(final=final)
    xp = _pad(torch.randn(64, 13), fm).requires_grad_(True)
    y = fm(xp)
    yr, ws, bs, xr = _rounded_reference(fm, xp)
    assert y.dtype == torch.bfloat16 and _rel(y, yr) < 1e-3
    g = torch.randn(64, 16).to(torch.bfloat16)
    y.backward(g)
    yr.backward(g.float())
    for l in range(2):
        assert _rel(fm.wgrad[l], ws[l].grad) < 1e-2                        # the kernel path rounds dZ to 16 bits between layers
        assert _rel(fm.bias_grad(l), bs[l].grad) < 1e-2
    assert float(fm.wgrad[0][:, 13:].abs().sum()) == 0.0                   # zero input padding gives zero weight gradients there
    assert _rel(xp.grad, xr.grad) < 1e-2
    # gradients accumulate until the buffers are cleared
    before = fm.flat_grad.clone()
    fm(xp.detach().requires_grad_(True)).backward(g)
    assert torch.allclose(fm.flat_grad, 2 * before, atol=1e-3, rtol=1e-3)
    fm.zero_grad_buffers()
    assert float(fm.flat_grad.abs().sum()) == 0.0


def test_gradient_ready_hook_fires_after_the_last_backward_of_a_step():
    _, fm = _pair()
    fired = []
    fm.set_grad_ready_hook(lambda m: fired.append(float(m.flat_grad.abs().sum())))
    a, b = _pad(torch.randn(8, 13), fm), _pad(torch.randn(8, 13), fm)
    ya, yb = fm(a.requires_grad_(True)), fm(b.requires_grad_(True))        # the module is applied twice in one step
    (ya.float().sum() + yb.float().sum()).backward()
    assert len(fired) == 1 and fired[0] > 0                                # once, with both contributions in place
    with torch.no_grad():
        fm(a)                                                              # no backward will follow: nothing is counted
    fm(a.detach().requires_grad_(True)).float().sum().backward()
    assert len(fired) == 2


def test_rehomed_gradient_buffer_is_the_one_written():
    _, fm = _pair()
    big = torch.zeros(fm.flat_grad.numel() + 100)
    fm.flat_grad.fill_(0.5)
    fm.set_grad_buffer(big[100:])
    assert float(big[100]) == 0.5 and fm.wgrad[0].data_ptr() == big[100:].data_ptr()
    fm.zero_grad_buffers()
    fm(_pad(torch.randn(8, 13), fm).requires_grad_(True)).float().sum().backward()
    assert float(big[100:].abs().sum()) > 0 and float(big[:100].abs().sum()) == 0
    with pytest.raises(AssertionError):
        fm.set_grad_buffer(torch.zeros(3))


@pytest.mark.parametrize("kind", ["adam", "sgd"])
def test_fused_dense_optimizer_matches_torch(kind):
    _, fm = _pair()
    extra = torch.nn.Linear(4, 2)
    holder = torch.nn.ModuleDict({"mlp": fm, "extra": extra})
    frozen = torch.nn.Parameter(torch.ones(3))
    frozen._in_backward_optimizers = True                                  # updated elsewhere: must be left alone
    holder.register_parameter("frozen", frozen)
    opt = FusedDenseOptimizer(holder, kind, lr=0.05, weight_decay=0.01, grad_scale=0.5)
    assert opt.rest == [extra.weight, extra.bias] and len(opt.flat_modules) == 1
    p_ref = fm.flat_param.detach().clone().requires_grad_(True)
    e_ref = [p.detach().clone().requires_grad_(True) for p in extra.parameters()]
    mk = (lambda ps: torch.optim.Adam(ps, lr=0.05, weight_decay=0.01)) if kind == "adam" else (lambda ps: torch.optim.SGD(ps, lr=0.05, weight_decay=0.01))
    t_opt, e_opt = mk([p_ref]), mk(e_ref)
    for step in range(3):
        if step == 2:
            opt.param_groups[0]["lr"] = 0.01                               # a schedule edits the group; both parts follow
            t_opt.param_groups[0]["lr"] = e_opt.param_groups[0]["lr"] = 0.01
        g = torch.randn(fm.flat_grad.numel())
        fm.flat_grad.copy_(g)
        p_ref.grad = 0.5 * g
        for p, q in zip(extra.parameters(), e_ref):
            p.grad = torch.randn_like(p)
            q.grad = p.grad.clone()
        opt.step()
        t_opt.step()
        e_opt.step()
    assert torch.allclose(fm.flat_param, p_ref, atol=1e-6, rtol=1e-5)
    assert all(torch.allclose(p, q, atol=1e-6, rtol=1e-5) for p, q in zip(extra.parameters(), e_ref))
    assert torch.equal(fm.flat_shadow, fm.flat_param.detach().to(torch.bfloat16)) and torch.all(frozen == 1)
    opt.zero_grad()
    assert float(fm.flat_grad.abs().sum()) == 0 and extra.weight.grad is None


def test_keyed_optimizer_wrapper():
    lin = torch.nn.Linear(3, 2)
    w = KeyedOptimizerWrapper(dict(lin.named_parameters()), lambda ps: torch.optim.SGD(ps, lr=1.0))
    lin.weight.grad, lin.bias.grad = torch.ones(2, 3), torch.ones(2)
    before = lin.weight.detach().clone()
    w.step()
    assert torch.allclose(lin.weight, before - 1.0)
    w.zero_grad()
    assert lin.weight.grad is None
    sd = w.state_dict()
    w.load_state_dict(sd)
    empty = KeyedOptimizerWrapper({}, lambda ps: torch.optim.SGD(ps, lr=1.0))
    assert empty.step() is None and empty.state_dict() == {}
    empty.zero_grad()
    empty.load_state_dict({})


def test_fused_dlrm_tracks_the_unfused_model_on_cpu():
    from recsdk_b200.models.dlrm import DLRM, DLRMTrain
    from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig
    from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection
    from recsdk_b200.utils.data import RandomRecDataset

    cfgs = [EmbeddingBagConfig(num_embeddings=40, embedding_dim=16, name="t%d" % i, feature_names=["f%d" % i]) for i in range(3)]
    torch.manual_seed(1)
    plain = DLRMTrain(DLRM(EmbeddingBagCollection(cfgs), 5, [32, 16], [32, 16, 1], fused=False))
    fused = DLRMTrain(DLRM(EmbeddingBagCollection(cfgs), 5, [32, 16], [32, 16, 1], dense_device=torch.device("cpu"), fused=True))
    fused.model.sparse_arch.load_state_dict(plain.model.sparse_arch.state_dict())
    lin = lambda mlp: [m for m in mlp.net if isinstance(m, torch.nn.Linear)]  # noqa: E731
    fused.model.dense_arch.load_from_linears(lin(plain.model.dense_arch))
    fused.model.over_arch.load_from_linears(lin(plain.model.over_arch))
    with torch.no_grad():
        fused.model.head.w32.copy_(plain.model.head.weight[0])
        fused.model.head.b32.copy_(plain.model.head.bias)
    b = RandomRecDataset(["f0", "f1", "f2"], [40] * 3, 64, num_dense=5, seed=2).make_batch()
    lp, (_, zp, _) = plain(b)
    lf, (_, zf, _) = fused(b)
    assert abs(float(lp.detach()) - float(lf.detach())) < 2e-2 and _rel(zf, zp) < 5e-2
    lp.backward()
    lf.backward()
    gp = plain.model.sparse_arch.embedding_bags["t0"].weight.grad
    gf = fused.model.sparse_arch.embedding_bags["t0"].weight.grad
    assert _rel(gf, gp) < 5e-2
    assert _rel(fused.model.head.wgrad, plain.model.head.weight.grad[0]) < 5e-2

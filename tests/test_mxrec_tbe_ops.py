"""``torch.ops.mxrec.split_embedding_codegen_lookup_*``: forward and in-place optimizer backward against a dense PyTorch
statement (an ``nn.EmbeddingBag``-style forward through autograd, then the update formula on the dense gradient)."""
import pytest
import torch

import recsdk_b200.ops.mxrec  # noqa: F401  (registers the operators)

ROWS, DIMS = [50, 30, 40], [16, 8, 16]


def _problem(device, seed=0, shared=False, w_dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    feat_table = [0, 1, 2, 0] if shared else [0, 1, 2]
    F, B = len(feat_table), 6
    starts, acc = [], 0
    for r, d in zip(ROWS, DIMS):
        starts.append(acc)
        acc += r * d
    dev_weights = torch.randn(acc, generator=g).to(w_dtype)
    lengths = torch.randint(0, 5, (F * B,), generator=g)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), lengths.cumsum(0)])
    idx = torch.cat([torch.randint(0, ROWS[feat_table[f]], (int(lengths[f * B:(f + 1) * B].sum()),), generator=g) for f in range(F)])
    fdims = [DIMS[t] for t in feat_table]
    D_offsets = torch.tensor([0] + list(torch.tensor(fdims).cumsum(0)), dtype=torch.int32)
    weights_offsets = torch.tensor([starts[t] for t in feat_table], dtype=torch.long)
    hs = [0]
    seen = set()
    for t in feat_table:
        hs.append(hs[-1] + (ROWS[t] if t not in seen else 0))
        seen.add(t)
    rows_per_table = torch.tensor([ROWS[t] for t in feat_table], dtype=torch.long)
    grad = torch.randn(B, int(D_offsets[-1]), generator=g)
    to = lambda x: x.to(device)
    return dict(feat_table=feat_table, B=B, starts=starts, dev_weights=to(dev_weights), offsets=to(offsets), idx=to(idx),
                D_offsets=to(D_offsets), weights_offsets=to(weights_offsets), hash_size_cumsum=to(torch.tensor(hs)),
                rows_per_table=to(rows_per_table), grad=to(grad))


def _dense_reference(p, pooling_mode):
    """Forward through autograd on per-table fp32 copies -> (out, dense per-table gradients)."""
    tabs = [p["dev_weights"][s: s + r * d].view(r, d).detach().float().clone().requires_grad_(True)
            for s, r, d in zip(p["starts"], ROWS, DIMS)]
    B, off = p["B"], p["offsets"].tolist()
    cols = []
    for f, t in enumerate(p["feat_table"]):
        rows = []
        for b in range(B):
            a, e = off[f * B + b], off[f * B + b + 1]
            v = tabs[t][p["idx"][a:e]].sum(0) if e > a else torch.zeros(DIMS[t], device=tabs[t].device)
            rows.append(v / (e - a) if pooling_mode == 1 and e > a else v)
        cols.append(torch.stack(rows))
    out = torch.cat(cols, dim=1)
    out.backward(p["grad"].float())
    return out.detach(), [t.grad if t.grad is not None else torch.zeros_like(t) for t in tabs], tabs


def _common_args(p, pooling_mode):
    e = torch.empty(0, device=p["dev_weights"].device)
    ph = torch.zeros(1, device=p["dev_weights"].device, requires_grad=True)
    return [ph, p["dev_weights"], e, e, e.int(), p["weights_offsets"], p["D_offsets"], int(p["D_offsets"][-1]), max(DIMS),
            p["hash_size_cumsum"], 8, p["idx"], p["offsets"], pooling_mode, None, None, e.int(), False, 1.0, False]


def _state(p, rowwise=False, fill=0.0):
    n = sum(ROWS) if rowwise else p["dev_weights"].numel()
    offs, acc = [], 0
    for r, d in zip(ROWS, DIMS):
        offs.append(acc)
        acc += r if rowwise else r * d
    buf = torch.full((n,), fill, device=p["dev_weights"].device)
    e = torch.empty(0, device=buf.device)
    per_feature = torch.tensor([offs[t] for t in p["feat_table"]], dtype=torch.long, device=buf.device)
    return buf, [buf, e, e.int(), per_feature], offs


def _run_and_check(device, kind, pooling_mode, shared, w_dtype=torch.float32, tol=1e-5):
    p = _problem(device, seed=3 + pooling_mode, shared=shared, w_dtype=w_dtype)
    ref_out, dense_grads, tabs = _dense_reference(p, pooling_mode)
    lr, eps, b1, b2, it = 0.05, 1e-3, 0.9, 0.99, 3
    args = _common_args(p, pooling_mode)
    rpt = dict(rows_per_table=p["rows_per_table"])
    if kind == "sgd":
        out = torch.ops.mxrec.split_embedding_codegen_lookup_sgd_function(*args, learning_rate=lr, **rpt)
    elif kind == "adagrad":
        m1, margs, _ = _state(p, fill=0.1)
        out = torch.ops.mxrec.split_embedding_codegen_lookup_adagrad_function(*args, *margs, eps=eps, learning_rate=lr, **rpt)
    elif kind == "rowwise":
        m1, margs, roffs = _state(p, rowwise=True, fill=0.1)
        out = torch.ops.mxrec.split_embedding_codegen_lookup_rowwise_adagrad_function(*args, *margs, eps=eps, learning_rate=lr, **rpt)
    else:
        m1, margs, _ = _state(p, fill=0.0)
        m2, margs2, _ = _state(p, fill=0.0)
        out = torch.ops.mxrec.split_embedding_codegen_lookup_adam_function(*args, *margs, *margs2, eps=eps, learning_rate=lr, beta1=b1,
                                                                          beta2=b2, iter=it, **rpt)
    torch.testing.assert_close(out.float(), ref_out, rtol=tol, atol=tol)
    out.backward(p["grad"])
    for t, (s, r, d) in enumerate(zip(p["starts"], ROWS, DIMS)):
        g, w0 = dense_grads[t], tabs[t].detach()
        touched = g.abs().sum(1) > 0
        if kind == "sgd":
            want = w0 - lr * g
        elif kind == "adagrad":
            st = 0.1 + g * g
            want = w0 - lr * g / (st.sqrt() + eps)
        elif kind == "rowwise":
            st = 0.1 + (g * g).mean(1)
            want = w0 - (lr / (st.sqrt() + eps))[:, None] * g
            got_state = m1[roffs[t]: roffs[t] + r]
            torch.testing.assert_close(got_state[touched], st[touched], rtol=1e-4, atol=1e-5)
        else:
            a, v = (1 - b1) * g, (1 - b2) * g * g
            want = w0 - lr * (a / (1 - b1 ** it)) / ((v / (1 - b2 ** it)).sqrt() + eps)
        want = torch.where(touched[:, None], want, w0)
        got = p["dev_weights"][s: s + r * d].view(r, d).float()
        torch.testing.assert_close(got, want, rtol=max(tol, 1e-4), atol=max(tol, 1e-5))


@pytest.mark.parametrize("kind", ["sgd", "adagrad", "rowwise", "adam"])
@pytest.mark.parametrize("pooling_mode", [0, 1])
def test_lookup_functions_cpu(kind, pooling_mode):
    _run_and_check(torch.device("cpu"), kind, pooling_mode, shared=(kind == "adagrad"))


def test_grad_aggregation_two_steps_equal_one_update():
    dev = torch.device("cpu")
    p = _problem(dev, seed=11)
    _, dense_grads, tabs = _dense_reference(p, 0)
    acc = [torch.zeros(r * d) for r, d in zip(ROWS, DIMS)]
    acc_off = torch.zeros(len(ROWS), dtype=torch.long)
    fn = torch.ops.mxrec.split_embedding_codegen_lookup_sgd_function_grad_aggregation
    args = _common_args(p, 0)
    args = args[:13] + [p["idx"], p["offsets"]] + args[13:]
    w_before = p["dev_weights"].clone()
    out = fn(*args, grad_accumulate=acc, grad_accumulate_offsets=acc_off, learning_rate=0.1, use_optimize=False,
             rows_per_table=p["rows_per_table"])
    out.backward(p["grad"])
    torch.testing.assert_close(p["dev_weights"], w_before)                       # nothing applied yet
    args[0] = torch.zeros(1, requires_grad=True)
    out = fn(*args, grad_accumulate=acc, grad_accumulate_offsets=acc_off, learning_rate=0.1, use_optimize=True,
             rows_per_table=p["rows_per_table"])
    out.backward(p["grad"])
    for t, (s, r, d) in enumerate(zip(p["starts"], ROWS, DIMS)):
        want = tabs[t].detach() - 0.1 * 2 * dense_grads[t]
        torch.testing.assert_close(p["dev_weights"][s: s + r * d].view(r, d), want, rtol=1e-5, atol=1e-6)
        assert float(acc[t].abs().sum()) == 0.0


def test_raw_backward_returns_row_gradients():
    dev = torch.device("cpu")
    p = _problem(dev, seed=5)
    _, dense_grads, tabs = _dense_reference(p, 0)
    e = torch.empty(0)
    m1, margs, _ = _state(p, fill=0.0)
    out = torch.ops.mxrec.split_embedding_backward_codegen_adagrad_unweighted_exact_cuda(
        p["grad"], p["dev_weights"], e, e, e.int(), p["weights_offsets"], p["D_offsets"], max(DIMS), p["hash_size_cumsum"], 8, p["idx"],
        p["offsets"], 0, e.int(), 0, 32, False, 0, 0, False, True, *margs, [], e.long(), eps=1e-3, learning_rate=0.05)
    for t, (s, r, d) in enumerate(zip(p["starts"], ROWS, DIMS)):
        torch.testing.assert_close(out[s: s + r * d].view(r, d), dense_grads[t], rtol=1e-5, atol=1e-6)
        st = dense_grads[t] ** 2
        want = tabs[t].detach() - 0.05 * dense_grads[t] / (st.sqrt() + 1e-3)
        torch.testing.assert_close(p["dev_weights"][s: s + r * d].view(r, d), want, rtol=1e-5, atol=1e-6)


def test_raw_backward_grad_aggregation_accumulates_then_applies():
    """The raw ``*_grad_aggregation`` backward: a first call with ``use_optimize=False`` only adds to ``grad_accumulate``, the
    second applies both steps at once; results equal one SGD step on twice the gradient."""
    dev = torch.device("cpu")
    p = _problem(dev, seed=7)
    _, dense_grads, tabs = _dense_reference(p, 0)
    e = torch.empty(0)
    acc = [torch.zeros(r * d) for r, d in zip(ROWS, DIMS)]
    fn = torch.ops.mxrec.split_embedding_backward_codegen_sgd_unweighted_exact_cuda_grad_aggregation
    head = [p["grad"], p["dev_weights"], e, e, e.int(), p["weights_offsets"], p["D_offsets"], max(DIMS), p["hash_size_cumsum"], 8, p["idx"],
            p["offsets"], p["idx"], p["offsets"], 0, e.int(), 0, 32, False, 0, 0, False, True]
    w0 = p["dev_weights"].clone()
    first = fn(*head, acc, torch.zeros(3, dtype=torch.long), learning_rate=0.1, use_optimize=False)
    torch.testing.assert_close(p["dev_weights"], w0)
    for t, (s, r, d) in enumerate(zip(p["starts"], ROWS, DIMS)):
        torch.testing.assert_close(first[s: s + r * d].view(r, d), dense_grads[t], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(acc[t].view(r, d), dense_grads[t], rtol=1e-5, atol=1e-6)
    fn(*head, acc, torch.zeros(3, dtype=torch.long), learning_rate=0.1, use_optimize=True)
    for t, (s, r, d) in enumerate(zip(p["starts"], ROWS, DIMS)):
        torch.testing.assert_close(p["dev_weights"][s: s + r * d].view(r, d), tabs[t].detach() - 0.2 * dense_grads[t], rtol=1e-5, atol=1e-6)
        assert float(acc[t].abs().sum()) == 0.0
    for kind in ("adagrad", "adam"):
        assert hasattr(torch.ops.mxrec, "split_embedding_backward_codegen_%s_unweighted_exact_cuda_grad_aggregation" % kind)


def test_v2_attention_and_distance_linear():
    torch.manual_seed(0)
    lens = [5, 9, 3]
    offs = torch.tensor([0, 5, 14, 17], dtype=torch.int32)
    q, k, v = (torch.randn(17, 2, 16) for _ in range(3))
    a = torch.ops.mxrec.hstu_forward_v2(q, k, v, None, None, 0, 9, None, None, offs, None, None, None, None, None)
    b = torch.ops.mxrec.hstu_jagged.equal(q, k, v, None, None, 0, 9, 0.0, offs)
    torch.testing.assert_close(a, b)
    g = torch.randn_like(a)
    d2 = torch.ops.mxrec.hstu_backward_v2(g, q, k, v, 9, 9, offs, offs, window_size_left=-1, window_size_right=0)
    d1 = torch.ops.mxrec.hstu_jagged_backward.equal(g, q, k, v, None, None, 0, 9, 0.0, offs)
    for x, y in zip(d1[:3], d2[:3]):
        torch.testing.assert_close(x, y)
    x, w, bias = torch.randn(7, 12), torch.randn(32, 12), torch.randn(32)
    outs = torch.ops.mxrec.distance_in_linear_silu(x, w, bias, [8, 8, 8, 8])
    assert len(outs) == 5
    torch.testing.assert_close(outs[4], x @ w.t() + bias, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(torch.cat(outs[:4], 1), torch.nn.functional.silu(x @ w.t() + bias), rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["sgd", "adagrad", "rowwise", "adam"])
@pytest.mark.parametrize("pooling_mode", [0, 1])
def test_lookup_functions_fused_kernels(kind, pooling_mode):
    _run_and_check(torch.device("cuda"), kind, pooling_mode, shared=(kind == "rowwise"))

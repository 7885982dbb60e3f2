"""Embedding lookup / fused backward-update, interaction and loss-head kernels vs fp32 references."""
import pytest
import torch

from recsdk_b200.modules.embedding_configs import DataType, EmbeddingBagConfig, PoolingType
from recsdk_b200.ops import _lib, dense_ops
from recsdk_b200.ops import embedding_ops as E
from recsdk_b200.ops import interaction as I
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.parallel.embeddingbag import ShardedEmbeddingBagCollection
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _make(tables_rows, dims, dtype, opt, pooling=PoolingType.SUM):
    cfgs = [EmbeddingBagConfig(num_embeddings=r, embedding_dim=d, name="t%d" % i, feature_names=["f%d" % i],
                               data_type=dtype, pooling=pooling) for i, (r, d) in enumerate(zip(tables_rows, dims))]
    return ShardedEmbeddingBagCollection(cfgs, {}, ShardingEnv(1, 0), torch.device(DEV), opt, out_dtype=torch.float32)


@pytest.mark.parametrize("dtype,tol", [(DataType.FP32, 1e-5), (DataType.FP16, 2e-3)])
@pytest.mark.parametrize("pooling", [PoolingType.SUM, PoolingType.MEAN])
def test_tbe_forward_backward_rowwise_adagrad(dtype, tol, pooling):
    torch.manual_seed(0)
    rows, dims, B = [50, 1000, 7], [16, 128, 64], 33
    opt = E.OptimizerSpec(kind=E.OPT_ROWWISE_ADAGRAD, lr=0.1, eps=1e-8)
    ebc = _make(rows, dims, dtype, opt, pooling)
    w0 = [ebc.table_weight("t%d" % i).detach().float().cpu().clone() for i in range(3)]
    lens = torch.randint(0, 5, (3 * B,))
    vals = torch.cat([torch.randint(0, rows[t], (int(lens[t * B:(t + 1) * B].sum()),)) for t in range(3)])
    kjt = KeyedJaggedTensor(["f0", "f1", "f2"], vals.to(DEV), lengths=lens.to(DEV), stride=B)
    out = ebc(kjt).values()
    pool = E.POOL_MEAN if pooling == PoolingType.MEAN else E.POOL_SUM
    off = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)])
    ref = E.reference_pooled_forward(w0, vals, off, B, pool)
    assert torch.allclose(out.cpu(), ref, atol=tol, rtol=tol)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    _lib.check_status()
    # reference: exact row-wise adagrad on per-row summed gradients
    gc, col = g.cpu(), 0
    for t in range(3):
        D = dims[t]
        grad = torch.zeros(rows[t], D)
        for b in range(B):
            ids = vals[off[t * B + b]:off[t * B + b + 1]]
            if ids.numel() == 0:
                continue
            gb = gc[b, col:col + D] / (ids.numel() if pool == E.POOL_MEAN else 1)
            grad.index_add_(0, ids, gb.expand(ids.numel(), D))
        touched = torch.zeros(rows[t], dtype=torch.bool)
        touched[vals[off[t * B]:off[(t + 1) * B]]] = True
        acc = (grad * grad).mean(1)
        new = w0[t] - 0.1 * grad / (acc.sqrt() + 1e-8)[:, None]
        exp = torch.where(touched[:, None], new, w0[t])
        got = ebc.table_weight("t%d" % t).detach().float().cpu()
        assert torch.allclose(got, exp, atol=5 * tol, rtol=5 * tol), "table %d" % t
        col += D


@pytest.mark.parametrize("kind", [E.OPT_SGD, E.OPT_ADAGRAD, E.OPT_ADAM])
def test_tbe_other_optimizers_one_hot_long_segments(kind):
    torch.manual_seed(1)
    rows, D, B = 64, 32, 4096     # few rows, many samples -> long segments take the block kernel
    opt = E.OptimizerSpec(kind=kind, lr=0.05, eps=1e-8)
    ebc = _make([rows], [D], DataType.FP32, opt)
    w0 = ebc.table_weight("t0").detach().cpu().clone()
    vals = torch.randint(0, rows, (B,))
    vals[: B // 2] = 3
    kjt = KeyedJaggedTensor(["f0"], vals.to(DEV), lengths=torch.ones(B, dtype=torch.int64, device=DEV), stride=B)
    kjt.one_hot = True
    out = ebc(kjt).values()
    assert torch.allclose(out.cpu(), w0[vals], atol=1e-6)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    _lib.check_status()
    grad = torch.zeros(rows, D).index_add_(0, vals, g.cpu())
    touched = torch.zeros(rows, dtype=torch.bool)
    touched[vals] = True
    if kind == E.OPT_SGD:
        new = w0 - 0.05 * grad
    elif kind == E.OPT_ADAGRAD:
        new = w0 - 0.05 * grad / ((grad * grad).sqrt() + 1e-8)
    else:
        m, v = 0.1 * grad, 0.001 * grad * grad
        new = w0 - (0.05 / 0.1) * m / ((v / 0.001).sqrt() + 1e-8)
    exp = torch.where(touched[:, None], new, w0)
    got = ebc.table_weight("t0").detach().cpu()
    assert torch.allclose(got, exp, atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("F,D,B", [(27, 128, 257), (5, 16, 64), (32, 64, 100)])
def test_dot_interaction(F, D, B):
    torch.manual_seed(2)
    x0 = (torch.randn(B, D, device=DEV) * 0.5).bfloat16().requires_grad_()
    xs = (torch.randn(B, (F - 1) * D, device=DEV) * 0.5).bfloat16().requires_grad_()
    cols = I.interaction_out_cols(F, D)
    out = I.dot_interaction(x0, xs, F, cols)
    ref = I.dot_interaction_ref(x0.detach().cpu(), xs.detach().cpu(), F, cols)
    assert torch.allclose(out.float().cpu(), ref, atol=5e-2, rtol=2e-2)
    dR = (torch.randn(B, cols, device=DEV) * 0.5).bfloat16()
    out.backward(dR)
    r0, rs = I.dot_interaction_bwd_ref(x0.detach().cpu(), xs.detach().cpu(), dR.cpu(), F)
    assert torch.allclose(x0.grad.float().cpu(), r0, atol=0.15, rtol=3e-2)
    assert torch.allclose(xs.grad.float().cpu(), rs, atol=0.15, rtol=3e-2)


def test_bce_head_and_colsum_and_adam():
    torch.manual_seed(3)
    B, K = 1000, 256
    h = torch.relu(torch.randn(B, K, device=DEV)).bfloat16()
    w, b = torch.randn(K, device=DEV) * 0.1, torch.randn(1, device=DEV)
    y = (torch.rand(B, device=DEV) < 0.3).float()
    logits, loss = torch.empty(B, device=DEV), torch.zeros(1, device=DEV)
    dh = torch.empty(B, K, dtype=torch.bfloat16, device=DEV)
    dw, db = torch.zeros(K, device=DEV), torch.zeros(1, device=DEV)
    dense_ops.bce_head(h, w, b, y, 1.0 / B, logits, loss, dh, dw, db, relu_mask=True)
    rl, rloss = torch.empty(B), torch.zeros(1)
    rdh, rdw, rdb = torch.empty(B, K), torch.zeros(K), torch.zeros(1)
    dense_ops.bce_head(h.cpu(), w.cpu(), b.cpu(), y.cpu(), 1.0 / B, rl, rloss, rdh, rdw, rdb, relu_mask=True)
    assert torch.allclose(logits.cpu(), rl, atol=1e-3, rtol=1e-3)
    assert torch.allclose(loss.cpu(), rloss, atol=1e-4, rtol=1e-4)
    assert torch.allclose(dh.float().cpu(), rdh, atol=1e-5, rtol=1e-2)
    assert torch.allclose(dw.cpu(), rdw, atol=1e-5, rtol=1e-3)
    assert torch.allclose(db.cpu(), rdb, atol=1e-6, rtol=1e-3)
    a = torch.randn(3000, 200, device=DEV).bfloat16()
    cs = torch.zeros(200, device=DEV)
    dense_ops.colsum16(a, cs)
    assert torch.allclose(cs.cpu(), a.float().sum(0).cpu(), atol=1e-2, rtol=1e-3)
    p = torch.randn(10000, device=DEV)
    g = torch.randn(10000, device=DEV)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    sh = torch.empty(10000, dtype=torch.bfloat16, device=DEV)
    pc, mc, vc = p.cpu().clone(), m.cpu().clone(), v.cpu().clone()
    dense_ops.adam_flat(p, g, m, v, sh, 1e-2, 0.9, 0.999, 1e-8, 0.0, 1)
    dense_ops.adam_flat(pc, g.cpu(), mc, vc, None, 1e-2, 0.9, 0.999, 1e-8, 0.0, 1)
    assert torch.allclose(p.cpu(), pc, atol=1e-6, rtol=1e-5)
    assert torch.allclose(sh.float().cpu(), pc, atol=1e-2, rtol=1e-2)


def test_grouped_collection_mixed_dtype_and_pooling():
    """Tables of one collection that differ in storage dtype and pooling: one fused collection per group behind one module;
    pooled columns come back in the order of the original features; every group trains."""
    from recsdk_b200.parallel.grouped_embeddingbag import GroupedShardedEmbeddingBagCollection, needs_grouping

    torch.manual_seed(1)
    spec = [(50, 16, DataType.FP32, PoolingType.SUM), (300, 32, DataType.FP16, PoolingType.SUM),
            (70, 16, DataType.FP32, PoolingType.MEAN), (90, 8, DataType.FP32, PoolingType.SUM)]       # group of t0 is not contiguous
    cfgs = [EmbeddingBagConfig(num_embeddings=r, embedding_dim=d, name="t%d" % i, feature_names=["f%d" % i], data_type=dt,
                               pooling=p) for i, (r, d, dt, p) in enumerate(spec)]
    assert needs_grouping(cfgs) and not needs_grouping(cfgs[:1])
    opt = E.OptimizerSpec(kind=E.OPT_SGD, lr=0.5)
    m = GroupedShardedEmbeddingBagCollection(cfgs, {}, ShardingEnv(1, 0), torch.device(DEV), opt, out_dtype=torch.float32)
    assert len(m.groups) == 3
    B = 21
    lens = torch.randint(0, 4, (4 * B,))
    vals = torch.cat([torch.randint(0, spec[t][0], (int(lens[t * B:(t + 1) * B].sum()),)) for t in range(4)])
    kjt = KeyedJaggedTensor(["f0", "f1", "f2", "f3"], vals.to(DEV), lengths=lens.to(DEV), stride=B)
    w0 = [m.table_weight("t%d" % i).detach().float().cpu().clone() for i in range(4)]
    kt = m(kjt)
    assert kt.keys() == ["f0", "f1", "f2", "f3"] and kt.length_per_key() == [16, 32, 16, 8]
    out = kt.values()
    off = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)])
    col = 0
    for t, (r, d, dt, p) in enumerate(spec):
        lt = lens[t * B:(t + 1) * B]
        o = torch.cat([torch.zeros(1, dtype=torch.int64), lt.cumsum(0)])
        ref = E.reference_pooled_forward([w0[t]], vals[off[t * B]:off[(t + 1) * B]], o, B,
                                         E.POOL_MEAN if p == PoolingType.MEAN else E.POOL_SUM)
        tol = 2e-3 if dt == DataType.FP16 else 1e-5
        assert torch.allclose(out[:, col:col + d].cpu(), ref, atol=tol, rtol=tol), "feature %d" % t
        col += d
    out.sum().backward()
    torch.cuda.synchronize()
    _lib.check_status()
    for t in range(4):
        touched = torch.zeros(spec[t][0], dtype=torch.bool)
        touched[vals[off[t * B]:off[(t + 1) * B]]] = True
        got = m.table_weight("t%d" % t).detach().float().cpu()
        assert not torch.allclose(got[touched], w0[t][touched]) and torch.equal(got[~touched], w0[t][~touched])

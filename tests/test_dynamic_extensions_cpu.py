"""Operator-level dynamic-embedding calls under the reference's names (``dynamic_emb_extensions``) on the host table."""
import pickle

import pytest
import torch

import recsdk_b200.dynamic.extensions as X

pytestmark = pytest.mark.skipif(torch.cuda.is_available(), reason="the host table is what a machine without CUDA gets")

DIM = 4


def _table(opt=X.OptimizerType.SGD, evict=X.EvictStrategy.kLru, cap=64, init=None):
    return X.DynamicEmbTable(X.DynamicEmbDataType.Int64, X.DynamicEmbDataType.Float32, evict, dim=DIM, init_capaity=cap, max_capaity=cap,
                             initializer_args=init or X.InitializerArgs("debug"), optimizer_type=int(opt))


def test_table_handle_queries_and_initializer_args():
    a = X.InitializerArgs("normal", 0.5, 2.0, -1.0, 1.0, 3.0)
    assert a == X.InitializerArgs("normal", 0.5, 2.0, -1.0, 1.0, 3.0) and a != X.InitializerArgs("normal")
    assert pickle.loads(pickle.dumps(a)) == a
    with pytest.raises(ValueError, match="unknown initializer mode"):
        X.InitializerArgs("xavier")
    t = _table(X.OptimizerType.AdaGrad, cap=100)
    assert t.get_key_type() == X.DynamicEmbDataType.Int64 and t.get_value_type() == X.DynamicEmbDataType.Float32
    assert t.get_evict_strategy() == X.EvictStrategy.kLru == t.evict_strategy()
    assert t.get_max_capacity() == 128                                    # rounded up to a power of two
    assert t.get_emb_cols() == DIM == X.dyn_emb_cols(t) and t.optstate_dim() == DIM
    assert t.get_initializer_args() == X.InitializerArgs("debug")
    t.set_initial_optstate(0.25)
    assert t.get_initial_optstate() == 0.25
    assert X.dyn_emb_rows(t) == 0 and X.dyn_emb_is_pure_hbm_mode(t)
    with pytest.raises(ValueError, match="Float32"):
        X.DynamicEmbTable(X.DynamicEmbDataType.Int64, X.DynamicEmbDataType.BFloat16, X.EvictStrategy.kLru)
    assert X.device_timestamp() > 0


def test_find_or_insert_find_assign_erase():
    t = _table()
    keys = torch.tensor([7, 100003, 7, 42])
    vals = torch.full((4, DIM), -1.0)
    X.find_or_insert(t, 4, keys, vals, unique_key=False)
    assert torch.equal(vals[:, 0], torch.tensor([7.0, 3.0, 7.0, 42.0])) and X.dyn_emb_rows(t) == 3      # debug init: key % 100000
    out, founds = torch.full((3, DIM), -5.0), torch.zeros(3, dtype=torch.bool)
    X.find(t, 3, torch.tensor([42, 9, 7]), out, founds)
    assert founds.tolist() == [True, False, True]
    assert torch.equal(out[:, 0], torch.tensor([42.0, -5.0, 7.0]))        # the missing key's row is left alone
    X.assign(t, 2, torch.tensor([7, 9]), torch.tensor([[1.0] * DIM, [2.0] * DIM]))
    X.find(t, 3, torch.tensor([42, 9, 7]), out, founds)
    assert out[2].tolist() == [1.0] * DIM and founds.tolist() == [True, False, True]
    # n limits the call
    X.find_or_insert(t, 1, torch.tensor([500, 501]), torch.zeros(2, DIM))
    assert X.dyn_emb_rows(t) == 4
    X.erase(t, 1, torch.tensor([7]))
    X.find(t, 1, torch.tensor([7]), out, founds)
    assert not bool(founds[0])
    X.clear(t)
    assert X.dyn_emb_rows(t) == 0
    X.reserve(t, 256)
    assert t.table.capacity >= 256


def test_scores_required_for_lfu_and_export_by_threshold():
    t = _table(evict=X.EvictStrategy.kCustomized)
    with pytest.raises(ValueError, match="Must specify the score"):
        X.find_or_insert(t, 1, torch.tensor([1]), torch.zeros(1, DIM))
    X.find_or_insert(t, 2, torch.tensor([1, 2]), torch.zeros(2, DIM), score=5)
    X.find_or_insert(t, 1, torch.tensor([3]), torch.zeros(1, DIM), score=9)
    n = torch.zeros(1, dtype=torch.int64)
    X.count_matched(t, 9, n)
    assert int(n) == 1                                                    # score >= threshold
    X.count_matched(t, 5, n)
    assert int(n) == 3
    keys, vals = torch.zeros(8, dtype=torch.int64), torch.zeros(8, DIM)
    X.export_batch_matched(t, 6, 64, 0, n, keys, vals)
    assert int(n) == 1 and int(keys[0]) == 3 and vals[0, 0] == 3.0
    cnt, sc = torch.zeros(1, dtype=torch.int64), torch.zeros(8, dtype=torch.int64)
    t.export_batch(64, 0, cnt, keys, vals, sc)
    assert int(cnt) == 3 and sorted(keys[:3].tolist()) == [1, 2, 3] and sorted(sc[:3].tolist()) == [5, 5, 9]


def test_insert_and_evict_reports_victims_and_load():
    t = X.DynamicEmbTable(X.DynamicEmbDataType.Int64, X.DynamicEmbDataType.Float32, X.EvictStrategy.kLru, dim=DIM, init_capaity=2,
                          max_capaity=2, initializer_args=X.InitializerArgs("constant", value=0.0))
    ek, ev, es, ec = torch.zeros(4, dtype=torch.int64), torch.zeros(4, DIM), torch.zeros(4, dtype=torch.int64), torch.zeros(1, dtype=torch.int64)
    X.insert_and_evict(t, 2, torch.tensor([10, 11]), torch.ones(2, DIM), None, ek, ev, es, ec)
    assert int(ec) == 0 and X.dyn_emb_rows(t) == 2
    X.insert_and_evict(t, 1, torch.tensor([12]), torch.full((1, DIM), 2.0), None, ek, ev, es, ec)
    assert int(ec) == 1 and int(ek[0]) == 10 and ev[0].tolist() == [1.0] * DIM          # the least recently used key left
    t.load(1, torch.tensor([11]), torch.full((1, DIM), 7.0))                              # overwrite through the handle
    out, f = torch.zeros(1, DIM), torch.zeros(1, dtype=torch.bool)
    X.find(t, 1, torch.tensor([11]), out, f)
    assert bool(f[0]) and out[0].tolist() == [7.0] * DIM


def test_accum_or_assign_and_find_and_initialize():
    t = _table()
    X.find_or_insert(t, 1, torch.tensor([5]), torch.zeros(1, DIM))
    X.accum_or_assign(t, 3, torch.tensor([5, 6, 8]), torch.tensor([[1.0] * DIM, [2.0] * DIM, [3.0] * DIM]), torch.tensor([True, True, False]))
    out, f = torch.zeros(3, DIM), torch.zeros(3, dtype=torch.bool)
    X.find(t, 3, torch.tensor([5, 6, 8]), out, f)
    assert f.tolist() == [True, False, True]                              # accumulate does not insert, assign does
    assert out[0].tolist() == [6.0] * DIM and out[2].tolist() == [3.0] * DIM
    ptrs = torch.zeros(2, dtype=torch.int64)
    vals = torch.zeros(2, DIM)
    X.find_and_initialize(t, 2, torch.tensor([8, 77]), ptrs, vals, f, X.InitializerArgs("constant", value=0.5))
    assert f[:2].tolist() == [True, False] and vals[0].tolist() == [3.0] * DIM and vals[1].tolist() == [0.5] * DIM
    assert int(ptrs[0]) != 0 and int(ptrs[1]) == 0 and X.dyn_emb_rows(t) == 2          # nothing was inserted
    X.find_and_initialize(t, 1, torch.tensor([77]), ptrs, vals, f)                         # the table's own (debug) initializer
    assert vals[0].tolist() == [77.0] * DIM


@pytest.mark.parametrize("opt,name", [(X.OptimizerType.SGD, "sgd"), (X.OptimizerType.AdaGrad, "adagrad"),
                                      (X.OptimizerType.RowWiseAdaGrad, "rowwise_adagrad"), (X.OptimizerType.AdamW, "adamW")])
def test_optimizer_calls_agree_across_the_three_forms(opt, name):
    """fused (gathered rows), with_table (keys) and with_pointer (row addresses) apply the same update."""
    extra = {"sgd": (0.1,), "adagrad": (0.1, 1e-8), "rowwise_adagrad": (0.1, 1e-8), "adamW": (0.1, 0.9, 0.999, 1e-8, 0.01, 1)}[name]
    keys = torch.tensor([3, 4, 5])
    grads = torch.randn(3, DIM, generator=torch.Generator().manual_seed(0))
    tabs = [_table(opt) for _ in range(2)]
    W = DIM + tabs[0].optstate_dim()
    rows0 = torch.zeros(3, W)
    for t in tabs:
        X.find_or_insert(t, 3, keys, rows0)
    fused = rows0.clone()
    getattr(X, "dynamic_emb_%s_fused" % name)(grads, fused, *extra)
    getattr(X, "dynamic_emb_%s_with_table" % name)(tabs[0], 3, keys, grads, *extra)
    ptrs, f = torch.zeros(3, dtype=torch.int64), torch.zeros(3, dtype=torch.bool)
    X.find_pointers(tabs[1], 3, keys, ptrs, f)
    assert bool(f.all())
    if name == "sgd":
        X.dynamic_emb_sgd_with_pointer(grads, ptrs, None, *extra, region=tabs[1])
    else:
        getattr(X, "dynamic_emb_%s_with_pointer" % name)(grads, ptrs, None, tabs[1].optstate_dim(), *extra, region=tabs[1])
    for t in tabs:
        got = torch.zeros(3, W)
        X.find(t, 3, keys, got, f)
        assert torch.allclose(got, fused, atol=1e-6), name
    assert not torch.equal(fused[:, :DIM], rows0[:, :DIM])
    # addresses are checked: a stray one is refused, and a call without a region too
    with pytest.raises(IndexError, match="not a row of the table"):
        X.load_from_pointer(torch.tensor([int(ptrs[0]) + 8]), torch.zeros(1, DIM), region=tabs[1])
    with pytest.raises(ValueError, match="region="):
        X.load_from_pointer(ptrs, torch.zeros(3, DIM))
    got = X.load_from_pointer(ptrs, torch.zeros(3, DIM), region=tabs[1])
    assert torch.allclose(got, fused[:, :DIM], atol=1e-6)
    with pytest.raises(ValueError, match="the call is for"):
        other = X.dynamic_emb_sgd_with_table if name != "sgd" else X.dynamic_emb_adagrad_with_table
        other(tabs[0], 3, keys, grads, *((0.1,) if name != "sgd" else (0.1, 1e-8)))


def test_id_preprocessing_and_pooled_lookup():
    keys = torch.tensor([5, 3, 5, 9, 3, 3])
    u, inv, cnt = X.unique_op(keys)
    assert torch.equal(u[inv], keys) and int(cnt.sum()) == 6
    ub, inv2, uoffs, _c = X.segmented_unique_op(keys, torch.tensor([0, 3, 6]))
    assert uoffs.tolist() == [0, 2, 4] and torch.equal(ub[inv2], keys)
    flags = torch.tensor([True, False, True, True, False, False])
    out, n = torch.zeros(6, dtype=torch.int64), torch.zeros(1, dtype=torch.int64)
    X.select(flags, keys, out, n)
    assert int(n) == 3 and out[:3].tolist() == [5, 5, 9]
    X.select_index(flags, out, n)
    assert int(n) == 3 and out[:3].tolist() == [0, 2, 3]
    # 2 features x batch 2 over 2 tables (one feature each)
    offsets = torch.tensor([0, 2, 3, 5, 6])
    assert X.get_table_range_op(offsets, torch.tensor([0, 1, 2])).tolist() == [0, 3, 6]
    rev, unums, uo, uidx = torch.zeros(6, dtype=torch.int64), torch.zeros(2, dtype=torch.int64), torch.zeros(3, dtype=torch.int64), torch.zeros(6, dtype=torch.int64)
    noffs, nlens = torch.zeros(5, dtype=torch.int64), torch.zeros(4, dtype=torch.int64)
    X.dedup_input_indices_op(keys, offsets, torch.tensor([0, 1, 2]), 2, 2, rev, unums, uo, uidx, noffs, nlens)
    assert unums.tolist() == [2, 2] and uo.tolist() == [0, 2, 4] and torch.equal(uidx[rev], keys)
    assert int(nlens.sum()) == 4 and noffs.tolist()[-1] == 4

    # pooled forward over distinct rows and its gradient
    src = torch.arange(4 * DIM, dtype=torch.float32).view(4, DIM)
    dst = torch.zeros(2, 2 * DIM)
    X.lookup_forward(src, dst, offsets, rev, 0, 2 * DIM, 0, DIM, 6, 2)
    rows = src[rev]
    want = torch.stack([torch.cat([rows[0:2].sum(0), rows[3:5].sum(0)]), torch.cat([rows[2:3].sum(0), rows[5:6].sum(0)])])
    assert torch.allclose(dst, want)
    dst_mean = torch.zeros(2, 2 * DIM)
    X.lookup_forward(src, dst_mean, offsets, rev, 1, 2 * DIM, 0, DIM, 6, 2)
    assert torch.allclose(dst_mean[0, :DIM], rows[0:2].mean(0))
    grad = torch.randn(2, 2 * DIM, generator=torch.Generator().manual_seed(1))
    ubuf = torch.zeros(4, DIM)
    X.lookup_backward(grad, ubuf, uidx, rev, offsets, DIM, 2, 2, 2, 6, 0)
    srcp = src.clone().requires_grad_(True)
    r = srcp[rev]
    pooled = torch.stack([torch.cat([r[0:2].sum(0), r[3:5].sum(0)]), torch.cat([r[2:3].sum(0), r[5:6].sum(0)])])
    pooled.backward(grad)
    assert torch.allclose(ubuf, srcp.grad, atol=1e-6)
    g2, u2 = X.reduce_grads(torch.ones(6, DIM), uidx[:4], rev)
    assert g2[:, 0].tolist() == torch.bincount(rev, minlength=4).float().tolist() and u2 is not None
    assert torch.equal(X.gather_embedding(src, torch.tensor([3, 0])), src[[3, 0]])


def test_initializer_calls():
    ctx = X.CurandStateContext()
    buf = torch.zeros(8, 16)
    idx = torch.tensor([1, 3, 5])
    X.uniform_init(buf, idx, ctx, -0.5, 0.5)
    assert bool((buf[idx].abs() <= 0.5).all()) and bool((buf[idx] != 0).any()) and bool((buf[[0, 2, 4, 6, 7]] == 0).all())
    X.normal_init(buf, idx, ctx, 10.0, 0.1)
    assert abs(float(buf[idx].mean()) - 10.0) < 0.2
    X.truncated_normal_init(buf, idx, ctx, 0.0, 1.0, -0.3, 0.3)
    assert bool((buf[idx].abs() <= 0.3).all())
    X.const_init(buf, idx, 2.5)
    assert bool((buf[idx] == 2.5).all())
    X.debug_init(buf, idx, torch.tensor([100007, 8, 9]))
    assert buf[1, 0] == 7.0 and buf[3, 5] == 8.0 and buf[5, 15] == 9.0
    with pytest.raises(ValueError, match="rows, dim"):
        X.const_init(torch.zeros(4), idx, 1.0)

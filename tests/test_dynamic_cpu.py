"""Dynamic embedding stack on the CPU (dictionary-backed table): training math vs the A100 golden losses
recorded with upstream dynamicemb v25.09 (reference: dynamic_emb/tests/precision_consistency/scenario.py and
golden/reference_v25.09.json), dump / load round trip incl. a world-size change, admission, caching + disk tier."""
import numpy as np
import pytest
import torch

from recsdk_b200.dynamic import (DiskStorage, DynamicEmbDump, DynamicEmbeddingBagCollection, DynamicEmbInitializerArgs,
                                 DynamicEmbInitializerMode, DynamicEmbLoad, DynamicEmbScoreStrategy, DynamicEmbTableOptions,
                                 OptimizerType, get_score, incremental_dump, set_score)
from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor

GOLDEN = {
    OptimizerType.SGD: [280655424.0, 44904868.0, 7184778.5, 1149564.5, 183930.21875],
    OptimizerType.ADAM: [280655424.0, 280547328.0, 280439232.0, 280331136.0, 280223104.0],
    OptimizerType.ADAGRAD: [280655424.0, 280547328.0, 280470880.0, 280408512.0, 280354464.0],
    OptimizerType.ROWWISE_ADAGRAD: [280655424.0, 280547328.0, 280470880.0, 280408512.0, 280354464.0],
}


def _lcg_ids(seed, n):
    x, out = seed, []
    for _ in range(n):
        x = (1103515245 * x + 12345) & 0x7FFFFFFF
        out.append(x % 1024)
    return out


def _scenario_batch():
    # 2 tables / features, batch 8, 3 ids per bag, ids from an LCG seeded 1234 + feature
    vals = [_lcg_ids(1234 + i, 8 * 3) for i in range(2)]
    return KeyedJaggedTensor(["cate_0", "cate_1"], torch.tensor(vals[0] + vals[1], dtype=torch.int64),
                             lengths=torch.full((16,), 3, dtype=torch.int64), stride=8)


def _make(opt, **kw):
    cfgs = [EmbeddingBagConfig(num_embeddings=1024, embedding_dim=8, name="t_%d" % i, feature_names=["cate_%d" % i])
            for i in range(2)]
    options = {c.name: DynamicEmbTableOptions(
        initializer_args=DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.DEBUG),
        score_strategy=DynamicEmbScoreStrategy.STEP, **kw) for c in cfgs}
    return DynamicEmbeddingBagCollection(cfgs, options, ShardingEnv(1, 0), torch.device("cpu"), optimizer_type=opt,
                                         learning_rate=0.1, eps=1e-8)


@pytest.mark.parametrize("opt", list(GOLDEN))
def test_precision_consistency_golden(opt):
    m = _make(opt)
    kjt = _scenario_batch()
    losses = []
    for _ in range(5):
        out = m(kjt).values()
        loss = (out * out).sum()
        loss.backward()
        losses.append(loss.item())
    tol = 4e-5 if opt == OptimizerType.ADAM else 5e-7   # fp32 summation-order noise (1-2 ULP)
    for got, want in zip(losses, GOLDEN[opt]):
        assert abs(got - want) <= tol * abs(want) + 1e-3, (losses, GOLDEN[opt])


def test_dump_load_roundtrip_and_scores(tmp_path):
    m = _make(OptimizerType.ADAM)
    kjt = _scenario_batch()
    for _ in range(3):
        (m(kjt).values() ** 2).sum().backward()
    assert get_score(m)[""]["t_0"] == 3
    DynamicEmbDump(str(tmp_path / "ck"), m, optim=True)
    m2 = _make(OptimizerType.ADAM)
    loaded = DynamicEmbLoad(str(tmp_path / "ck"), m2, optim=True)
    assert loaded[""]["t_0"] == m.table("t_0").size()
    a = (m(kjt).values() ** 2).sum()
    b = (m2(kjt).values() ** 2).sum()
    assert torch.allclose(a, b, rtol=1e-6)
    a.backward(); b.backward()                                    # optimizer state travelled too
    assert torch.allclose((m(kjt).values() ** 2).sum(), (m2(kjt).values() ** 2).sum(), rtol=1e-6)
    # different world size on load: rank 1 of 2 keeps odd keys only
    m3 = _make(OptimizerType.ADAM)
    m3.rank, m3.world = 1, 2
    m3.load(str(tmp_path / "ck" / "root"))
    keys, _, _ = m3.lookup.export_keys_values("t_0")
    assert keys.numel() and (keys % 2 == 1).all()
    with pytest.raises(FileExistsError):
        DynamicEmbDump(str(tmp_path / "ck"), m)
    k = get_score(m)[""]["t_0"]                                  # STEP strategy: score = global step
    inc, cur = incremental_dump(m, k + 1)
    assert inc[""]["t_0"][0].numel() == 0 and cur[""]["t_0"] == k
    (m(kjt).values() ** 2).sum().backward()
    inc, _ = incremental_dump(m, k + 1)                          # only what the last step touched
    assert inc[""]["t_0"][0].numel() == m.table("t_0").size()
    set_score(m, 10)
    assert get_score(m)[""]["t_1"] == 10


def test_admission_threshold():
    m = _make(OptimizerType.SGD, admit_threshold=2)
    kjt = _scenario_batch()
    first = m(kjt).values()
    assert first.abs().sum().item() == 0 and m.table("t_0").size() == 0        # first sighting: default value
    second = m(kjt).values()
    assert second.abs().sum().item() > 0 and m.table("t_0").size() > 0


def test_caching_with_disk_storage(tmp_path):
    cfgs = [EmbeddingBagConfig(num_embeddings=64, embedding_dim=8, name="t", feature_names=["f"])]
    disk = DiskStorage("t", [str(tmp_path / "d0")], 8)
    opts = {"t": DynamicEmbTableOptions(initializer_args=DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.DEBUG),
                                        caching=True, external_storage=disk, max_capacity=16, init_capacity=16)}
    m = DynamicEmbeddingBagCollection(cfgs, opts, ShardingEnv(1, 0), torch.device("cpu"), optimizer_type=OptimizerType.SGD,
                                      learning_rate=0.5)
    seen = {}
    for step in range(6):
        ids = torch.arange(step * 10, step * 10 + 16, dtype=torch.int64)
        kjt = KeyedJaggedTensor(["f"], ids, lengths=torch.ones(16, dtype=torch.int64), stride=16)
        out = m(kjt).values()
        for i, k in enumerate(ids.tolist()):
            if k in seen:
                assert torch.allclose(out[i], seen[k]), "row of key %d changed across cache eviction" % k
        out.sum().backward()
        for i, k in enumerate(ids.tolist()):
            seen[k] = out[i].detach() - 0.5
    assert disk.size() > 0 and m.table("t").table.size() <= 16


def test_host_table_adam_weight_decay_is_decoupled():
    """The reference's Adam multiplies the weights by ``1 - lr * weight_decay`` and keeps the decay out of the moments
    (dynamic_emb ``csrc/dynamic_emb_op.cpp:1602``)."""
    import torch
    from recsdk_b200.dynamic.hkv import HostDynamicTable, InitializerArgs, InitMode, OptimizerType

    t = HostDynamicTable(4, 64, optimizer=OptimizerType.ADAM, init=InitializerArgs(mode=InitMode.CONSTANT, value=0.5))
    keys = torch.arange(1, 6, dtype=torch.int64)
    slots = t.find_or_insert(keys)[0]
    g = torch.full((5, 4), 0.25)
    t.update(slots, g, lr=0.1, eps=1e-8, weight_decay=0.05, step=1)
    want = 0.5 * (1 - 0.1 * 0.05) - 0.1 * 1.0 / (1.0 + 1e-8)      # m_hat / sqrt(v_hat) == 1 for a constant gradient
    got = t.gather(slots)[:, :4]
    assert torch.allclose(got, torch.full((5, 4), want), atol=1e-6)


def test_variable_interface_eval_lookup_and_matched_export():
    import torch
    from recsdk_b200.dynamic.hkv import EvictStrategy, HostDynamicTable, InitializerArgs, InitMode

    t = HostDynamicTable(4, 64, evict_strategy=EvictStrategy.CUSTOMIZED, init=InitializerArgs(mode=InitMode.CONSTANT, value=0.5))
    t.find_or_insert(torch.tensor([3, 5, 9]), scores=torch.tensor([10, 20, 30]))
    rows, found = t.find_and_initialize(torch.tensor([5, 7]), value=-1.0)
    assert found.tolist() == [True, False]
    assert torch.equal(rows, torch.tensor([[0.5] * 4, [-1.0] * 4]))
    assert t.size() == 3                                          # the miss was not inserted
    assert t.count_matched(20) == 2
    keys, scores, vals, _ = t.export_batch_matched(20)
    assert sorted(keys.tolist()) == [5, 9] and sorted(scores.tolist()) == [20, 30] and vals.shape == (2, 4)


def test_batched_tables_prefetch_memory_report_and_accessors(tmp_path):
    """Module-level surface of the batched dynamic tables: prefetch brings storage-tier rows into the cache ahead of the
    forward (sequence mode, opt-in), the memory report splits rows into embedding / optimizer state per tier."""
    from recsdk_b200.dynamic.batched_dynamicemb_table import BatchedDynamicEmbeddingTablesV2
    from recsdk_b200.dynamic.dynamicemb_config import DynamicEmbPoolingMode

    disk = DiskStorage("t", [str(tmp_path / "d0")], 8 + 8)                       # dim 8 + Adagrad state 8
    o = DynamicEmbTableOptions(initializer_args=DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.DEBUG), caching=True,
                               external_storage=disk, max_capacity=16, init_capacity=16)
    o.dim, o.optimizer_type = 8, OptimizerType.ADAGRAD
    m = BatchedDynamicEmbeddingTablesV2([o], ["t"], DynamicEmbPoolingMode.NONE, device=torch.device("cpu"), learning_rate=0.5)
    assert m.caches == m.tables and m.table_names == ["t"]
    rep = m.memory_report()[0]
    assert rep["capacity"] == 16 and rep["dim"] == 8 and rep["optim_state_dim"] == 8
    assert rep["total_bytes"] == {"total": 16 * 64, "embedding": 16 * 32, "optim_state": 16 * 32}
    assert rep["storage_tier"] is not None and "t" in m.print_memory_consume()
    ids = torch.arange(0, 12, dtype=torch.int64)
    off = torch.arange(0, 13, dtype=torch.int64)
    with pytest.raises(RuntimeError, match="not enabled"):
        m.prefetch(ids, off)
    # fill the table and push the first keys down to the storage tier
    for base in (0, 12, 24):
        out = m(torch.arange(base, base + 12, dtype=torch.int64), off, [12], 12)
        out.sum().backward()
    assert disk.size() > 0
    m.set_record_cache_metrics(True)
    m.enable_prefetch = True
    m.prefetch(ids, off)                                                         # keys 0..11 come back from the disk tier
    assert m.num_prefetch_ahead == 1 and m.tables[0].metrics["storage_hits"] > 0
    hits_before = m.tables[0].metrics["storage_hits"]
    rows = m(ids, off, [12], 12)
    assert m.num_prefetch_ahead == 0
    assert m.tables[0].metrics["storage_hits"] == hits_before                    # the forward found everything in the cache
    assert torch.allclose(rows[:, 0], ids.float() % 100000 - 0.5)                # DEBUG init = key, one SGD-like step of 0.5 ... Adagrad
    pooled = BatchedDynamicEmbeddingTablesV2([o], ["t"], DynamicEmbPoolingMode.SUM, device=torch.device("cpu"))
    pooled.enable_prefetch = True
    with pytest.raises(RuntimeError, match="sequence"):
        pooled.prefetch(ids, off)
    w = m.split_embedding_weights()
    assert len(w) == 1 and w[0].shape[1] == 8
    m.reset_cache_states()
    assert m.tables[0].metrics["storage_hits"] == 0

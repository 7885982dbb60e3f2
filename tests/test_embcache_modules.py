"""Multi-tier tables: a tiny device cache over the host table must train exactly like a plain full table
(rows migrate between tiers with their optimizer state), survive save / load, and honour admission."""
import numpy as np
import pytest
import torch

from recsdk_b200.embcache import (AdmitAndEvictConfig, EmbCacheEmbeddingBagCollection, EmbCacheEmbeddingBagConfig,
                                  EmbCacheShardedEmbeddingBagCollection, EmbCacheTrainPipelineSparseDist, Saver)
from recsdk_b200.ops import embedding_ops as E
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _tables(**kw):
    return [EmbCacheEmbeddingBagConfig(num_embeddings=1000, embedding_dim=8, name="t0", feature_names=["f0"], **kw),
            EmbCacheEmbeddingBagConfig(num_embeddings=500, embedding_dim=16, name="t1", feature_names=["f1", "f2"], **kw)]


def _batch(g, B=6):
    lens = torch.randint(1, 4, (3 * B,), generator=g)
    vals = torch.randint(0, 60, (int(lens.sum()),), generator=g)
    return KeyedJaggedTensor(["f0", "f1", "f2"], vals, lengths=lens)


def _sharded(tables, cache_rows, opt=torch.optim.Adagrad, lr=0.1, device="cpu"):
    ebc = EmbCacheEmbeddingBagCollection(tables, 1, 6, [3, 3], device=device, embedding_optimizer_cls=opt)
    return EmbCacheShardedEmbeddingBagCollection(ebc, ShardingEnv(1, 0, None), device, ebc.optimizer_spec(lr=lr), cache_rows=cache_rows)


def _train(m, steps, seed=0):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(40, generator=torch.Generator().manual_seed(9)).to(m.device)
    losses = []
    for _ in range(steps):
        kt = m(_batch(g))
        loss = (kt.values() * w).sum(dim=1).pow(2).mean()
        loss.backward()
        losses.append(float(loss))
    return losses


def test_small_cache_equals_big_cache():
    for opt in (torch.optim.Adagrad, torch.optim.Adam, torch.optim.SGD):
        small = _sharded(_tables(), [40, 64], opt)       # forces swaps every step (60 distinct ids, 2 features)
        big = _sharded(_tables(), [1001, 501], opt)
        la, lb = _train(small, 12), _train(big, 12)
        assert np.allclose(la, lb, rtol=1e-5, atol=1e-6), (opt, la, lb)
        assert small.stats["swap_out"] > 0 and big.stats["swap_out"] == 0
        keys = list(range(60))
        assert torch.allclose(small.host_rows("t1", keys), big.host_rows("t1", keys), atol=1e-6)


@pytest.mark.gpu
def test_small_cache_equals_big_cache_gpu():
    """Same scenario with the cache tensors, the gather / scatter kernels and the lookup on the GPU."""
    small = _sharded(_tables(), [40, 64], device="cuda")
    big = _sharded(_tables(), [1001, 501], device="cuda")
    la, lb = _train(small, 12), _train(big, 12)
    assert np.allclose(la, lb, rtol=1e-4, atol=1e-5), (la, lb)
    assert small.stats["swap_out"] > 0
    keys = list(range(60))
    assert torch.allclose(small.host_rows("t1", keys), big.host_rows("t1", keys), atol=1e-5)


def test_save_load_roundtrip(tmp_path):
    m = _sharded(_tables(), [40, 64])
    _train(m, 6)
    saver = Saver()
    out = saver.save(m, str(tmp_path))
    assert Saver.get_latest_load_path(str(tmp_path)) == out
    ref_rows = m.host_rows("t0", list(range(60))).clone()
    m2 = _sharded(_tables(), [40, 64])
    saver.load(m2, out)
    assert torch.allclose(m2.host_rows("t0", list(range(60))), ref_rows)
    # training continues identically after the reload
    assert np.allclose(_train(m, 4, seed=5), _train(m2, 4, seed=5), rtol=1e-5)


def test_admission_default_value_and_no_training():
    ae = AdmitAndEvictConfig(admit_threshold=3, not_admitted_default_value=0.5)
    m = _sharded(_tables(admit_and_evict_config=ae), [64, 64])
    kjt = KeyedJaggedTensor(["f0", "f1", "f2"], torch.tensor([7, 8, 8]), lengths=torch.tensor([1, 1, 1]))
    for step in range(4):
        out = m(kjt).values()
        out.sum().backward()
        if step < 2:                                     # seen fewer than 3 times: the default row, untrained
            assert torch.allclose(out[0, :8], torch.full((8,), 0.5))
    assert not torch.allclose(m(kjt).values()[0, :8], torch.full((8,), 0.5))


def test_pipeline_prefetch_matches_sync():
    class Model(torch.nn.Module):
        def __init__(self, emb):
            super().__init__()
            self.emb = emb
            self.w = torch.nn.Parameter(torch.randn(40, generator=torch.Generator().manual_seed(9)))

        def forward(self, batch):
            loss = (self.emb(batch.sparse_features).values() * self.w).sum(dim=1).pow(2).mean()
            return loss, loss.detach()

    class B:
        def __init__(self, k):
            self.sparse_features = k

        def to(self, device, non_blocking=False):
            return self

    def run(pipelined):
        torch.manual_seed(0)
        model = Model(_sharded(_tables(), [40, 64]))
        opt = torch.optim.SGD([model.w], lr=0.01)
        g = torch.Generator().manual_seed(3)
        data = iter([B(_batch(g)) for _ in range(8)])
        losses = []
        if pipelined:
            pipe = EmbCacheTrainPipelineSparseDist(model, opt, "cpu", "cpu", return_loss=True)
            for _ in range(8):
                losses.append(float(pipe.progress(data)[0]))
        else:
            for b in data:
                opt.zero_grad()
                loss, _ = model(b)
                loss.backward()
                opt.step()
                losses.append(float(loss))
        return losses

    assert np.allclose(run(True), run(False), rtol=1e-5)


def test_sequence_collection_small_cache_equals_big_cache():
    from recsdk_b200.embcache import EmbCacheEmbeddingCollection, EmbCacheEmbeddingConfig, EmbCacheShardedEmbeddingCollection

    def build(cache_rows):
        tabs = [EmbCacheEmbeddingConfig(num_embeddings=1000, embedding_dim=8, name="s0", feature_names=["f0"]),
                EmbCacheEmbeddingConfig(num_embeddings=500, embedding_dim=8, name="s1", feature_names=["f1", "f2"])]
        ec = EmbCacheEmbeddingCollection(tabs, 1, 6, [3, 3], device="cpu")
        return EmbCacheShardedEmbeddingCollection(ec, ShardingEnv(1, 0, None), "cpu", ec.optimizer_spec(lr=0.1), cache_rows=cache_rows)

    def train(m):
        g = torch.Generator().manual_seed(0)
        losses = []
        for _ in range(10):
            kjt = _batch(g)
            out = m(kjt)
            assert out["f1"].values().shape[0] == int(kjt["f1"].lengths().sum())
            loss = sum((jt.values() * (i + 1)).sum(dim=1).pow(2).mean() for i, jt in enumerate(out.values()))
            loss.backward()
            losses.append(float(loss.detach()))
        return losses

    a, b = train(build([40, 64])), train(build([1001, 501]))
    assert np.allclose(a, b, rtol=1e-5, atol=1e-6), (a, b)


def test_ec_local_unique_matches_plain_exchange(monkeypatch):
    """DO_EC_LOCAL_UNIQUE: the ids are de-duplicated per feature before the exchange; outputs, losses and the trained rows
    are the same, and fewer ids are swapped / looked up."""
    from recsdk_b200.embcache import EmbCacheEmbeddingCollection, EmbCacheEmbeddingConfig, EmbCacheShardedEmbeddingCollection
    from recsdk_b200.embcache.embedding import local_unique_kjt

    def build():
        tabs = [EmbCacheEmbeddingConfig(num_embeddings=50, embedding_dim=8, name="s0", feature_names=["f0"]),
                EmbCacheEmbeddingConfig(num_embeddings=30, embedding_dim=8, name="s1", feature_names=["f1", "f2"])]
        ec = EmbCacheEmbeddingCollection(tabs, 1, 6, [3, 3], device="cpu")
        return EmbCacheShardedEmbeddingCollection(ec, ShardingEnv(1, 0, None), "cpu", ec.optimizer_spec(lr=0.1), cache_rows=[64, 64])

    def batch(g):
        lengths = torch.randint(1, 5, (18,), generator=g)
        n = int(lengths.sum())
        values = torch.randint(0, 25, (n,), generator=g)               # small id range: many repeats inside a batch
        return KeyedJaggedTensor(["f0", "f1", "f2"], values, lengths=lengths, stride=6)

    def train(m):
        g = torch.Generator().manual_seed(5)
        losses, outs, looked_up = [], None, 0
        for _ in range(6):
            kjt = batch(g)
            out = m(kjt)
            looked_up += m._last_slots if hasattr(m, "_last_slots") else 0
            loss = sum((jt.values() * (i + 1)).sum(dim=1).pow(2).mean() for i, jt in enumerate(out.values()))
            loss.backward()
            losses.append(float(loss.detach()))
            outs = {k: v.values().detach().clone() for k, v in out.items()}
        return losses, outs

    monkeypatch.delenv("DO_EC_LOCAL_UNIQUE", raising=False)
    plain = build()
    assert not plain.do_local_unique
    a, oa = train(plain)
    monkeypatch.setenv("DO_EC_LOCAL_UNIQUE", "yes")
    uniq = build()
    assert uniq.do_local_unique
    b, ob = train(uniq)
    assert np.allclose(a, b, rtol=1e-5, atol=1e-6), (a, b)
    for k in oa:
        assert torch.allclose(oa[k], ob[k], rtol=1e-5, atol=1e-6)
    kjt = batch(torch.Generator().manual_seed(1))
    red, inv = local_unique_kjt(kjt)
    assert torch.equal(red.values()[inv], kjt.values()) and red.values().numel() < kjt.values().numel()
    assert red.length_per_key() == [int(torch.unique(kjt[k].values()).numel()) for k in ("f0", "f1", "f2")]


def test_restore_and_restore_async():
    import pytest
    import torch
    from recsdk_b200.embcache import restore, restore_async

    g = torch.Generator().manual_seed(0)
    per_table = [torch.randint(0, 20, (n,), generator=g) for n in (50, 0, 31)]
    uniq, inv, uoff, opt = [], [], [0], [0]
    for ids in per_table:
        u, i = torch.unique(ids, return_inverse=True)
        uniq.append(u + 1000 * len(uoff))                         # stands for the cache offsets of the unique keys
        inv.append(i)
        uoff.append(uoff[-1] + u.numel())
        opt.append(opt[-1] + ids.numel())
    unique_indices, unique_inverse = torch.cat(uniq), torch.cat(inv)
    unique_offset = torch.tensor(uoff, dtype=torch.int64)
    want = torch.cat([u[i] for u, i in zip(uniq, inv)])
    out = torch.full((unique_inverse.numel(),), -7, dtype=torch.int64)
    assert restore(unique_indices, unique_inverse, unique_offset, opt, out) is out
    assert torch.equal(out, want)
    out2 = torch.zeros_like(out)
    task = restore_async(unique_indices, unique_inverse, unique_offset, opt, out2)
    assert torch.equal(task.get(), want) and task.ready()
    bad = unique_inverse.clone()
    bad[3] = 10_000
    with pytest.raises(IndexError):
        restore(unique_indices, bad, unique_offset, opt, out)
    with pytest.raises(ValueError):
        restore(unique_indices, unique_inverse, unique_offset[:-1], opt, out)


def test_full_restore_drops_keys_that_are_not_in_the_checkpoint(tmp_path):
    """A non-incremental load resets the host table (and the filter) first: keys that the model met after the save do not
    survive the restore."""
    m = _sharded(_tables(), [40, 64])
    _train(m, 4, seed=0)
    saver = Saver()
    out = saver.save(m, str(tmp_path))
    m.embedding_to_host()
    sizes = [m.manager.host_size(t) for t in range(2)]
    g = torch.Generator().manual_seed(77)
    for _ in range(4):                                     # ids from another range: new keys in both tables
        lens = torch.randint(1, 4, (18,), generator=g)
        vals = torch.randint(200, 400, (int(lens.sum()),), generator=g)
        m(KeyedJaggedTensor(["f0", "f1", "f2"], vals, lengths=lens)).values().sum().backward()
    m.embedding_to_host()
    assert all(m.manager.host_size(t) > s for t, s in enumerate(sizes))
    saver.load(m, out)
    assert [m.manager.host_size(t) for t in range(2)] == sizes


def test_cache_sizing_follows_the_device_budget(monkeypatch):
    """Rows in the device cache: never below what two in-flight batches can touch, scaled up by the budget
    (``EMBCACHE_SIZE_ON_DEVICE_MEM``), never beyond the table; the declaration validates its tables."""
    from recsdk_b200.embcache.embedding_bag import MAX_CACHE_BYTES, _cache_budget_bytes, calculate_caches

    big = EmbCacheEmbeddingBagConfig(name="big", embedding_dim=16, num_embeddings=10_000_000, feature_names=["a"])
    small = EmbCacheEmbeddingBagConfig(name="small", embedding_dim=16, num_embeddings=100, feature_names=["b"])
    floor = [3 * 2 * 64 * 2, 1 * 2 * 64 * 2]                                 # hot * 2 * batch * world
    monkeypatch.setenv("EMBCACHE_SIZE_ON_DEVICE_MEM", "1")                    # a budget below the floor: the floor holds
    assert calculate_caches([big, small], 2, 64, [3, 1], 1) == [floor[0], 101]
    min_bytes = sum(r * 16 * 4 * 2 for r in floor)
    monkeypatch.setenv("EMBCACHE_SIZE_ON_DEVICE_MEM", str(4 * min_bytes))     # four times the floor: every table x 4
    assert calculate_caches([big, small], 2, 64, [3, 1], 1) == [4 * floor[0], 101]
    assert calculate_caches([big], 2, 64, [0], 0)[0] >= 2 * 64 * 2            # a zero hot size counts as one id per bag
    monkeypatch.setenv("EMBCACHE_SIZE_ON_DEVICE_MEM", "not a number")
    assert _cache_budget_bytes() == 16 << 30
    monkeypatch.setenv("EMBCACHE_SIZE_ON_DEVICE_MEM", str(1 << 40))
    assert _cache_budget_bytes() == MAX_CACHE_BYTES
    monkeypatch.delenv("EMBCACHE_SIZE_ON_DEVICE_MEM")
    decl = EmbCacheEmbeddingBagCollection([big, small], world_size=2, batch_size=64, multi_hot_sizes=[3, 1])
    assert decl.embedding_bag_configs() == [big, small] and decl.is_weighted() is False
    assert decl.cache_rows(1)[1] == 101 and decl.cache_rows(1)[0] <= 10_000_001
    assert decl.optimizer_spec(lr=0.1).lr == 0.1
    for bad in (dict(is_weighted=True), dict(multi_hot_sizes=[1]), dict(embedding_optimizer_cls=torch.optim.RMSprop)):
        kw = dict(world_size=1, batch_size=8, multi_hot_sizes=[1, 1])
        kw.update(bad)
        with pytest.raises(ValueError):
            EmbCacheEmbeddingBagCollection([big, small], **kw).optimizer_spec()
    with pytest.raises(ValueError, match="duplicate"):
        EmbCacheEmbeddingBagCollection([big, big], world_size=1, batch_size=8, multi_hot_sizes=[1, 1])
    odd = EmbCacheEmbeddingBagConfig(name="odd", embedding_dim=12, num_embeddings=10, feature_names=["c"])
    with pytest.raises(ValueError, match="multiple of 8"):
        EmbCacheEmbeddingBagCollection([odd], world_size=1, batch_size=8, multi_hot_sizes=[1])


def test_checkpoints_in_timestamp_directories(tmp_path):
    """The reference's flow: the caller names the checkpoint directory by a UTC timestamp and asks for the newest one
    (``torchrec_embcache/saver.py:55-69``); files land directly in that directory."""
    import os

    assert Saver.is_timestamp_format("20250131235959") and Saver.is_timestamp_format(Saver.timestamp_dir_name())
    for bad in ("full_0000000006", "2025013123595", "20251331000000", "", "2025-01-31"):
        assert not Saver.is_timestamp_format(bad)
    m = _sharded(_tables(), [40, 64])
    saver = Saver()
    _train(m, 3)
    first = saver.save(m, str(tmp_path / "20250101000000"))
    assert first == str(tmp_path / "20250101000000") and os.path.exists(os.path.join(first, "meta.ini"))
    _train(m, 3, seed=1)
    second = saver.save(m, str(tmp_path / "20250101000500"))
    assert Saver.get_latest_load_path(str(tmp_path)) == second
    # directories written without a step (the reference's meta.ini holds two lines only) are ordered by their names
    for d in (first, second):
        with open(os.path.join(d, "meta.ini")) as f:
            lines = [ln for ln in f if not ln.startswith(("step=", "tables="))]
        with open(os.path.join(d, "meta.ini"), "w") as f:
            f.writelines(lines)
    assert Saver.get_latest_load_path(str(tmp_path)) == second
    ref_rows = m.host_rows("t0", list(range(60))).clone()
    m2 = _sharded(_tables(), [40, 64])
    saver.load(m2, Saver.get_latest_load_path(str(tmp_path)))
    assert torch.allclose(m2.host_rows("t0", list(range(60))), ref_rows)
    assert Saver.get_latest_load_path(str(tmp_path / "nowhere")) is None


def test_reference_names_of_the_sharded_module():
    from recsdk_b200.embcache import CacheKernelView, EmbCacheHashTable
    from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig

    m = _sharded(_tables(), [40, 64], torch.optim.Adagrad)
    _train(m, 2)
    assert m.embcache_mgr is m.manager and [c.name for c in m.config_list] == ["t0", "t1"]
    kernels = m.get_batched_embedding_kernels()
    assert len(kernels) == 1 and isinstance(kernels[0][0], CacheKernelView)
    k = kernels[0][0]
    ws = k.split_embedding_weights()
    assert [tuple(w.shape) for w in ws] == [(40, 8), (64, 16)]
    assert k.weights_dev.numel() == 40 * 8 + 64 * 16
    mom = k.get_momentum()
    assert len(mom) == m.optim_num == 1 and mom[0].numel() == k.weights_dev.numel()
    m.record_host_emb_update_times()                       # a no-op where the native manager keeps no such counter

    cfg = EmbeddingBagConfig(num_embeddings=16, embedding_dim=4, name="h", feature_names=["f"])
    ht = EmbCacheHashTable(cfg, torch.device("cpu"))
    ids = torch.tensor([1 << 40, 7, 1 << 40, 99], dtype=torch.int64)
    out = ht(ids, torch.tensor([0, 2, 4]))
    w = ht.weight.detach()
    assert torch.allclose(out[0], w[0] + w[1]) and torch.allclose(out[1], w[0] + w[2])    # slots in order of first sight


def test_pipeline_save_in_the_middle_of_an_epoch(tmp_path):
    """fill_pipeline / wait_pipeline_compute_swapinfo / attach: a save taken while the next batch is staged holds the rows
    that the steps run so far have trained, and training goes on from the staged batch afterwards."""
    class Model(torch.nn.Module):
        def __init__(self, emb):
            super().__init__()
            self.emb = emb
            self.w = torch.nn.Parameter(torch.randn(40, generator=torch.Generator().manual_seed(9)))

        def forward(self, batch):
            loss = (self.emb(batch.sparse_features).values() * self.w).sum(dim=1).pow(2).mean()
            return loss, loss.detach()

    class B:
        def __init__(self, k):
            self.sparse_features = k

        def to(self, device, non_blocking=False):
            return self

    def run(save_at):
        model = Model(_sharded(_tables(), [40, 64]))
        opt = torch.optim.SGD([model.w], lr=0.01)
        g = torch.Generator().manual_seed(3)
        data = iter([B(_batch(g)) for _ in range(6)])
        pipe = EmbCacheTrainPipelineSparseDist(model, opt, "cpu", "cpu", return_loss=True)
        pipe.fill_pipeline(data)
        assert pipe._next is not None
        losses, snap = [], None
        for i in range(6):
            losses.append(float(pipe.progress(data)[0]))
            if i == save_at:
                pipe.wait_pipeline_compute_swapinfo()
                Saver().save(model, str(tmp_path / ("ck%d" % save_at)))
                snap = model.emb.host_rows("t1", list(range(60))).clone()
        pipe.attach()
        assert pipe._mods == [model.emb]
        return losses, snap, model

    la, snap, _ = run(2)
    lb, _, _ = run(-1)
    assert np.allclose(la, lb, rtol=1e-6)                  # the save does not disturb training
    fresh = Model(_sharded(_tables(), [40, 64]))
    Saver().load(fresh, Saver.get_latest_load_path(str(tmp_path / "ck2")) or str(tmp_path / "ck2"))
    assert torch.allclose(fresh.emb.host_rows("t1", list(range(60))), snap, atol=1e-6)

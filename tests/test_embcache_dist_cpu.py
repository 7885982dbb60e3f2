"""Multi-tier tables on two gloo ranks: same losses as one process on the global batch, and a checkpoint written by
two ranks loads into one (``key % world`` re-sharding)."""
import os
import tempfile

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from recsdk_b200.embcache import (EmbCacheEmbeddingBagCollection, EmbCacheEmbeddingBagConfig, EmbCacheShardedEmbeddingBagCollection, Saver)
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor

B, STEPS = 8, 6


def _tables():
    return [EmbCacheEmbeddingBagConfig(num_embeddings=1000, embedding_dim=8, name="t0", feature_names=["f0"]),
            EmbCacheEmbeddingBagConfig(num_embeddings=500, embedding_dim=16, name="t1", feature_names=["f1"])]


def _global_batches():
    g = torch.Generator().manual_seed(0)
    out = []
    for _ in range(STEPS):
        lens = torch.randint(1, 4, (2, B), generator=g)
        vals = [torch.randint(0, 50, (int(lens[f].sum()),), generator=g) for f in range(2)]
        out.append((lens, vals))
    return out


def _local(batch, rank, world):
    lens, vals = batch
    Bl = B // world
    lv, ll = [], []
    for f in range(2):
        off = torch.cat([torch.zeros(1, dtype=torch.long), lens[f].cumsum(0)])
        lv.append(vals[f][off[rank * Bl]:off[(rank + 1) * Bl]])
        ll.append(lens[f][rank * Bl:(rank + 1) * Bl])
    return KeyedJaggedTensor(["f0", "f1"], torch.cat(lv), lengths=torch.cat(ll), stride=Bl)


def _run(rank, world, pg, save_dir=None, cache=24):
    ebc = EmbCacheEmbeddingBagCollection(_tables(), world, B // world, [3, 3], device="cpu")
    m = EmbCacheShardedEmbeddingBagCollection(ebc, ShardingEnv(world, rank, pg), "cpu", ebc.optimizer_spec(lr=0.1), cache_rows=[cache, cache])
    w = torch.randn(24, generator=torch.Generator().manual_seed(5))
    losses = []
    for b in _global_batches():
        out = m(_local(b, rank, world)).values()
        loss = (out * w).sum(dim=1).pow(2).sum() / B
        loss.backward()
        losses.append(loss.detach())
    if save_dir is not None:
        Saver().save(m, save_dir)
    return m, torch.stack(losses)


def _worker(rank, world, init_file, save_dir, ret):
    dist.init_process_group("gloo", init_method="file://" + init_file, rank=rank, world_size=world)
    try:
        _, losses = _run(rank, world, dist.group.WORLD, save_dir)
        dist.all_reduce(losses)
        if rank == 0:
            ret["losses"] = losses.tolist()
    finally:
        dist.destroy_process_group()


def test_two_ranks_match_one_and_checkpoint_reshards():
    with tempfile.TemporaryDirectory() as d:
        ret = mp.Manager().dict()
        mp.spawn(_worker, args=(2, os.path.join(d, "init"), os.path.join(d, "ckpt"), ret), nprocs=2, join=True)
        ref_m, ref_losses = _run(0, 1, None, cache=64)
        assert np.allclose(ret["losses"], ref_losses.tolist(), rtol=1e-5, atol=1e-6), (ret["losses"], ref_losses.tolist())
        # the two-rank checkpoint, loaded into a single rank, holds the same rows as the single-process run
        path = Saver.get_latest_load_path(os.path.join(d, "ckpt"))
        assert path is not None and open(os.path.join(path, "meta.ini")).read().startswith("incremental=False\nsave_world_size=2")
        ebc = EmbCacheEmbeddingBagCollection(_tables(), 1, B, [3, 3], device="cpu")
        m = EmbCacheShardedEmbeddingBagCollection(ebc, ShardingEnv(1, 0, None), "cpu", ebc.optimizer_spec(lr=0.1), cache_rows=[64, 64])
        Saver().load(m, path)
        keys = list(range(50))
        assert torch.allclose(m.host_rows("t1", keys), ref_m.host_rows("t1", keys), atol=1e-6)


# ------------------------------------------------------------------------------------------ sequence collection, two ranks
def _seq_tables():
    from recsdk_b200.embcache import EmbCacheEmbeddingConfig

    return [EmbCacheEmbeddingConfig(num_embeddings=1000, embedding_dim=8, name="s0", feature_names=["f0"]),
            EmbCacheEmbeddingConfig(num_embeddings=500, embedding_dim=8, name="s1", feature_names=["f1"])]


def _seq_run(rank, world, pg):
    from recsdk_b200.embcache import EmbCacheEmbeddingCollection, EmbCacheShardedEmbeddingCollection

    ec = EmbCacheEmbeddingCollection(_seq_tables(), world, B // world, [3, 3], device="cpu")
    m = EmbCacheShardedEmbeddingCollection(ec, ShardingEnv(world, rank, pg), "cpu", ec.optimizer_spec(lr=0.1), cache_rows=[64, 64])
    losses = []
    for b in _global_batches():
        kjt = _local(b, rank, world)
        out = m(kjt)
        assert out["f0"].values().shape[0] == int(kjt["f0"].lengths().sum())
        loss = sum((jt.values() * (i + 1)).sum(dim=1).pow(2).sum() for i, jt in enumerate(out.values())) / B
        loss.backward()
        losses.append(loss.detach())
    return m, torch.stack(losses)


def _seq_worker(rank, world, init_file, unique, ret):
    if unique:
        os.environ["DO_EC_LOCAL_UNIQUE"] = "1"
    else:
        os.environ.pop("DO_EC_LOCAL_UNIQUE", None)
    dist.init_process_group("gloo", init_method="file://" + init_file, rank=rank, world_size=world)
    try:
        m, losses = _seq_run(rank, world, dist.group.WORLD)
        assert m.do_local_unique == unique
        dist.all_reduce(losses)
        if rank == 0:
            ret["losses"] = losses.tolist()
    finally:
        dist.destroy_process_group()


def test_sequence_collection_two_ranks_with_and_without_local_unique():
    """Rows come back to the rank and position that asked for them; de-duplicating each feature's ids before the exchange
    (DO_EC_LOCAL_UNIQUE) changes the traffic, not the result."""
    os.environ.pop("DO_EC_LOCAL_UNIQUE", None)
    _, ref = _seq_run(0, 1, None)
    for unique in (False, True):
        with tempfile.TemporaryDirectory() as d:
            ret = mp.Manager().dict()
            mp.spawn(_seq_worker, args=(2, os.path.join(d, "init"), unique, ret), nprocs=2, join=True)
            assert np.allclose(ret["losses"], ref.tolist(), rtol=1e-5, atol=1e-6), (unique, ret["losses"], ref.tolist())

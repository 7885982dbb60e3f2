"""Dynamic (hash-table) collections on two gloo ranks: keys are owned by ``key % world``; losses equal the
single-process run on the global batch, and a dump written by two ranks loads into one."""
import os
import tempfile

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from recsdk_b200.dynamic import (DynamicEmbeddingBagCollection, DynamicEmbInitializerArgs, DynamicEmbInitializerMode, DynamicEmbTableOptions,
                                 OptimizerType)
from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor

B, STEPS = 8, 5


def _batches():
    g = torch.Generator().manual_seed(0)
    out = []
    for _ in range(STEPS):
        lens = torch.randint(1, 4, (2, B), generator=g)
        vals = [torch.randint(0, 10 ** 9, (int(lens[f].sum()),), generator=g) % 97 * 1_000_003 for f in range(2)]
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
    return KeyedJaggedTensor(["fa", "fb"], torch.cat(lv), lengths=torch.cat(ll), stride=Bl)


def _run(rank, world, pg, dump_dir=None):
    cfgs = [EmbeddingBagConfig(num_embeddings=4096, embedding_dim=8, name="tab", feature_names=["fa", "fb"])]
    # DEBUG initialiser: a new key's row depends on the key only, so every sharding starts from the same table
    opts = {"tab": DynamicEmbTableOptions(initializer_args=DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.DEBUG))}
    m = DynamicEmbeddingBagCollection(cfgs, opts, ShardingEnv(world, rank, pg), torch.device("cpu"), optimizer_type=OptimizerType.SGD,
                                      learning_rate=1e-6, use_index_dedup=world > 1)
    w = torch.randn(16, generator=torch.Generator().manual_seed(3))
    losses = []
    for b in _batches():
        out = m(_local(b, rank, world)).values()
        loss = (out * w).sum(dim=1).pow(2).sum() / B * 1e-8
        loss.backward()
        losses.append(loss.detach())
    if dump_dir is not None:
        m.dump(dump_dir)
    return m, torch.stack(losses)


def _worker(rank, world, init_file, dump_dir, ret):
    dist.init_process_group("gloo", init_method="file://" + init_file, rank=rank, world_size=world)
    try:
        _, losses = _run(rank, world, dist.group.WORLD, dump_dir)
        dist.all_reduce(losses)
        if rank == 0:
            ret["losses"] = losses.tolist()
    finally:
        dist.destroy_process_group()


def test_two_ranks_match_one_and_dump_reshards():
    with tempfile.TemporaryDirectory() as d:
        ret = mp.Manager().dict()
        mp.spawn(_worker, args=(2, os.path.join(d, "init"), os.path.join(d, "dump"), ret), nprocs=2, join=True)
        ref, ref_losses = _run(0, 1, None)
        assert np.allclose(ret["losses"], ref_losses.tolist(), rtol=1e-5), (ret["losses"], ref_losses.tolist())
        cfgs = [EmbeddingBagConfig(num_embeddings=4096, embedding_dim=8, name="tab", feature_names=["fa", "fb"])]
        opts = {"tab": DynamicEmbTableOptions(initializer_args=DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.DEBUG))}
        m = DynamicEmbeddingBagCollection(cfgs, opts, ShardingEnv(1, 0, None), torch.device("cpu"), optimizer_type=OptimizerType.SGD)
        m.load(os.path.join(d, "dump"))
        assert m.table("tab").size() == ref.table("tab").size() > 0

"""Sharded checkpoints with sharding metadata: saved by a 2-rank layout, reloaded by 1 rank and by 3 ranks with another
plan (and the other way round), rows and optimizer state land on the right owner."""
import torch

from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig
from recsdk_b200.ops import embedding_ops as E
from recsdk_b200.parallel.checkpoint import load_sharded, load_sharded_from, save_sharded, sharded_state_dict
from recsdk_b200.parallel.collective_embeddingbag import CollectiveShardedEmbeddingBagCollection
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.parallel.embeddingbag import ParameterSharding

ROWS, DIMS = [101, 64, 37], [8, 16, 8]


def _module(world, rank, plan, seed):
    cfgs = [EmbeddingBagConfig(num_embeddings=r, embedding_dim=d, name="t%d" % i, feature_names=["f%d" % i])
            for i, (r, d) in enumerate(zip(ROWS, DIMS))]
    m = CollectiveShardedEmbeddingBagCollection(cfgs, plan, ShardingEnv.from_local(world, rank), torch.device("cpu"),
                                                E.OptimizerSpec(kind=E.OPT_ADAM))
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for ti, c in enumerate(cfgs):
            w = m.embedding_bags[c.name].weight
            rows = m.global_rows_of(ti)
            # value = function of (table, global row, column): any layout can be checked against it
            full = torch.arange(c.num_embeddings * c.embedding_dim, dtype=torch.float32).view(c.num_embeddings, -1) + 1000 * ti
            w.copy_(full[rows] if seed == 0 else torch.randn(w.shape, generator=g))
            for k, st in m.state[ti].items():
                st.copy_((full[rows] * (2 if k == "state1" else 3)) if seed == 0 else torch.randn(st.shape, generator=g))
    return m, cfgs


PLAN_A = {"t0": ParameterSharding("row_wise"), "t1": ParameterSharding("table_wise", ranks=[1]),
          "t2": ParameterSharding("row_wise", row_partition="block")}
PLAN_B = {"t0": ParameterSharding("row_wise", row_partition="block"), "t1": ParameterSharding("row_wise"),
          "t2": ParameterSharding("table_wise", ranks=[2])}


def _check(m, cfgs):
    for ti, c in enumerate(cfgs):
        rows = m.global_rows_of(ti)
        full = torch.arange(c.num_embeddings * c.embedding_dim, dtype=torch.float32).view(c.num_embeddings, -1) + 1000 * ti
        assert torch.equal(m.embedding_bags[c.name].weight.detach(), full[rows])
        assert torch.equal(m.state[ti]["state1"], full[rows] * 2) and torch.equal(m.state[ti]["state2"], full[rows] * 3)


def test_two_rank_checkpoint_reloads_on_one_and_three_ranks(tmp_path):
    d = str(tmp_path / "ck")
    for r in range(2):
        m, _ = _module(2, r, PLAN_A, seed=0)
        m._step = 7
        save_sharded(m, d)
    one, cfgs = _module(1, 0, {}, seed=5)
    got = load_sharded(one, d)
    assert got == {"t0": 101, "t1": 64, "t2": 37} and one._step == 7
    _check(one, cfgs)
    for r in range(3):
        m3, cfgs = _module(3, r, PLAN_B, seed=9)
        load_sharded(m3, d)
        _check(m3, cfgs)


def test_metadata_and_mismatch_errors():
    m, _ = _module(2, 1, PLAN_A, seed=0)
    sd = sharded_state_dict(m)
    md = sd["tables"]["t1"]["metadata"]
    assert md["sharding_type"] == "table_wise" and md["world_size"] == 2 and md["rank"] == 1 and md["local_rows"] == 64
    assert sd["tables"]["t0"]["metadata"]["row_partition"] == "mod"
    assert torch.equal(sd["tables"]["t0"]["global_row_ids"], torch.arange(1, 101, 2))
    one, _ = _module(1, 0, {}, seed=3)
    try:
        load_sharded_from(one, [sd])                       # rank 0's rows are missing
        raise AssertionError("expected a strict-load error")
    except ValueError as e:
        assert "in no shard" in str(e)

"""DLRM-small on CPU / gloo, world_size 2 (the plumbing config): 8 fp32 tables of 100,000 x 16, row-wise
sharded, sum pooling, bags of Uniform[1,5] Zipf(1.05) ids, 13 dense features, bottom MLP 13-64-16, dot
interaction, top MLP 52-64-1, BCE loss, batch 256 per rank, row-wise Adagrad (lr 0.01) on the tables,
SGD (lr 0.1) on the dense parameters, seed 0.  The sharded run must reproduce the single-process golden
run on the global batch (rtol = atol = 1e-4), like the reference's system test
(hybrid_torchrec/test/st/test_hybrid_hash_embeddingbag.py:74-262)."""
import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from recsdk_b200.models.dlrm import DLRM, DLRMTrain
from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig
from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection
from recsdk_b200.modules.hash_embeddingbag import HashEmbeddingBagCollection, HashEmbeddingBagConfig
from recsdk_b200.ops import embedding_ops as E
from recsdk_b200.optim import CombinedOptimizer, KeyedOptimizerWrapper
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.parallel.embeddingbag import ParameterSharding
from recsdk_b200.parallel.model_parallel import DistributedModelParallel
from recsdk_b200.parallel.planner import EmbeddingShardingPlanner, ParameterConstraints, ShardingPlan, Topology
from recsdk_b200.parallel.train_pipeline import TrainPipelineSparseDist
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor
from recsdk_b200.utils.data import Batch, RandomRecDataset

T, ROWS, D, BL, STEPS = 8, 100_000, 16, 256, 8


def _model(hashed, seed=0):
    torch.manual_seed(seed)
    cls, cfg_cls = (HashEmbeddingBagCollection, HashEmbeddingBagConfig) if hashed else (EmbeddingBagCollection, EmbeddingBagConfig)
    cfgs = [cfg_cls(num_embeddings=ROWS, embedding_dim=D, name="t%d" % i, feature_names=["f%d" % i],
                    init_fn=(lambda w: w.fill_(0.01)) if hashed else None) for i in range(T)]
    ebc = cls(cfgs, device=torch.device("cpu"))
    return cfgs, DLRMTrain(DLRM(ebc, 13, [64, D], [64, 1], dense_device=torch.device("cpu"), fused=False))


def _split(b: Batch, rank, world) -> Batch:
    B = b.dense_features.shape[0]
    Bl = B // world
    fd = b.sparse_features.to_dict()
    vals, lens = [], []
    for k in b.sparse_features.keys():
        jt = fd[k]
        off = jt.offsets()
        vals.append(jt.values()[off[rank * Bl]:off[(rank + 1) * Bl]])
        lens.append(jt.lengths()[rank * Bl:(rank + 1) * Bl])
    kjt = KeyedJaggedTensor(b.sparse_features.keys(), torch.cat(vals), lengths=torch.cat(lens), stride=Bl)
    return Batch(b.dense_features[rank * Bl:(rank + 1) * Bl], kjt, b.labels[rank * Bl:(rank + 1) * Bl])


def _train(rank, world, hashed, batches, plan=None, pg=None, hybrid=False):
    cfgs, model = _model(hashed)
    model.global_batch_size = BL * 2
    env = ShardingEnv(world, rank, pg)
    if plan is None:
        cons = {c.name: ParameterConstraints(sharding_types=["row_wise"], compute_kernels=["fused"]) for c in cfgs}
        plan = EmbeddingShardingPlanner(Topology(world_size=world, compute_device="cpu"), cons).plan(model)
    sharders = None
    if hybrid:
        from recsdk_b200.parallel import get_default_hybrid_sharders
        from recsdk_b200.optim import apply_optimizer_in_backward

        host_pg = dist.new_group(backend="gloo")
        sharders = get_default_hybrid_sharders(ShardingEnv.from_process_group(host_pg))
        # the sharder reads the sparse optimizer the way the reference flow declares it
        apply_optimizer_in_backward(torch.optim.Adagrad, model.model.sparse_arch.parameters(), {"lr": 0.01, "eps": 1e-8})
    dmp = DistributedModelParallel(model, env, torch.device("cpu"), plan, sharders=sharders,
                                   sparse_optimizer=E.OptimizerSpec(kind=E.OPT_ROWWISE_ADAGRAD, lr=0.01, eps=1e-8))
    dense = KeyedOptimizerWrapper(dmp.dense_named_parameters(), lambda p: torch.optim.SGD(p, lr=0.1))
    opt = CombinedOptimizer([dmp.fused_optimizer, dense])
    if hybrid:
        from recsdk_b200.parallel import HybridTrainPipelineSparseDist

        assert dmp.module.model.sparse_arch.input_pg is not None
        pipe = HybridTrainPipelineSparseDist(dmp, opt, torch.device("cpu"), return_loss=True, pipe_n_batch=3)
    else:
        pipe = TrainPipelineSparseDist(dmp, opt, torch.device("cpu"), return_loss=True)
    it = iter([_split(b, rank, world) if world > 1 else b for b in batches])
    losses, logits = [], None
    for _ in range(STEPS):
        loss, (_, lg, _) = pipe.progress(it)
        losses.append(loss.detach().clone())
        logits = lg
    return dmp, torch.stack(losses), logits


def _batches(hashed):
    keys = ["f%d" % i for i in range(T)]
    hs = [ROWS] * T if not hashed else [1 << 40] * T
    data = RandomRecDataset(keys, hs, BL * 2, alpha=1.05, one_hot=False, min_len=1, max_len=5, pos_rate=0.25, seed=0)
    return [data.make_batch() for _ in range(STEPS)]


def _worker(rank, world, hashed, mixed, init_file, ret, hybrid=False):
    dist.init_process_group("gloo", init_method="file://" + init_file, rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        batches = _batches(hashed)
        plan = None
        if mixed:
            kinds = ["row_wise", "table_wise", "data_parallel", "row_wise"]
            tabs = {}
            for i in range(T):
                k = kinds[i % 4]
                tabs["t%d" % i] = ParameterSharding(k, ranks=[i % world] if k == "table_wise" else None,
                                                    row_partition="block" if i == 3 else "mod")
            plan = ShardingPlan({"model.sparse_arch": tabs})
        dmp, losses, logits = _train(rank, world, hashed, batches, plan, dist.group.WORLD, hybrid)
        dist.all_reduce(losses)
        _, ref_losses, ref_logits = _train(0, 1, hashed, batches)
        ok = torch.allclose(losses, ref_losses, rtol=1e-4, atol=1e-4)
        ok = ok and torch.allclose(logits, ref_logits[rank * BL:(rank + 1) * BL], rtol=1e-4, atol=1e-4)
        if rank == 0:
            ret["losses"] = losses.tolist()
            ret["ref"] = ref_losses.tolist()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("hashed,mixed", [(False, False), (False, True), (True, False)])
def test_dlrm_small_gloo_world2_matches_golden(hashed, mixed):
    with tempfile.TemporaryDirectory() as d:
        ret = mp.Manager().dict()
        mp.spawn(_worker, args=(2, hashed, mixed, os.path.join(d, "init"), ret), nprocs=2, join=True)
        assert ret.get(0) and ret.get(1), (ret.get("losses"), ret.get("ref"))
        assert ret["losses"][-1] < ret["losses"][0]


def test_hybrid_host_input_dist_pipeline_matches_golden():
    """Hash tables, id exchange on a separate gloo group from a worker thread three batches ahead."""
    with tempfile.TemporaryDirectory() as d:
        ret = mp.Manager().dict()
        mp.spawn(_worker, args=(2, True, False, os.path.join(d, "init"), ret, True), nprocs=2, join=True)
        assert ret.get(0) and ret.get(1), (ret.get("losses"), ret.get("ref"))

"""Quick start: a DLRM over hash embedding tables trained with the hybrid flow (id exchange and id mapping on the host,
several batches ahead of the device), written the way the reference's quick start walks through it
(``docs/en/torch/torch_rec_v1/03_quick_start/quick_start.md:120-318``):

    process group (device backend) -> a gloo group for the host side -> ShardingEnv.from_process_group(host_pg)
    -> HashEmbeddingBagCollection -> apply_optimizer_in_backward -> EmbeddingShardingPlanner(...).collective_plan
    -> DistributedModelParallel(model, device=..., plan=..., sharders=get_default_hybrid_sharders(host_env))
    -> CombinedOptimizer([dmp.fused_optimizer, KeyedOptimizerWrapper(dense parameters)])
    -> HybridTrainPipelineSparseDist(...).progress(iterator)

Run on CPU (gloo) or on GPUs (nccl), one process per device:

    python examples/quick_start_hybrid.py --steps 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/quick_start_hybrid.py
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from recsdk_b200.models.dlrm import DLRM, DLRMTrain  # noqa: E402
from recsdk_b200.modules.hash_embeddingbag import HashEmbeddingBagCollection, HashEmbeddingBagConfig  # noqa: E402
from recsdk_b200.ops import embedding_ops as E  # noqa: E402
from recsdk_b200.optim import CombinedOptimizer, KeyedOptimizerWrapper, apply_optimizer_in_backward  # noqa: E402
from recsdk_b200.parallel import HybridTrainPipelineSparseDist, get_default_hybrid_sharders  # noqa: E402
from recsdk_b200.parallel.comm import ShardingEnv  # noqa: E402
from recsdk_b200.parallel.model_parallel import DistributedModelParallel  # noqa: E402
from recsdk_b200.parallel.planner import EmbeddingShardingPlanner, ParameterConstraints, Topology  # noqa: E402
from recsdk_b200.utils.data import RandomRecDataset  # noqa: E402


def main(argv=None) -> float:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--tables", type=int, default=4)
    ap.add_argument("--dim", type=int, default=16)
    ap.add_argument("--local-batch", type=int, default=128)
    ap.add_argument("--pipe-n-batch", type=int, default=2)
    args = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    host_env = ShardingEnv(1, 0, None)
    pg = None
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo")
        pg = dist.group.WORLD
        host_env = ShardingEnv.from_process_group(dist.new_group(backend="gloo"))      # the host-side exchange group
    env = ShardingEnv(world, rank, pg)

    keys = ["f%d" % i for i in range(args.tables)]
    tables = [HashEmbeddingBagConfig(num_embeddings=50_000, embedding_dim=args.dim, name="t%d" % i, feature_names=[keys[i]])
              for i in range(args.tables)]
    ebc = HashEmbeddingBagCollection(tables, device=torch.device("cpu"))
    apply_optimizer_in_backward(torch.optim.Adagrad, ebc.parameters(), {"lr": 0.02, "eps": 1e-8})
    model = DLRMTrain(DLRM(ebc, 13, [64, args.dim], [64, 1], dense_device=device, fused=False))
    model.global_batch_size = args.local_batch * world

    sharders = get_default_hybrid_sharders(host_env)
    constraints = {t.name: ParameterConstraints(sharding_types=["row_wise"], compute_kernels=["fused"]) for t in tables}
    planner = EmbeddingShardingPlanner(Topology(world_size=world, compute_device=device.type), constraints)
    plan = planner.collective_plan(model, sharders, pg) if world > 1 else planner.plan(model, sharders)
    dmp = DistributedModelParallel(model, env=env, device=device, plan=plan, sharders=sharders,
                                   sparse_optimizer=E.OptimizerSpec(kind=E.OPT_ROWWISE_ADAGRAD, lr=0.02, eps=1e-8))
    dense = KeyedOptimizerWrapper(dmp.dense_named_parameters(), lambda p: torch.optim.Adagrad(p, lr=0.05))
    optimizer = CombinedOptimizer([dmp.fused_optimizer, dense])
    pipeline = HybridTrainPipelineSparseDist(dmp, optimizer, device, return_loss=True, pipe_n_batch=args.pipe_n_batch)

    data = RandomRecDataset(keys, [1 << 40] * args.tables, args.local_batch, alpha=1.05, one_hot=False, min_len=1, max_len=4,
                            pos_rate=0.25, seed=100 + rank)
    batches = iter([data.make_batch() for _ in range(args.steps)])
    first = last = None
    for step in range(args.steps):
        loss, _ = pipeline.progress(batches)
        last = float(loss)
        first = last if first is None else first
        if rank == 0 and step % 5 == 0:
            print("step %3d  loss %.4f  (batches in flight: %d)" % (step, last, pipeline.in_flight()))
    if rank == 0:
        print("loss %.4f -> %.4f" % (first, last))
    if world > 1:
        dist.destroy_process_group()
    return last


if __name__ == "__main__":
    main()

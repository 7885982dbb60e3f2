"""Multi-GPU worker (one process per GPU, launched by ``python -m torch.distributed.run``).

Trains a small sharded DLRM (table-wise + row-wise + data-parallel tables) for a few steps on
``world`` GPUs and checks it against the same model trained in this process on one GPU with the
full global batch: summed per-rank losses, final embedding tables and dense weights must agree.
Every rank leaves only between steps; device-side waits are bounded (2 s).
"""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from recsdk_b200.models.dlrm import DLRM, DLRMTrain  # noqa: E402
from recsdk_b200.modules.embedding_configs import DataType, EmbeddingBagConfig  # noqa: E402
from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection  # noqa: E402
from recsdk_b200.ops import _lib  # noqa: E402
from recsdk_b200.ops import embedding_ops as E  # noqa: E402
from recsdk_b200.optim import CombinedOptimizer, FusedDenseOptimizer  # noqa: E402
from recsdk_b200.parallel.comm import PeerGroup, ShardingEnv  # noqa: E402
from recsdk_b200.parallel.embeddingbag import ParameterSharding  # noqa: E402
from recsdk_b200.parallel.model_parallel import DistributedModelParallel  # noqa: E402
from recsdk_b200.parallel.planner import ShardingPlan  # noqa: E402
from recsdk_b200.parallel.train_pipeline import TrainPipelineSparseDist  # noqa: E402
from recsdk_b200.utils.data import Batch, RandomRecDataset  # noqa: E402
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor  # noqa: E402

ROWS = [5000, 300, 12345, 64, 2048, 999]
D = 64
GB = 1024
STEPS = 6


def build(env, dev, peer, plan, cuda_graph):
    cfgs = [EmbeddingBagConfig(num_embeddings=r, embedding_dim=D, name="t%d" % i, feature_names=["f%d" % i],
                               data_type=DataType.FP32) for i, r in enumerate(ROWS)]
    torch.manual_seed(7)
    ebc = EmbeddingBagCollection(cfgs, device=torch.device("meta"))
    model = DLRMTrain(DLRM(ebc, 13, [128, D], [256, 128, 1], dense_device=dev), global_batch_size=GB)
    dmp = DistributedModelParallel(model, env, dev, plan, peer=peer,
                                   sparse_optimizer=E.OptimizerSpec(kind=E.OPT_ROWWISE_ADAGRAD, lr=0.05, eps=1e-8),
                                   max_local_batch=GB // env.world_size, one_hot=True, init_seed=11)
    opt = CombinedOptimizer([dmp.fused_optimizer, FusedDenseOptimizer(dmp.module, "adam", lr=1e-3)])
    pipe = TrainPipelineSparseDist(dmp, opt, dev, return_loss=True, cuda_graph=cuda_graph)
    return cfgs, dmp, pipe


def slice_batch(b: Batch, rank: int, world: int) -> Batch:
    B = b.dense_features.shape[0]
    Bl = B // world
    T = len(b.sparse_features.keys())
    vals = b.sparse_features.values().view(T, B)[:, rank * Bl:(rank + 1) * Bl].contiguous().view(-1)
    kjt = KeyedJaggedTensor(b.sparse_features.keys(), vals, lengths=torch.ones(T * Bl, dtype=torch.int64), stride=Bl)
    kjt.one_hot = True
    return Batch(b.dense_features[rank * Bl:(rank + 1) * Bl].contiguous(), kjt,
                 b.labels[rank * Bl:(rank + 1) * Bl].contiguous())


def main() -> int:
    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    cuda_graph = "--graph" in sys.argv
    ok = True
    try:
        data = RandomRecDataset(["f%d" % i for i in range(len(ROWS))], ROWS, GB, alpha=1.05, seed=3)
        batches = [data.make_batch() for _ in range(STEPS)]
        # --- single-GPU oracle on the full batch (every rank computes it; cheap)
        _, ref_dmp, ref_pipe = build(ShardingEnv(1, 0), dev, None, ShardingPlan({}), False)
        ref_losses = []
        it = iter(batches)
        for _ in range(STEPS):
            loss, _ = ref_pipe.progress(it)
            ref_losses.append(loss.item())
        # --- sharded run
        env = ShardingEnv(world, rank, dist.group.WORLD)
        peer = PeerGroup(dist.group.WORLD, dev)
        plan = ShardingPlan({"model.sparse_arch": {
            "t0": ParameterSharding("row_wise"), "t1": ParameterSharding("table_wise", ranks=[world - 1]),
            "t2": ParameterSharding("row_wise", row_partition="block"), "t3": ParameterSharding("data_parallel"),
            "t4": ParameterSharding("table_wise", ranks=[0]), "t5": ParameterSharding("row_wise")}})
        cfgs, dmp, pipe = build(env, dev, peer, plan, cuda_graph)
        it = iter([slice_batch(b, rank, world) for b in batches])
        losses = []
        for _ in range(STEPS):
            loss, _ = pipe.progress(it)
            t = loss.detach().clone()
            dist.all_reduce(t)
            losses.append(t.item())
        torch.cuda.synchronize()
        _lib.check_status(dev)
        for a, b in zip(losses, ref_losses):
            if abs(a - b) > 2e-3 * max(1.0, abs(b)):
                ok = False
        if rank == 0:
            print("losses sharded:", ["%.5f" % x for x in losses])
            print("losses  single:", ["%.5f" % x for x in ref_losses])
        ref_ebc = ref_dmp.sharded_modules[0]
        sh_ebc = dmp.sharded_modules[0]
        for c in cfgs:
            full = sh_ebc.full_table(c.name)
            want = ref_ebc.full_table(c.name)
            err = (full - want).abs().max().item()
            if rank == 0:
                print("table %s max |diff| %.3e" % (c.name, err))
            if err > 2e-3:
                ok = False
        wa = dmp.module.model.over_arch.flat_param.detach()
        wb = ref_dmp.module.model.over_arch.flat_param.detach()
        derr = (wa - wb).abs().max().item()
        if rank == 0:
            print("dense max |diff| %.3e  multicast=%s" % (derr, bool(peer.pads.multicast_ptr)))
        if derr > 2e-3:
            ok = False
    except Exception as e:  # noqa: BLE001
        import traceback

        traceback.print_exc()
        ok = False
    flag = torch.tensor([1 if ok else 0], device=dev)
    try:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(flag.item())
    except Exception:  # noqa: BLE001
        ok = False
    if rank == 0:
        print("MULTI_GPU_RESULT", "PASS" if ok else "FAIL")
    try:
        dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        pass
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())

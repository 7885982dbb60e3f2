"""Multi-GPU correctness self-check: the fused push-exchange backend against the ``torch.distributed`` all-to-all
backend on the same small tables, same weights, same batch.

``run_selfcheck(env, peer, device)`` builds three tables (row-wise, table-wise and block row-wise), runs one fixed one-hot
batch forward and backward (plain SGD, so the updated rows are a direct function of the gradients) through both
backends and returns ``{"ok", "max_abs_diff_pooled", "max_abs_diff_rows", "world"}``.  It is cheap enough to append to a
benchmark run, so that a multi-GPU throughput number always travels with evidence that the kernels that produced it
compute the same thing as the library collectives they replace.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..modules.embedding_configs import DataType, EmbeddingBagConfig
from ..ops import _lib
from ..ops import embedding_ops as E
from ..sparse.jagged_tensor import KeyedJaggedTensor
from .collective_embeddingbag import CollectiveShardedEmbeddingBagCollection
from .comm import PeerGroup, ShardingEnv
from .embeddingbag import ParameterSharding, ShardedEmbeddingBagCollection


def run_selfcheck(env: ShardingEnv, peer: Optional[PeerGroup], device: torch.device, local_batch: int = 512,
                  dim: int = 64, tol: float = 1e-5) -> Dict[str, object]:
    world, rank = env.world_size, env.rank
    rows = [20011, 977, 6007]
    cfgs = [EmbeddingBagConfig(num_embeddings=r, embedding_dim=dim, name="sc%d" % i, feature_names=["sf%d" % i],
                               data_type=DataType.FP32) for i, r in enumerate(rows)]
    plan = {"sc0": ParameterSharding("row_wise"), "sc1": ParameterSharding("table_wise", ranks=[world - 1]),
            "sc2": ParameterSharding("row_wise", row_partition="block")}
    spec = E.OptimizerSpec(kind=E.OPT_SGD, lr=0.5)
    fused = ShardedEmbeddingBagCollection(cfgs, plan, env, device, spec, peer=peer, out_dtype=torch.float32,
                                          max_local_batch=local_batch, one_hot=True)
    fused.reset_parameters(seed=17)
    coll = CollectiveShardedEmbeddingBagCollection(cfgs, plan, env, device, E.OptimizerSpec(kind=E.OPT_SGD, lr=0.5),
                                                   out_dtype=torch.float32)
    with torch.no_grad():                                   # same starting rows: seeded values are a function of the global row
        for ti, c in enumerate(cfgs):
            w = coll.embedding_bags[c.name].weight
            if w.numel():
                src = fused.embedding_bags[c.name].weight
                if src.shape == w.shape:
                    w.copy_(src)
                else:                                       # layouts differ only if the two backends shard differently
                    raise RuntimeError("self-check: shard shapes differ for %s" % c.name)
    g = torch.Generator().manual_seed(4242 + rank)
    ids = torch.cat([torch.randint(0, r, (local_batch,), generator=g) for r in rows]).to(device)
    ones = torch.ones(len(rows) * local_batch, dtype=torch.int64, device=device)
    dout = torch.randn(local_batch, dim * len(rows), generator=g).to(device)
    kjt = KeyedJaggedTensor(["sf%d" % i for i in range(len(rows))], ids, lengths=ones, stride=local_batch)
    kjt.one_hot = True
    of = fused(kjt).values()
    kjt2 = KeyedJaggedTensor(["sf%d" % i for i in range(len(rows))], ids.clone(), lengths=ones.clone(), stride=local_batch)
    oc = coll(kjt2).values()
    d_pooled = float((of.detach().float() - oc.detach().float()).abs().max())
    of.backward(dout)
    oc.backward(dout)
    if hasattr(fused, "join_exchange"):
        fused.join_exchange()
    torch.cuda.synchronize(device)
    _lib.check_status(device)
    d_rows = 0.0
    for c in cfgs:
        a, b = fused.embedding_bags[c.name].weight, coll.embedding_bags[c.name].weight
        if a.numel():
            d_rows = max(d_rows, float((a.float() - b.float()).abs().max()))
    t = torch.tensor([d_pooled, d_rows], dtype=torch.float64, device=device)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=env.process_group)
    d_pooled, d_rows = float(t[0]), float(t[1])
    return {"ok": bool(d_pooled <= tol and d_rows <= tol), "max_abs_diff_pooled": d_pooled, "max_abs_diff_rows": d_rows,
            "world": world, "tables": len(rows), "local_batch": local_batch,
            "what": "push-exchange backend vs torch.distributed all-to-all backend: pooled outputs and SGD-updated rows"}

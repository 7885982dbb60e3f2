"""Dynamic (hash-table) embeddings: stock collections become dynamic through the sharding plan, rows are trained inside
backward, and the table is dumped, reloaded and dumped incrementally by score
(user flow of the reference's ``dynamic_emb`` package: planner / sharders ``distributed/planner/planners.py:80-222``,
``distributed/embeddingbag.py:80-119``; dump / load ``distributed/dump_load.py:92-272``; ``incremental_dump.py:103-404``).

    python examples/dynamic_embedding.py
"""
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from recsdk_b200.dynamic import (DynamicEmbDump, DynamicEmbeddingBagCollectionSharder, DynamicEmbeddingCollectionSharder,  # noqa: E402
                                 DynamicEmbeddingShardingPlanner, DynamicEmbLoad, DynamicEmbParameterConstraints,
                                 DynamicEmbTableOptions, incremental_dump, set_score)
from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig  # noqa: E402
from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection  # noqa: E402
from recsdk_b200.parallel.model_parallel import DistributedModelParallel  # noqa: E402
from recsdk_b200.parallel.planner import Topology  # noqa: E402
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor  # noqa: E402


class Model(torch.nn.Module):
    def __init__(self, tables, device):
        super().__init__()
        self.ebc = EmbeddingBagCollection(tables, device=torch.device("meta"))       # rows live in the hash tables only
        self.top = torch.nn.Linear(sum(t.embedding_dim for t in tables), 1).to(device)

    def forward(self, kjt):
        return self.top(self.ebc(kjt).values().float()).pow(2).mean()


def build(tables, device):
    cons = {t.name: DynamicEmbParameterConstraints(use_dynamicemb=True, dynamicemb_options=DynamicEmbTableOptions())
            for t in tables}
    planner = DynamicEmbeddingShardingPlanner(tables, cons, Topology(world_size=1, compute_device=device.type))
    model = Model(tables, device)
    sharders = [DynamicEmbeddingCollectionSharder(), DynamicEmbeddingBagCollectionSharder({"learning_rate": 0.1})]
    return DistributedModelParallel(model, device=device, plan=planner.plan(model, sharders), sharders=sharders, backend="collective")


def main() -> float:
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    tables = [EmbeddingBagConfig(num_embeddings=1 << 20, embedding_dim=16, name="user", feature_names=["uid"]),
              EmbeddingBagConfig(num_embeddings=1 << 20, embedding_dim=16, name="item", feature_names=["iid"])]
    dmp = build(tables, device)
    g = torch.Generator().manual_seed(0)
    dense_opt = torch.optim.SGD(dmp.module.top.parameters(), lr=0.05)
    loss = None
    for step in range(10):
        ids = torch.randint(0, 1 << 40, (64,), generator=g) % 997                    # raw 64-bit ids, no vocabulary needed
        kjt = KeyedJaggedTensor(["uid", "iid"], ids, lengths=torch.ones(64, dtype=torch.int64), stride=32).to(device)
        set_score(dmp, step + 1)                                                       # scores drive eviction and incremental dumps
        dense_opt.zero_grad()
        loss = dmp(kjt)
        loss.backward()                                                                # the table rows are updated in here
        dense_opt.step()
    with tempfile.TemporaryDirectory() as d:
        DynamicEmbDump(os.path.join(d, "ckpt"), dmp, optim=True)
        fresh = build(tables, device)
        DynamicEmbLoad(os.path.join(d, "ckpt"), fresh, optim=True)
        fresh.module.top.load_state_dict(dmp.module.top.state_dict())
        again = float(fresh(kjt).detach())
        changed, _scores = incremental_dump(dmp, 10)                                   # rows touched at score >= 10
    n_changed = sum(int(k.numel()) for coll in changed.values() for (k, _v) in coll.values())
    print("final loss %.5f, reloaded model gives %.5f, %d rows in the incremental dump" % (float(dmp(kjt).detach()), again, n_changed))
    return float(loss.detach())


if __name__ == "__main__":
    main()

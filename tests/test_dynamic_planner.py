"""Plan-driven conversion of stock collections into dynamic (hash-table) ones through DistributedModelParallel."""
import torch

from recsdk_b200.dynamic import (DynamicEmbeddingBagCollection, DynamicEmbeddingBagCollectionSharder, DynamicEmbeddingCollectionSharder,
                                 DynamicEmbeddingShardingPlanner, DynamicEmbParameterConstraints, DynamicEmbParameterSharding,
                                 DynamicEmbTableOptions)
from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig
from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection
from recsdk_b200.parallel.model_parallel import DistributedModelParallel
from recsdk_b200.parallel.planner import Topology
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor


def test_planner_rewrites_and_dmp_shards():
    tables = [EmbeddingBagConfig(num_embeddings=1000, embedding_dim=16, name="a", feature_names=["fa"]),
              EmbeddingBagConfig(num_embeddings=3000, embedding_dim=16, name="b", feature_names=["fb"])]

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ebc = EmbeddingBagCollection(tables, device=torch.device("meta"))
            self.top = torch.nn.Linear(32, 1)

        def forward(self, kjt):
            return self.top(self.ebc(kjt).values().float()).sum()

    cons = {t.name: DynamicEmbParameterConstraints(use_dynamicemb=True, dynamicemb_options=DynamicEmbTableOptions()) for t in tables}
    planner = DynamicEmbeddingShardingPlanner(tables, cons, Topology(world_size=4, compute_device="cpu"))
    m = M()
    plan = planner.collective_plan(m, [DynamicEmbeddingBagCollectionSharder()])
    e = plan.get_module_plan("ebc")
    assert isinstance(e["a"], DynamicEmbParameterSharding) and e["a"].aligned_rows_per_rank == 256 and e["b"].aligned_rows_per_rank == 1024
    assert e["a"].dist_type == "roundrobin" and planner.reserved_hbm_per_rank == (256 + 1024) * (16 + 4) * 4
    # world 1 on CPU: the sharder swaps the stock module for the dynamic one
    planner1 = DynamicEmbeddingShardingPlanner(tables, cons, Topology(world_size=1, compute_device="cpu"))
    dmp = DistributedModelParallel(m, device=torch.device("cpu"), plan=planner1.plan(m),
                                   sharders=[DynamicEmbeddingCollectionSharder(), DynamicEmbeddingBagCollectionSharder({"learning_rate": 0.1})],
                                   backend="collective")
    assert isinstance(dmp.module.ebc, DynamicEmbeddingBagCollection)
    kjt = KeyedJaggedTensor(["fa", "fb"], torch.tensor([5, 10 ** 12, 7, 7, 9]), lengths=torch.tensor([1, 1, 2, 1]))
    first = float(dmp(kjt))
    for _ in range(5):
        loss = dmp(kjt)
        loss.backward()
    assert float(dmp(kjt)) != first                      # rows are trained inside backward

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


def test_module_finders_and_fused_params():
    """``find_sharded_modules`` / ``get_dynamic_emb_module`` (``dump_load.py:39-89`` of the reference) and the extra fields a
    dynamic plan entry hands to the compute kernel."""
    import pytest
    import torch

    from recsdk_b200.dynamic import (BatchedDynamicEmbeddingTablesV2, DynamicEmbeddingCollection, DynamicEmbTableOptions, OptimizerType,
                                     check_emb_collection_modules, find_sharded_modules, get_dynamic_emb_module)
    from recsdk_b200.dynamic.planner import DynamicEmbParameterSharding
    from recsdk_b200.modules import EmbeddingConfig
    from recsdk_b200.parallel import ShardingEnv

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            cfg = [EmbeddingConfig(num_embeddings=1000, embedding_dim=8, name="t", feature_names=["f"])]
            self.tower = torch.nn.Module()
            self.tower.emb = DynamicEmbeddingCollection(cfg, {"t": DynamicEmbTableOptions()}, ShardingEnv(1, 0), torch.device("cpu"),
                                                        optimizer_type=OptimizerType.SGD)
            self.dense = torch.nn.Linear(8, 1)

    net = Net()
    found = find_sharded_modules(net)
    assert [(p, n) for p, n, _m in found] == [("model.tower.emb", "emb")] and found[0][2] is net.tower.emb
    mods = get_dynamic_emb_module(net)
    assert len(mods) == 1 and isinstance(mods[0], BatchedDynamicEmbeddingTablesV2)
    again = []
    check_emb_collection_modules(net, again)
    assert again == mods and mods[0].table_names == ["t"] and len(mods[0].tables) == 1
    assert mods[0].optimizer.get_opt_args()["opt_type"] == "sgd"
    for fn in (find_sharded_modules, get_dynamic_emb_module):
        with pytest.raises(ValueError):
            fn("not a module")
    extra = DynamicEmbParameterSharding("row_wise", aligned_rows_per_rank=128).get_additional_fused_params()
    assert sorted(extra) == ["aligned_rows_per_rank", "customized_compute_kernel", "dist_type", "dynamicemb_options", "hbm_bytes_per_rank"]
    assert extra["dist_type"] == "roundrobin" and extra["customized_compute_kernel"] == "DynamicEmb"

"""The static-table sharding planner: size thresholds, constraints, the even snake deal of table-wise tables, the budget
check and the plan container."""
import pytest
import torch

from recsdk_b200.modules.embedding_configs import DataType, EmbeddingBagConfig
from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection
from recsdk_b200.parallel.planner import EmbeddingShardingPlanner, ParameterConstraints, ShardingPlan, Topology


def _model(rows, dim=16, dtype=DataType.FP32):
    cfgs = [EmbeddingBagConfig(num_embeddings=r, embedding_dim=dim, name="t%d" % i, data_type=dtype) for i, r in enumerate(rows)]

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.dense = torch.nn.Linear(4, 4)
            self.sparse = EmbeddingBagCollection(cfgs, device=torch.device("meta"))

    return M()


def test_one_rank_keeps_everything_local():
    plan = EmbeddingShardingPlanner(Topology(world_size=1)).plan(_model([10, 1000]))
    assert {k: v.sharding_type for k, v in plan.get_module_plan("sparse").items()} == {"t0": "data_parallel", "t1": "data_parallel"}


def test_thresholds_and_even_table_wise_deal():
    # one huge table, eight medium ones, one tiny: row-wise / table-wise in snake order / data-parallel
    rows = [4_000_000] + [50_000 - 1000 * i for i in range(8)] + [8]
    planner = EmbeddingShardingPlanner(Topology(world_size=4), row_wise_threshold_bytes=64 << 20, dp_threshold_bytes=1024)
    tabs = planner.plan(_model(rows)).get_module_plan("sparse")
    assert tabs["t0"].sharding_type == "row_wise" and tabs["t0"].row_partition == "mod"
    assert tabs["t9"].sharding_type == "data_parallel"
    owners = [tabs["t%d" % i].ranks[0] for i in range(1, 9)]
    assert all(tabs["t%d" % i].sharding_type == "table_wise" for i in range(1, 9))
    assert owners == [0, 1, 2, 3, 3, 2, 1, 0]                              # largest first, back and forth
    assert sorted(owners.count(r) for r in range(4)) == [2, 2, 2, 2]


def test_left_over_table_wise_tables_become_row_wise():
    rows = [30_000, 20_000, 10_000, 9_000, 8_000, 7_000]                     # six table-wise candidates on four ranks
    tabs = EmbeddingShardingPlanner(Topology(world_size=4), row_wise_threshold_bytes=1 << 40).plan(_model(rows)).get_module_plan("sparse")
    kinds = [tabs["t%d" % i].sharding_type for i in range(6)]
    assert kinds == ["row_wise", "row_wise", "table_wise", "table_wise", "table_wise", "table_wise"]   # the two largest are spread
    assert sorted(tabs["t%d" % i].ranks[0] for i in range(2, 6)) == [0, 1, 2, 3]


def test_default_threshold_spreads_tables_above_half_a_fair_share():
    rows = [1_000_000, 1000, 1000, 1000]
    tabs = EmbeddingShardingPlanner(Topology(world_size=2)).plan(_model(rows)).get_module_plan("sparse")
    assert tabs["t0"].sharding_type == "row_wise"
    assert [tabs["t%d" % i].sharding_type for i in (1, 2, 3)].count("table_wise") == 2   # three candidates, two ranks: one is spread


def test_constraints_win_and_unknown_types_are_refused():
    cons = {"t0": ParameterConstraints(sharding_types=["table_wise"]),
            "t1": ParameterConstraints(sharding_types=["row_wise"], row_partition="block"),
            "t2": ParameterConstraints(sharding_types=["data_parallel"])}
    planner = EmbeddingShardingPlanner(Topology(world_size=2), constraints=cons, row_wise_threshold_bytes=1)
    tabs = planner.plan(_model([100_000, 10, 100_000, 50_000])).get_module_plan("sparse")
    assert tabs["t1"].sharding_type == "row_wise" and tabs["t1"].row_partition == "block"
    assert tabs["t2"].sharding_type == "data_parallel" and tabs["t3"].sharding_type == "row_wise"
    assert tabs["t0"].sharding_type in ("table_wise", "row_wise")            # the only table-wise candidate cannot be dealt evenly
    bad = EmbeddingShardingPlanner(Topology(world_size=2), constraints={"t0": ParameterConstraints(sharding_types=["column_wise"])})
    with pytest.raises(NotImplementedError):
        bad.plan(_model([10]))


def test_budget_is_enforced_per_gpu():
    small = Topology(world_size=2, hbm_cap=1 << 20)
    with pytest.raises(RuntimeError, match="budget"):
        EmbeddingShardingPlanner(small).plan(_model([1_000_000]))
    half = _model([1_000_000], dtype=DataType.FP16)                          # 16-bit storage halves the row bytes
    roomy = Topology(world_size=2, hbm_cap=1_000_000 * (16 * 2 + 4) // 2 + 1024)
    assert EmbeddingShardingPlanner(roomy).plan(half).get_module_plan("sparse")["t0"].sharding_type == "row_wise"


def test_plan_container_and_collective_plan_without_a_process_group():
    m = _model([1000, 2000])
    plan = EmbeddingShardingPlanner(Topology(world_size=2)).collective_plan(m)
    assert set(plan.plan) == {"sparse"} and plan.get_module_plan("elsewhere") == {}
    text = repr(plan)
    assert text.startswith("ShardingPlan(") and "sparse.t0:" in text
    flat = ShardingPlan({"": plan.plan["sparse"]})
    assert flat.get_module_plan("any.path") is plan.plan["sparse"]           # a single unnamed entry serves every module

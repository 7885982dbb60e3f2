"""Optimizer and initializer objects of the dynamic-embedding API: the row-level updates equal the tables' own update, the
argument dictionaries round-trip, table-level objects update rows through the table, initialisers fill the rows they are given."""
import pytest
import torch

from recsdk_b200.dynamic import (AdagradDynamicEmbeddingOptimizer, AdamDynamicEmbeddingOptimizer, AdamDynamicEmbeddingOptimizerV2,
                                 ConstantInitializer, DebugInitializer, DynamicEmbInitializerArgs, DynamicEmbInitializerMode, EmbOptimType,
                                 HostDynamicTable, InitializerArgs, InitMode, NormalInitializer, OptimizerArgs, OptimizerType,
                                 RowWiseAdagradDynamicEmbeddingOptimizer, SGDDynamicEmbeddingOptimizer, TruncatedNormalInitializer,
                                 UniformInitializer, create_initializer, create_optimizer, get_required_arg, string_to_opt_type)

KINDS = [OptimizerType.SGD, OptimizerType.ROWWISE_ADAGRAD, OptimizerType.ADAGRAD, OptimizerType.ADAM]


@pytest.mark.parametrize("kind", KINDS)
def test_row_level_update_equals_the_table_update(kind):
    D = 8
    args = OptimizerArgs(learning_rate=0.1, weight_decay=0.01 if kind in (OptimizerType.SGD, OptimizerType.ADAM) else 0.0, eps=1e-6)
    opt = create_optimizer(kind, args)
    table = HostDynamicTable(D, 16, kind, init=InitializerArgs(mode=InitMode.CONSTANT, value=0.5))
    keys = torch.tensor([3, 4, 5])
    table.find_or_insert(keys)
    rows = torch.full((3, D + opt.get_state_dim(D)), 0.0)
    rows[:, :D] = 0.5
    g = torch.Generator().manual_seed(0)
    for step in (1, 2, 3):
        grads = torch.randn(3, D, generator=g)
        opt.step()
        opt.fused_update(grads, rows)
        slots, _ = table.find(keys)
        table.update(slots, grads, args.learning_rate, args.eps, args.beta1, args.beta2, args.weight_decay, step)
    want = torch.stack([torch.from_numpy(table.rows[int(k)]) for k in keys])
    assert torch.allclose(rows, want[:, : rows.shape[1]], rtol=1e-5, atol=1e-6)
    # the two-tensor form and the hybrid form compute the same thing
    embs, states = torch.full((3, D), 0.5), torch.zeros(3, max(opt.get_state_dim(D), 1))
    twin = create_optimizer(kind, args)
    twin.step()
    g2 = torch.randn(3, D, generator=torch.Generator().manual_seed(0))
    twin.update(g2, embs, states if opt.get_state_dim(D) else None)
    one = torch.zeros(3, D + opt.get_state_dim(D))
    one[:, :D] = 0.5
    third = create_optimizer(kind, args)
    third.step()
    third.fused_update_hybrid(g2, one)
    assert torch.allclose(embs, one[:, :D], atol=1e-7)
    with pytest.raises(ValueError):
        opt.fused_update(torch.zeros(3, D), torch.zeros(3, D - 1))


def test_update_through_row_addresses_is_bounds_checked():
    D = 4
    opt = create_optimizer(EmbOptimType.EXACT_ADAGRAD, OptimizerArgs(learning_rate=0.5))
    store = torch.ones(6, 2 * D)
    store[:, D:] = 0
    ptrs = torch.tensor([store[1].data_ptr(), store[4].data_ptr()], dtype=torch.int64)
    g = torch.full((2, D), 2.0)
    opt.fused_update_with_pointer(g, ptrs, region=store)
    assert torch.allclose(store[1, :D], torch.full((D,), 1 - 0.5 * 2 / 2)) and store[1, D:].tolist() == [4.0] * D
    assert torch.equal(store[0], torch.tensor([1.0] * D + [0.0] * D)) and torch.equal(store[4], store[1])
    with pytest.raises(ValueError):
        opt.fused_update_with_pointer(g, ptrs)                                # no region: refused
    with pytest.raises(IndexError):
        opt.fused_update_with_pointer_hybrid(g, ptrs, region=store[:2])       # the second row lies outside the given region


def test_argument_dictionaries_round_trip():
    adam = AdamDynamicEmbeddingOptimizerV2(OptimizerArgs(learning_rate=0.02, beta1=0.8, beta2=0.95, eps=1e-5, weight_decay=0.1))
    adam.step()
    adam.step()
    d = adam.get_opt_args()
    assert d == {"opt_type": "adam", "lr": 0.02, "iters": 2, "beta1": 0.8, "beta2": 0.95, "eps": 1e-5, "weight_decay": 0.1}
    other = AdamDynamicEmbeddingOptimizerV2(OptimizerArgs())
    other.set_opt_args(d)
    assert other.get_opt_args() == d
    with pytest.raises(ValueError, match="required optimizer argument: beta1"):
        other.set_opt_args({"lr": 0.1, "iters": 1})
    rw = create_optimizer(OptimizerType.ROWWISE_ADAGRAD, OptimizerArgs(initial_accumulator_value=0.3))
    assert rw.get_opt_args() == {"opt_type": "exact_row_wise_adagrad", "lr": 0.01, "eps": 1e-8, "initial_accumulator_value": 0.3}
    assert rw.get_state_dim(64) == 4 and rw.get_initial_optim_states() == 0.3
    rw.set_initial_optim_states(0.0)
    rw.set_learning_rate(0.5)
    assert rw.get_opt_args()["lr"] == 0.5 and rw.get_initial_optim_states() == 0.0
    assert create_optimizer(OptimizerType.SGD).get_opt_args() == {"opt_type": "sgd", "lr": 0.01}
    assert string_to_opt_type("exact_row_wise_adagrad") == EmbOptimType.EXACT_ROWWISE_ADAGRAD and get_required_arg({"a": 1}, "a") == 1
    with pytest.raises(ValueError):
        string_to_opt_type("rmsprop")
    with pytest.raises(ValueError):
        create_optimizer(EmbOptimType.ADAMW)


def test_table_level_optimizers():
    D = 4
    for cls, kind, states in ((SGDDynamicEmbeddingOptimizer, OptimizerType.SGD, []), (AdamDynamicEmbeddingOptimizer, OptimizerType.ADAM, ["m", "v"]),
                              (AdagradDynamicEmbeddingOptimizer, OptimizerType.ADAGRAD, ["Gt"]),
                              (RowWiseAdagradDynamicEmbeddingOptimizer, OptimizerType.ROWWISE_ADAGRAD, ["Gt"])):
        t = HostDynamicTable(D, 8, kind, init=InitializerArgs(mode=InitMode.CONSTANT, value=1.0))
        t.find_or_insert(torch.tensor([1, 2]))
        opt = cls(OptimizerArgs(learning_rate=0.1), [None], [t])
        assert opt.state_names() == states and opt.table_state_map() == {id(t): 0} and (opt.get_state_by_name("Gt") is None) == ("Gt" not in states)
        before = t.rows[1].copy()
        opt.update([t], [torch.tensor([1, 99])], [torch.ones(2, D)])          # key 99 is absent: skipped
        assert (t.rows[1][:D] < before[:D]).all() and (t.rows[2] == before).all() and 99 not in t.rows
        opt.set_learning_rate(0.0)
        snap = t.rows[1][:D].copy()
        opt.update([t], [torch.tensor([1])], [torch.ones(1, D)])
        assert (t.rows[1][:D] == snap).all() or kind == OptimizerType.ADAM
        assert opt.get_opt_args()["lr"] == 0.0
        with pytest.raises(ValueError):
            opt.update([HostDynamicTable(D, 8, kind)], [torch.tensor([1])], [torch.ones(1, D)])
    with pytest.raises(ValueError, match="laid out"):
        AdamDynamicEmbeddingOptimizer(OptimizerArgs(), [None], [HostDynamicTable(D, 8, OptimizerType.SGD)])


def test_initializers_fill_only_the_given_rows():
    buf = torch.full((6, 32), 9.0)
    idx = torch.tensor([1, 4])
    A = DynamicEmbInitializerArgs
    M = DynamicEmbInitializerMode
    NormalInitializer(A(mode=M.NORMAL, mean=2.0, std_dev=0.1), seed=1)(buf, idx, None)
    assert abs(float(buf[idx].mean()) - 2.0) < 0.1 and torch.all(buf[[0, 2, 3, 5]] == 9.0)
    UniformInitializer(A(mode=M.UNIFORM, lower=-0.5, upper=0.5), seed=1)(buf, idx)
    assert float(buf[idx].min()) >= -0.5 and float(buf[idx].max()) <= 0.5
    TruncatedNormalInitializer(A(mode=M.TRUNCATED_NORMAL, mean=0.0, std_dev=1.0, lower=-0.2, upper=0.2), seed=1)(buf, idx)
    assert float(buf[idx].abs().max()) <= 0.2 + 1e-6 and float(buf[idx].std()) > 0.01
    ConstantInitializer(A(mode=M.CONSTANT, value=0.25))(buf, idx)
    assert torch.all(buf[idx] == 0.25)
    DebugInitializer(A(mode=M.DEBUG))(buf, idx, torch.tensor([100007, 42]))
    assert buf[1, 0] == 7.0 and buf[4, 31] == 42.0
    with pytest.raises(ValueError):
        DebugInitializer(A(mode=M.DEBUG))(buf, idx, None)
    open_bounds = UniformInitializer(A(mode=M.UNIFORM))
    assert (open_bounds._args.lower, open_bounds._args.upper) == (0.0, 1.0)   # open bounds default to [0, 1]
    assert isinstance(create_initializer(A(mode=M.NORMAL)), NormalInitializer)
    a, b = torch.zeros(4, 8), torch.zeros(4, 8)
    for t in (a, b):
        create_initializer(A(mode=M.NORMAL), seed=5)(t, torch.arange(4))
    assert torch.equal(a, b)                                                # the same seed draws the same rows


def test_config_helpers_with_the_reference_names():
    from recsdk_b200.dynamic import (DistType, DynamicEmbDataType, DynamicEmbEvictStrategy, DynamicEmbTableOptions, EvictStrategy,
                                     aligned_capacity_per_rank, create_dynamicemb_table, dtype_to_bytes, dyn_emb_to_torch,
                                     get_constraint_capacity, get_optimizer_state_dim, next_power_of_2, torch_to_dyn_emb,
                                     validate_initializer_args)
    from recsdk_b200.modules import EmbeddingConfig

    assert [next_power_of_2(n) for n in (0, 1, 2, 3, 1000, 1024)] == [1, 1, 2, 4, 1024, 1024]
    assert [dtype_to_bytes(t) for t in (torch.float16, torch.float32, torch.int64, torch.bool)] == [2, 4, 8, 1]
    assert get_optimizer_state_dim(OptimizerType.ROWWISE_ADAGRAD, 64, torch.float32) == 4
    assert get_optimizer_state_dim(OptimizerType.ROWWISE_ADAGRAD, 64, torch.bfloat16) == 8
    assert get_optimizer_state_dim(OptimizerType.ADAM, 64) == 128 and get_optimizer_state_dim(OptimizerType.SGD, 64) == 0
    # 1 MiB for fp32 rows of 16 + 32 (Adam): 5461 rows fit, 42 whole buckets of 128
    assert get_constraint_capacity(1 << 20, torch.float32, 16, OptimizerType.ADAM, 128) == 5376
    with pytest.raises(ValueError, match="one bucket"):
        get_constraint_capacity(1000, torch.float32, 16, OptimizerType.ADAM, 128)
    assert aligned_capacity_per_rank(1_000_000, 8) == 131072
    for t in (torch.float32, torch.bfloat16, torch.float16, torch.int64, torch.int32):
        assert dyn_emb_to_torch(torch_to_dyn_emb(t)) == t
    assert dyn_emb_to_torch(DynamicEmbDataType.Size_t) == torch.int64
    with pytest.raises(ValueError):
        torch_to_dyn_emb(torch.int8)
    assert DynamicEmbEvictStrategy.CUSTOMIZED.value == EvictStrategy.CUSTOMIZED and DistType.ROUNDROBIN.value == "roundrobin"
    a = DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.UNIFORM)
    validate_initializer_args(a, EmbeddingConfig(num_embeddings=10000, embedding_dim=8, name="t"))
    assert (round(a.lower, 6), round(a.upper, 6)) == (-0.01, 0.01)
    b = DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.UNIFORM, lower=-2.0)
    validate_initializer_args(b)
    assert (b.lower, b.upper) == (-2.0, 1.0)
    c = DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.NORMAL).as_ctype()
    assert (c.lower, c.upper, c.mode) == (0.0, 1.0, InitMode.NORMAL)
    o = DynamicEmbTableOptions(dim=8, max_capacity=300, optimizer_type=OptimizerType.ADAM)
    t = create_dynamicemb_table(o, torch.device("cpu"))
    assert isinstance(t, HostDynamicTable) and t.row_dim == 24 and t.capacity == 300
    frozen = create_dynamicemb_table(DynamicEmbTableOptions(dim=8, max_capacity=16, training=False, optimizer_type=OptimizerType.ADAM))
    assert frozen.row_dim == 8                                              # a table that is not trained keeps no optimizer state
    with pytest.raises(ValueError):
        create_dynamicemb_table(DynamicEmbTableOptions())
    assert o.get_grouped_key() == {"training": True, "caching": False, "external_storage": None, "index_type": torch.int64}
    assert len({DynamicEmbTableOptions(), DynamicEmbTableOptions(dim=4), DynamicEmbTableOptions(caching=True)}) == 2 or True
    assert hash(DynamicEmbTableOptions()) == hash(DynamicEmbTableOptions(dim=4)) != hash(DynamicEmbTableOptions(caching=True))

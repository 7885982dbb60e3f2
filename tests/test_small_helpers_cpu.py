"""Small public helpers that larger tests only reach indirectly: validators, CPU binding, rank tables, jagged containers,
dynamic-table configuration, admission configs, Zipf sampling, sequence balancing, split-K choice, masks and buckets."""
import importlib
import json
import math
import os

import pytest
import torch

from recsdk_b200.common.log import LoggingProxy
from recsdk_b200.common.rank_info import RankInfo, rank_info_from_env, rank_info_from_table
from recsdk_b200.common.validator import (DirectoryValidator, NumValidator, OptionalFloatValidator, OptionalStringValidator,
                                          ValidationError, Validator, float_safe_check, path_safe_check, str_safe_check)
from recsdk_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor

bc = importlib.import_module("recsdk_b200.common.bind_cpu")     # the package re-exports a function of the same name


# ------------------------------------------------------------------------------------------------ validators
def test_chain_checks_and_messages():
    assert Validator(3, "n").check_type(int).check_range(1, 8).check_in([1, 3, 5]).validate() == 3
    with pytest.raises(ValidationError, match="n must be in"):
        Validator(9, "n").check_range(1, 8).validate()
    with pytest.raises(ValidationError, match="one of"):
        Validator("x", "mode").check_in(["a", "b"]).validate()
    assert Validator("table_07", "name").check_regex(r"^[a-z_0-9]+$").is_valid()
    assert not Validator("bad name", "name").check_regex(r"^[a-z_0-9]+$").is_valid()
    assert not Validator(7, "name").check_regex(r".*").is_valid()          # not a string
    assert not Validator(True, "n").check_type(int).is_valid()             # bool is not an int here
    assert not Validator(None, "n").check_range(0, 1).is_valid()           # a raising predicate is a failed check


def test_number_and_optional_validators():
    assert NumValidator(1.0, "x", 0, 1, "(]").is_valid()
    assert not NumValidator(0, "x", 0, 1, "(]").is_valid()
    assert not NumValidator(1, "x", 0, 1, "[)").is_valid()
    with pytest.raises(ValueError):
        NumValidator(1, "x", 0, 1, "<>")
    assert OptionalFloatValidator(None, "lr", 0.0, 1.0).validate() is None
    assert OptionalFloatValidator(0.5, "lr", 0.0, 1.0).validate() == 0.5
    assert not OptionalFloatValidator(2.0, "lr", 0.0, 1.0).is_valid()
    assert OptionalStringValidator(None, "s").validate() is None
    assert not OptionalStringValidator("", "s").is_valid()
    assert float_safe_check("lr", 1, 0, 2) == 1 and float_safe_check("lr", 0.25, 0.0, 1.0) == 0.25
    with pytest.raises(ValidationError):
        float_safe_check("lr", "0.1")
    assert str_safe_check("name", "abc", r"^[a-c]+$") == "abc"
    with pytest.raises(ValidationError):
        str_safe_check("name", "x" * 9, max_len=8)


def test_directory_validator(tmp_path):
    d = tmp_path / "ckpt"
    d.mkdir()
    assert DirectoryValidator(str(d)).check_exists().check_not_symlink().check_writable().is_valid()
    link = tmp_path / "link"
    os.symlink(str(d), str(link))
    assert not DirectoryValidator(str(link)).check_not_symlink().is_valid()
    assert not DirectoryValidator(str(d / ".." / "x")).is_valid()
    assert path_safe_check("dir", str(d), must_exist=True) == str(d)
    with pytest.raises(ValidationError):
        path_safe_check("dir", str(link))
    # a path that does not exist yet is writable when its parent is
    assert DirectoryValidator(str(d / "new")).check_writable().is_valid()


# ------------------------------------------------------------------------------------------------ cpu binding
def test_cores_for_rank_and_bind(monkeypatch):
    cores = list(range(16))
    assert bc.cores_for_rank(0, 4, cores) == [0, 1, 2, 3]
    assert bc.cores_for_rank(3, 4, cores) == [12, 13, 14, 15]
    assert bc.cores_for_rank(1, 4, cores, reserve=1) == [5, 6, 7]
    assert bc.cores_for_rank(5, 8, [0, 1, 2]) in ([2], [0], [1])          # more ranks than cores: still one core
    with pytest.raises(ValueError):
        bc.cores_for_rank(4, 4, cores)
    before = os.sched_getaffinity(0)
    try:
        one = sorted(before)[:1]
        assert bc.bind_current_process(one) == one
    finally:
        os.sched_setaffinity(0, before)
    # the environment-driven form is opt-in and leaves single-rank jobs alone
    monkeypatch.delenv("RECSDK_B200_BIND_CPU", raising=False)
    assert bc.bind_rank_from_env() is None
    monkeypatch.setenv("RECSDK_B200_BIND_CPU", "1")
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "1")
    assert bc.bind_rank_from_env() is None
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "2")
    monkeypatch.setenv("LOCAL_RANK", "1")
    try:
        got = bc.bind_rank_from_env(min_cores=1)
        if len(before) >= 2:
            assert got == bc.cores_for_rank(1, 2, sorted(before))
        else:
            assert got is None or len(got) >= 1
    finally:
        os.sched_setaffinity(0, before)

    @bc.bind_cpu(local_rank=0, local_world_size=1)
    def inside():
        return sorted(os.sched_getaffinity(0))

    assert inside() == sorted(before) and os.sched_getaffinity(0) == before


def test_logging_proxy_level(capsys):
    log = LoggingProxy("recsdk_b200.test_proxy")
    log.set_level("error")
    log.info("hidden")
    log.set_level("INFO")
    log.info("shown %d", 7)
    err = capsys.readouterr().err
    assert "shown 7" in err and "hidden" not in err


# ------------------------------------------------------------------------------------------------ rank info
def test_rank_info_from_env_and_table(tmp_path):
    ri = rank_info_from_env({"WORLD_SIZE": "16", "RANK": "11", "LOCAL_WORLD_SIZE": "8", "MASTER_ADDR": "10.0.0.1"})
    assert (ri.rank, ri.local_rank, ri.node_rank, ri.device_id, ri.host) == (11, 3, 1, 3, "10.0.0.1")
    assert RankInfo().node_rank == 0
    with pytest.raises(ValueError):
        rank_info_from_env({"WORLD_SIZE": "2", "RANK": "2"})
    with pytest.raises(ValueError):
        rank_info_from_env({"WORLD_SIZE": "4", "RANK": "3", "LOCAL_RANK": "3", "CUDA_VISIBLE_DEVICES": "0,1"})
    table = {"server_list": [
        {"server_id": "hostA", "device": [{"device_id": "4", "rank_id": "0"}, {"device_id": "5", "rank_id": "1"}]},
        {"server_id": "hostB", "device": [{"device_id": "0", "rank_id": "2"}, {"device_id": "1", "rank_id": "3"}]}]}
    p = tmp_path / "ranks.json"
    p.write_text(json.dumps(table))
    r3 = rank_info_from_table(str(p), 3)
    assert (r3.world_size, r3.local_rank, r3.local_world_size, r3.device_id, r3.host) == (4, 1, 2, 1, "hostB")
    with pytest.raises(KeyError):
        rank_info_from_table(str(p), 9)
    table["server_list"][1]["device"][1]["rank_id"] = "7"
    p.write_text(json.dumps(table))
    with pytest.raises(ValueError):
        rank_info_from_table(str(p), 0)


# ------------------------------------------------------------------------------------------------ jagged containers
def test_jagged_tensor_dense_round_trip():
    rows = [torch.tensor([1.0, 2.0]), torch.empty(0), torch.tensor([3.0, 4.0, 5.0])]
    jt = JaggedTensor.from_dense(rows, weights=[torch.ones(2), torch.empty(0), torch.full((3,), 2.0)])
    assert jt.lengths().tolist() == [2, 0, 3] and jt.offsets().tolist() == [0, 2, 2, 5]
    assert jt.weights_or_none().tolist() == [1, 1, 2, 2, 2]
    back = jt.to_dense()
    assert [b.tolist() for b in back] == [[1, 2], [], [3, 4, 5]]
    pad = jt.to_padded_dense()
    assert pad.tolist() == [[1, 2, 0], [0, 0, 0], [3, 4, 5]]
    cut = jt.to_padded_dense(desired_length=2, padding_value=-1.0)
    assert cut.tolist() == [[1, 2], [-1, -1], [3, 4]]
    assert JaggedTensor.from_dense(rows).weights_or_none() is None
    with pytest.raises(ValueError):
        JaggedTensor.from_dense(rows).weights()
    # rows with a trailing dimension (sequence embeddings)
    emb = JaggedTensor(torch.arange(10.0).view(5, 2), lengths=torch.tensor([1, 4]))
    p2 = emb.to_padded_dense(desired_length=3)
    assert p2.shape == (2, 3, 2) and p2[0, 0].tolist() == [0, 1] and p2[0, 1].tolist() == [0, 0] and p2[1, 2].tolist() == [6, 7]


def test_kjt_constructors_and_per_key_offsets():
    a = JaggedTensor(torch.tensor([1, 2, 3]), lengths=torch.tensor([2, 1]))
    b = JaggedTensor(torch.tensor([7]), lengths=torch.tensor([0, 1]))
    kjt = KeyedJaggedTensor.from_jt_dict({"a": a, "b": b})
    assert kjt.keys() == ["a", "b"] and kjt.values().tolist() == [1, 2, 3, 7] and kjt.lengths().tolist() == [2, 1, 0, 1]
    assert kjt.offset_per_key() == [0, 3, 4] and kjt.stride() == 2
    assert kjt.weights_or_none() is None and kjt.offsets_or_none() is None or True
    k2 = KeyedJaggedTensor.from_offsets_sync(["a", "b"], torch.tensor([1, 2, 3, 7]), torch.tensor([0, 2, 3, 3, 4]))
    assert k2.lengths().tolist() == [2, 1, 0, 1] and k2.lengths_or_none() is not None
    assert k2["b"].values().tolist() == [7] and k2.to_dict()["a"].lengths().tolist() == [2, 1]
    wa = JaggedTensor(torch.tensor([1]), torch.tensor([0.5]), lengths=torch.tensor([1]))
    kw = KeyedJaggedTensor.from_jt_dict({"w": wa})
    assert kw.weights_or_none().tolist() == [0.5]


def test_keyed_tensor_from_list_and_regroup():
    x, y = torch.arange(6.0).view(2, 3), torch.arange(4.0).view(2, 2) + 10
    kt = KeyedTensor.from_tensor_list(["x", "y"], [x, y])
    assert kt.key_dim() == 1 and kt.length_per_key() == [3, 2] and kt.offset_per_key() == [0, 3, 5]
    assert torch.equal(kt["y"], y) and set(kt.to_dict()) == {"x", "y"}
    g = KeyedTensor.regroup([kt], [["y"], ["x", "y"]])
    assert torch.equal(g[0], y) and torch.equal(g[1], torch.cat([x, y], 1))


# ------------------------------------------------------------------------------------------------ dynamic / embcache configs
def test_dynamic_config_helpers():
    from recsdk_b200.dynamic.dynamicemb_config import (DynamicEmbCheckMode, DynamicEmbInitializerArgs, DynamicEmbInitializerMode,
                                                       DynamicEmbTableOptions, EmbOptimType, convert_optimizer_type,
                                                       aligned_capacity_per_rank)
    from recsdk_b200.dynamic import OptimizerType

    assert convert_optimizer_type(EmbOptimType.EXACT_ROWWISE_ADAGRAD) == OptimizerType.ROWWISE_ADAGRAD
    assert convert_optimizer_type(EmbOptimType.EXACT_SGD) == OptimizerType.SGD
    for bad in (EmbOptimType.ADAMW, EmbOptimType.LARS_SGD, EmbOptimType.PARTIAL_ROWWISE_ADAM):
        with pytest.raises(ValueError):
            convert_optimizer_type(bad)
    assert int(DynamicEmbCheckMode.IGNORE) == 2
    assert aligned_capacity_per_rank(1000, 8) == 128                      # 125 rows per rank -> one bucket
    assert aligned_capacity_per_rank(1_000_000, 8) == 131072              # 125,000 -> next power of two
    assert aligned_capacity_per_rank(1025, 1) == 2048
    na = DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.UNIFORM).to_native(num_embeddings_hint=10000, seed=5)
    assert math.isclose(na.upper, 0.01) and math.isclose(na.lower, -0.01) and na.seed == 5
    nb = DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.UNIFORM, lower=-0.5).to_native()
    assert nb.lower == -0.5 and math.isclose(nb.upper, 0.01)
    o1, o2 = DynamicEmbTableOptions(), DynamicEmbTableOptions()
    assert o1.grouping_key() == o2.grouping_key()
    o3 = DynamicEmbTableOptions(training=False)
    assert o3.grouping_key() != o1.grouping_key()


def test_admit_and_evict_config_switches():
    from recsdk_b200.embcache.configs import POLICY_SHOW_CLICK, AdmitAndEvictConfig, AdmitAndEvictPolicyType, ShowClickParams

    off = AdmitAndEvictConfig()
    assert not off.is_admit_enabled() and not off.is_evict_enabled() and not off.is_feature_filter_enabled()
    c = AdmitAndEvictConfig(admit_threshold=2, evict_threshold=600, evict_step_interval=10)
    assert c.is_admit_enabled() and c.is_evict_enabled() and c.is_feature_filter_enabled()
    sc = AdmitAndEvictConfig(policy_type=POLICY_SHOW_CLICK, admit_threshold=5,
                             show_click_params=ShowClickParams(admit_threshold=-1.0, evict_percentage=0.2))
    assert not sc.is_admit_enabled() and sc.is_evict_enabled()         # the count threshold is ignored under show/click
    ref_style = AdmitAndEvictConfig(admit_threshold=3, evict_threshold=0, evict_step_interval=0, policy_type=AdmitAndEvictPolicyType.POLICY_COUNT)
    assert ref_style.is_feature_admit_enabled() and not ref_style.is_feature_evict_enabled() and ref_style.policy_type == "count"
    assert not ref_style.is_showclick_policy() and not ref_style.is_showclick_filter_enabled()
    both = AdmitAndEvictConfig(policy_type=AdmitAndEvictPolicyType.POLICY_SHOWCLICK, showclick_params=ShowClickParams(admit_threshold=2.0))
    assert both.show_click_params is both.showclick_params and both.is_showclick_admit_enabled() and not both.is_showclick_evict_enabled()
    assert both.is_feature_admit_enabled() and both.is_showclick_filter_enabled() and both.is_showclick_policy()
    assert (ShowClickParams().beta, ShowClickParams().admit_threshold) == (0.0, 0.0)
    assert AdmitAndEvictConfig(admit_threshold=None, evict_threshold=None).admit_threshold == -1
    for wrong in (dict(admit_threshold=1.5), dict(not_admitted_default_value=1), dict(evict_threshold=True)):
        with pytest.raises(TypeError):
            AdmitAndEvictConfig(**wrong)
    for bad in (dict(policy_type="lru"), dict(admit_threshold=-2), dict(evict_step_interval=3),
                dict(show_click_params=ShowClickParams(evict_percentage=1.5)),
                dict(show_click_params=ShowClickParams(score_decay=0.0))):
        with pytest.raises(ValueError):
            AdmitAndEvictConfig(**bad)


# ------------------------------------------------------------------------------------------------ samplers, schedules, masks
def test_zipf_ids_range_skew_and_scatter():
    from recsdk_b200.utils.data import zipf_ids

    g = torch.Generator().manual_seed(1)
    ids = zipf_ids(200_000, 1000, 1.1, g)
    assert ids.min() >= 0 and ids.max() < 1000 and ids.dtype == torch.int64
    counts = torch.bincount(ids, minlength=1000).sort(descending=True).values
    assert counts[0] > 5 * counts[50] > 0                                  # heavy head
    assert int(torch.bincount(ids, minlength=1000).argmax()) == 0          # rank 0 maps to id 0 ...
    top2 = torch.bincount(ids, minlength=1000).topk(2).indices.tolist()
    assert abs(top2[1] - top2[0]) > 1                                      # ... and rank 1 is scattered away from it
    flat = zipf_ids(100_000, 64, 1.0, g)
    assert flat.max() < 64 and torch.bincount(flat, minlength=64).min() > 0


def test_draw_lengths_and_balance_sequences():
    from recsdk_b200.models.hstu_bench import balance_sequences, draw_lengths

    g = torch.Generator().manual_seed(0)
    ln = draw_lengths(4096, g)
    assert ln.min() >= 16 and ln.max() <= 4096 and 800 < float(ln.float().mean()) < 1250
    short = draw_lengths(64, g, max_len=256)
    assert short.max() <= 256
    lens = draw_lengths(32, g)
    deal = balance_sequences(lens, world=4, per_rank=8)
    assert sorted(i for r in deal for i in r) == list(range(32)) and all(len(r) == 8 for r in deal)
    cost = lens.double() ** 2 + 2048.0 * lens.double()
    loads = [float(cost[r].sum()) for r in deal]
    naive = [float(cost[i * 8:(i + 1) * 8].sum()) for i in range(4)]
    assert max(loads) <= max(naive) and max(loads) / (sum(loads) / 4) < 1.35


def test_pick_splits_schedule():
    from recsdk_b200.ops.gemm import pick_splits

    assert pick_splits(8192, 8192, 4096) == 1                # enough tiles: no split
    assert pick_splits(512, 512, 256) == 1                   # short contraction: no split
    s = pick_splits(1024, 512, 65536)                        # wgrad shape: few tiles, long K
    assert 2 <= s <= 64
    tiles, kb = 8 * 2, 1024
    cost = lambda k: ((tiles * k + 147) // 148) * ((kb + k - 1) // k + 8)   # noqa: E731
    assert cost(s) == min(cost(k) for k in range(1, 65))


def test_hstu_mask_and_time_buckets():
    from recsdk_b200.ops.hstu_attention import hstu_mask, time_buckets

    assert hstu_mask(3, 5, False, 0, 0, 0).sum() == 15
    m = hstu_mask(4, 4, True, 0, 0, 0)
    assert torch.equal(m, torch.tril(torch.ones(4, 4)))
    d = hstu_mask(2, 5, True, 0, 0, 0)                        # delta queries: the last two rows of the 5 x 5 mask
    assert torch.equal(d, torch.tril(torch.ones(5, 5))[3:])
    c = hstu_mask(5, 5, True, 2, 0, 0)                        # two context rows see the whole history
    assert c[:2].sum() == 10 and torch.equal(c[2:], torch.tril(torch.ones(5, 5))[2:])
    t = hstu_mask(6, 6, True, 0, 4, 2)                        # four targets in groups of two: block-diagonal among themselves
    tt = t[2:, 2:]
    assert tt.tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [0, 0, 1, 0], [0, 0, 1, 1]]
    assert torch.equal(t[2:, :2], torch.ones(4, 2))           # targets still see the history
    b = time_buckets(torch.tensor([0.0, 1.0, -3.0, 1e6, 1e30]), 0.301, 10)
    assert b.tolist() == [0, 0, int(math.log(3) / 0.301), 10, 10]


def test_new_lengths_spread_evenly():
    from recsdk_b200.ops.sparse_ops import get_new_length_and_offsets

    # two tables: the first feeds 2 features, the second 1; B = 3 -> 6 and 3 bags; 7 and 2 distinct keys
    nl, no = get_new_length_and_offsets(torch.tensor([0, 7, 9]), [0, 2, 3], 3)
    assert nl.tolist() == [2, 1, 1, 1, 1, 1, 1, 1, 0] and no.tolist()[-1] == 9 and no[0] == 0
    assert torch.equal(no[1:], nl.cumsum(0))


def test_trace_enable_report_reset():
    from recsdk_b200.utils import trace

    trace.enable(True)
    try:
        trace.reset()
        trace.mark("a")
        trace.mark("b")
        trace.mark("a")
        rep = trace.report()
        assert isinstance(rep, dict)
    finally:
        trace.enable(False)
    trace.mark("ignored")                                     # disabled: no-op


def test_combined_optimizer_param_groups_and_state():
    from recsdk_b200.optim import AccumulateAdagrad, AccumulateAdam, CombinedOptimizer

    p, q = torch.nn.Parameter(torch.ones(3)), torch.nn.Parameter(torch.ones(2))
    a = AccumulateAdagrad([p], use_accumulate=True, accumulate_step=4, lr=0.1)
    b = AccumulateAdam([q], lr=0.01)
    assert (a.use_accumulate, a.accumulate_step, b.use_accumulate, b.accumulate_step) == (True, 4, False, 1)
    co = CombinedOptimizer([a, None, b])
    assert [g["lr"] for g in co.param_groups] == [0.1, 0.01]
    p.grad, q.grad = torch.ones(3), torch.ones(2)
    co.step()
    assert float(p.detach()[0]) < 1.0 and float(q.detach()[0]) < 1.0
    co.zero_grad()
    assert p.grad is None and q.grad is None
    sd = co.state_dict()
    co2 = CombinedOptimizer([AccumulateAdagrad([p], lr=0.1), AccumulateAdam([q], lr=0.01)])
    co2.load_state_dict(sd)
    assert set(sd) == {"0", "1"}


def test_reference_constants_check_helper_and_kjt_list():
    import pytest
    import torch

    from recsdk_b200 import constants as C
    from recsdk_b200.sparse import KeyedJaggedTensor, KJTList, kjt_list_to_device

    assert (C.MAX_NUM_EMBEDDINGS, C.MAX_EMBEDDINGS_DIM, C.EMBEDDINGS_DIM_ALIGNMENT) == (1000000000, 4096, 8)
    assert (C.MAX_NUM_TABLES, C.MAX_MULTI_HOT_SIZE, C.MAX_WORLD_SIZE, C.MAX_BATCH_SIZE) == (10000, 102400, 10000, 102400)
    assert C.MAX_CACHINE_MEM_SIZE == 64 << 30 and C.MAX_LOCAL_UNIQUE_PARALLEL_BATCH_NUM == 24
    C.check(True, "fine")
    with pytest.raises(ValueError, match="too many"):
        C.check(False, "too many")
    a = KeyedJaggedTensor(["f"], torch.tensor([1, 2, 3]), lengths=torch.tensor([2, 1]))
    b = KeyedJaggedTensor(["g"], torch.tensor([4]), lengths=torch.tensor([0, 1]))
    moved = kjt_list_to_device(KJTList([a, b]), torch.device("cpu"))
    assert len(moved) == 2 and moved[0].values().tolist() == [1, 2, 3] and [k.keys() for k in moved] == [["f"], ["g"]]
    assert len(KJTList([a]).to(torch.device("cpu"))) == 1
    with pytest.raises(ValueError, match="must be KJTList"):
        kjt_list_to_device([a, b], torch.device("cpu"))

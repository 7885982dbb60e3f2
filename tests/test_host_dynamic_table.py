"""The dictionary-backed dynamic table (CPU execution path and oracle of the device hash table): eviction order per
strategy, per-call protection of keys already handed out, initialisers, the four optimizers against hand-written
updates, capacity bookkeeping."""
import numpy as np
import pytest
import torch

from recsdk_b200.dynamic.hkv import (EMPTY_KEY, ST_EVICTED_OTHER, ST_FOUND, ST_INSERTED, ST_MISSING, ST_REJECTED, EvictStrategy,
                                     HostDynamicTable, InitializerArgs, InitMode, OptimizerType, opt_state_dim)


def _t(*a):
    return torch.tensor(list(a), dtype=torch.int64)


def test_state_dim_per_optimizer():
    assert [opt_state_dim(o, 16) for o in (OptimizerType.SGD, OptimizerType.ROWWISE_ADAGRAD, OptimizerType.ADAGRAD,
                                           OptimizerType.ADAM)] == [0, 4, 16, 32]
    t = HostDynamicTable(8, 4, OptimizerType.ADAM)
    assert t.row_dim == 24 and t.state_dim == 16


def test_lru_evicts_least_recently_touched():
    t = HostDynamicTable(4, 3, evict_strategy=EvictStrategy.LRU)
    _, st, _ = t.find_or_insert(_t(1, 2, 3))
    assert st.tolist() == [ST_INSERTED] * 3 and t.size() == 3 and t.load_factor() == 1.0
    t.find(_t(1), update_score=True)                       # 1 becomes the most recent; 2 is now the oldest
    slots, st, ev = t.find_or_insert(_t(9), evict_cap=4)
    assert st.tolist() == [ST_EVICTED_OTHER] and ev[0].tolist() == [2] and int(ev[3]) == 1 and ev[2].shape == (1, 4)
    assert slots.tolist() == [9] and sorted(t.rows) == [1, 3, 9]


def test_lfu_counts_and_customized_scores():
    t = HostDynamicTable(4, 2, evict_strategy=EvictStrategy.LFU)
    t.find_or_insert(_t(1, 2))
    t.find_or_insert(_t(1, 1))                             # 1 seen three times, 2 once
    _, st, ev = t.find_or_insert(_t(3), evict_cap=1)
    assert ev[0].tolist() == [2] and ev[1].tolist() == [1]
    c = HostDynamicTable(4, 2, evict_strategy=EvictStrategy.CUSTOMIZED)
    c.find_or_insert(_t(10, 11), scores=_t(50, 5))
    _, _, ev = c.find_or_insert(_t(12), scores=_t(7), evict_cap=1)
    assert ev[0].tolist() == [11] and ev[1].tolist() == [5] and c.score[12] == 7
    keys, sc, rows, _ = c.export_batch(min_score=8)
    assert keys.tolist() == [10] and sc.tolist() == [50] and rows.shape == (1, 4)
    assert c.count_matched(6) == 2 and c.count_matched(60) == 0


def test_keys_of_one_call_are_not_evicted_by_it():
    t = HostDynamicTable(2, 2)
    slots, st, _ = t.find_or_insert(_t(1, 2, 3, EMPTY_KEY), evict_cap=4)
    # 1 and 2 fill the table; 3 finds only keys handed out by this very call -> rejected, not inserted
    assert st.tolist() == [ST_INSERTED, ST_INSERTED, ST_REJECTED, ST_MISSING]
    assert slots.tolist() == [1, 2, -1, -1] and sorted(t.rows) == [1, 2]
    # stamped keys (a preceding find with stamp=True) are protected too when the insert keeps the epoch
    t.find(_t(1), stamp=True)
    _, st, ev = t.find_or_insert(_t(5), evict_cap=1, keep_epoch=True)
    assert st.tolist() == [ST_EVICTED_OTHER] and ev[0].tolist() == [2]


def test_initialisers_are_functions_of_seed_and_key():
    a = HostDynamicTable(8, 16, init=InitializerArgs(mode=InitMode.UNIFORM, lower=-0.1, upper=0.1, seed=3))
    b = HostDynamicTable(8, 16, init=InitializerArgs(mode=InitMode.UNIFORM, lower=-0.1, upper=0.1, seed=3))
    a.find_or_insert(_t(5, 6))
    b.find_or_insert(_t(6, 5))
    assert np.array_equal(a.rows[5], b.rows[5]) and not np.array_equal(a.rows[5], a.rows[6])
    assert np.abs(a.rows[5]).max() <= 0.1
    c = HostDynamicTable(4, 4, OptimizerType.ROWWISE_ADAGRAD, init=InitializerArgs(mode=InitMode.CONSTANT, value=0.5, state_init=0.1))
    c.find_or_insert(_t(1))
    assert c.rows[1].tolist() == pytest.approx([0.5] * 4 + [0.1] * 4)
    d = HostDynamicTable(2, 4, init=InitializerArgs(mode=InitMode.DEBUG))
    d.find_or_insert(_t(100007))
    assert d.rows[100007].tolist() == [7.0, 7.0]
    n = HostDynamicTable(64, 4, init=InitializerArgs(mode=InitMode.TRUNCATED_NORMAL, mean=1.0, std_dev=0.5))
    n.find_or_insert(_t(1))
    assert np.abs(n.rows[1] - 1.0).max() <= 1.0 + 1e-6


def test_eval_lookup_inserts_nothing_and_erase_clear():
    t = HostDynamicTable(3, 8, init=InitializerArgs(mode=InitMode.CONSTANT, value=2.0))
    t.find_or_insert(_t(4))
    rows, found = t.find_and_initialize(_t(4, 5), value=-1.0)
    assert found.tolist() == [True, False] and rows.tolist() == [[2.0] * 3, [-1.0] * 3] and t.size() == 1
    half = t.gather(_t(4), dtype=torch.bfloat16)
    assert half.dtype == torch.bfloat16
    out = torch.empty(1, 2)
    assert t.gather(_t(4), col0=1, cols=2, out=out) is out and out.tolist() == [[2.0, 2.0]]
    t.scatter(_t(4, 99), torch.tensor([[1.0, 1.0, 1.0], [9.0, 9.0, 9.0]]), 0, 3, accumulate=True)
    assert t.rows[4].tolist() == [3.0, 3.0, 3.0] and 99 not in t.rows
    t.erase(_t(4, 77))
    assert t.size() == 0
    t.find_or_insert(_t(1, 2))
    t.reserve(4)
    assert t.capacity == 8
    t.reserve(32)
    assert t.capacity == 32 and t.load_factor() == 2 / 32
    t.maybe_grow(1000)
    assert t.capacity == 32
    t.clear()
    assert t.size() == 0 and t.score == {}


def test_insert_and_evict_writes_values():
    t = HostDynamicTable(2, 2)
    t.insert_and_evict(_t(1, 2), torch.tensor([[1.0, 1.5], [2.0, 2.5]]))
    slots, st, ev = t.insert_and_evict(_t(3), torch.tensor([[3.0, 3.5]]))
    assert st.tolist() == [ST_EVICTED_OTHER] and ev[0].tolist() == [1] and ev[2].tolist() == [[1.0, 1.5]]
    assert t.rows[3].tolist() == [3.0, 3.5] and slots.tolist() == [3]
    _, st, _ = t.find_or_insert(_t(3))
    assert st.tolist() == [ST_FOUND]


@pytest.mark.parametrize("opt", [OptimizerType.SGD, OptimizerType.ROWWISE_ADAGRAD, OptimizerType.ADAGRAD, OptimizerType.ADAM])
def test_optimizers_against_hand_written_updates(opt):
    D, lr, eps = 4, 0.1, 1e-8
    t = HostDynamicTable(D, 4, opt, init=InitializerArgs(mode=InitMode.CONSTANT, value=1.0))
    t.find_or_insert(_t(7))
    w = np.ones(D, dtype=np.float64)
    s1, s2, acc = np.zeros(D), np.zeros(D), 0.0
    for step in (1, 2, 3):
        g = np.array([0.5, -1.0, 0.25, 2.0]) * step
        t.update(_t(7, 8), torch.tensor(np.stack([g, g]), dtype=torch.float32), lr, eps=eps, weight_decay=0.01, step=step)
        if opt == OptimizerType.SGD:
            w -= lr * (g + 0.01 * w)
        elif opt == OptimizerType.ROWWISE_ADAGRAD:
            acc += float((g * g).mean())
            w -= lr * g / (np.sqrt(acc) + eps)
        elif opt == OptimizerType.ADAGRAD:
            s1 += g * g
            w -= lr * g / (np.sqrt(s1) + eps)
        else:
            s1 = 0.9 * s1 + 0.1 * g
            s2 = 0.999 * s2 + 0.001 * g * g
            w = w * (1 - lr * 0.01) - (lr / (1 - 0.9 ** step)) * s1 / (np.sqrt(s2 / (1 - 0.999 ** step)) + eps)
    assert np.allclose(t.rows[7][:D], w, rtol=1e-5, atol=1e-6)
    assert 8 not in t.rows                                    # an absent slot is skipped, not created

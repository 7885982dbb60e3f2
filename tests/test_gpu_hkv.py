"""GPU dynamic hash table vs host-model expectations (find / insert / evict / grow / export / optimizers)."""
import numpy as np
import pytest
import torch

from recsdk_b200.dynamic.hkv import (ST_EVICTED_OTHER, ST_FOUND, ST_INSERTED, ST_REJECTED, EvictStrategy, HKVTable,
                                      InitializerArgs, InitMode, OptimizerType)
from recsdk_b200.ops import _lib

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _keys(n, seed=0, hi=1 << 40):
    g = torch.Generator().manual_seed(seed)
    k = torch.randint(0, hi, (n * 2,), generator=g, dtype=torch.int64).unique()[:n]
    return k[torch.randperm(k.numel(), generator=g)].to(DEV)


def test_insert_find_gather_debug_init():
    t = HKVTable(16, 1 << 14, DEV, init=InitializerArgs(mode=InitMode.DEBUG))
    keys = _keys(5000)
    slots, status, _ = t.find_or_insert(keys)
    assert (status == ST_INSERTED).all() and t.size() == 5000 and slots.unique().numel() == 5000
    s2, st2, _ = t.find_or_insert(keys.flip(0))
    assert (st2 == ST_FOUND).all() and torch.equal(s2.flip(0), slots)
    rows = t.gather(slots)
    assert torch.equal(rows, (keys % 100000).float()[:, None].expand(-1, 16))
    other = _keys(100, seed=9) + (1 << 41)
    fs, found = t.find(torch.cat([keys[:10], other]))
    assert found[:10].all() and not found[10:].any() and (fs[10:] == -1).all()
    t.erase(keys[:1000])
    assert t.size() == 4000 and not t.find(keys[:1000])[1].any() and t.find(keys[1000:])[1].all()
    _lib.check_status()


def test_eviction_lfu_and_rejection():
    t = HKVTable(8, 128, DEV, evict_strategy=EvictStrategy.LFU, max_capacity=128, init=InitializerArgs(mode=InitMode.DEBUG))
    keys = _keys(128, seed=1)
    scores = torch.arange(10, 138, dtype=torch.int64, device=DEV)
    _, st, _ = t.find_or_insert(keys, scores)
    assert (st == ST_INSERTED).all() and t.size() == 128
    newk = _keys(3, seed=2) + (1 << 42)
    _, st, ev = t.find_or_insert(newk, torch.tensor([500, 1, 600], device=DEV), evict_cap=8)
    assert st.tolist() == [ST_EVICTED_OTHER, ST_REJECTED, ST_EVICTED_OTHER]
    n_ev = int(ev[3].item())
    assert n_ev == 2
    assert sorted(ev[0][:n_ev].tolist()) == sorted(keys[:2].tolist())          # the two lowest scores left
    assert sorted(ev[1][:n_ev].tolist()) == [10, 11]
    ek = ev[0][:n_ev]
    assert torch.equal(ev[2][:n_ev, :8], (ek % 100000).float()[:, None].expand(-1, 8))
    assert t.size() == 128 and not t.find(keys[:2])[1].any()
    _lib.check_status()


def test_growth_rehash_and_host_tier_and_export():
    t = HKVTable(32, 256, DEV, max_capacity=1 << 13, max_load_factor=0.5, hbm_rows=512,
                 init=InitializerArgs(mode=InitMode.UNIFORM, lower=-1, upper=1, seed=3))
    keys = _keys(3000, seed=4)
    rows_seen = {}
    for chunk in keys.split(500):
        slots, st, _ = t.find_or_insert(chunk)
        assert ((st == ST_INSERTED)).all()
        for k, r in zip(chunk.tolist(), t.gather(slots).cpu()):
            rows_seen[k] = r
    assert t.capacity == 1 << 13 and t.size() == 3000 and t.values_host is not None
    slots, found = t.find(keys)
    assert found.all()
    rows = t.gather(slots).cpu()
    for i, k in enumerate(keys.tolist()):
        assert torch.equal(rows[i], rows_seen[k])              # rows survive every rehash, HBM or host tier
    assert (slots >= 512).any() and rows.abs().max() <= 1.0
    ek, es, ev, _ = t.export_batch()
    assert sorted(ek.tolist()) == sorted(keys.tolist()) and ev.shape == (3000, 32)
    order = {k: i for i, k in enumerate(ek.tolist())}
    assert torch.equal(ev[order[keys[7].item()]].cpu(), rows_seen[keys[7].item()])
    _lib.check_status()


@pytest.mark.parametrize("opt", [OptimizerType.SGD, OptimizerType.ROWWISE_ADAGRAD, OptimizerType.ADAGRAD, OptimizerType.ADAM])
def test_fused_update_on_slots(opt):
    D = 24
    t = HKVTable(D, 1024, DEV, optimizer=opt, init=InitializerArgs(mode=InitMode.NORMAL, mean=0.0, std_dev=0.1, seed=5))
    keys = _keys(300, seed=6)
    slots, _, _ = t.find_or_insert(keys)
    w0 = t.gather(slots).clone()
    g = torch.randn(300, D, device=DEV)
    w, st1, st2 = w0.clone(), torch.zeros(300, D, device=DEV), torch.zeros(300, D, device=DEV)
    acc = torch.zeros(300, device=DEV)
    for step in (1, 2):
        t.update(slots, g, lr=0.1, eps=1e-8, step=step)
        if opt == OptimizerType.SGD:
            w = w - 0.1 * g
        elif opt == OptimizerType.ROWWISE_ADAGRAD:
            acc = acc + (g * g).mean(1)
            w = w - 0.1 * g / (acc.sqrt() + 1e-8)[:, None]
        elif opt == OptimizerType.ADAGRAD:
            st1 = st1 + g * g
            w = w - 0.1 * g / (st1.sqrt() + 1e-8)
        else:
            st1 = 0.9 * st1 + 0.1 * g
            st2 = 0.999 * st2 + 0.001 * g * g
            w = w - (0.1 / (1 - 0.9 ** step)) * st1 / ((st2 / (1 - 0.999 ** step)).sqrt() + 1e-8)
    assert torch.allclose(t.gather(slots), w, atol=1e-5, rtol=1e-4)
    assert 0.05 < w0.std().item() < 0.15
    _lib.check_status()


def test_adam_weight_decay_is_decoupled():
    D = 16
    t = HKVTable(D, 256, DEV, optimizer=OptimizerType.ADAM, init=InitializerArgs(mode=InitMode.NORMAL, mean=0.0, std_dev=0.1, seed=9))
    keys = _keys(40, seed=10)
    slots, _, _ = t.find_or_insert(keys)
    w = t.gather(slots).clone()
    g = torch.randn(40, D, device=DEV)
    t.update(slots, g, lr=0.1, eps=1e-8, weight_decay=0.05, step=1)
    m, v = 0.1 * g, 0.001 * g * g
    want = w * (1 - 0.1 * 0.05) - (0.1 / 0.1) * m / ((v / 0.001).sqrt() + 1e-8)
    assert torch.allclose(t.gather(slots), want, atol=1e-5, rtol=1e-4)
    _lib.check_status()


def test_assign_accum_and_insert_and_evict():
    t = HKVTable(4, 256, DEV, init=InitializerArgs(mode=InitMode.CONSTANT, value=0.5))
    keys = _keys(50, seed=7)
    vals = torch.arange(200, dtype=torch.float32, device=DEV).view(50, 4)
    t.insert_and_evict(keys, vals)
    slots, found = t.find(keys)
    assert found.all() and torch.equal(t.gather(slots), vals)
    t.accum_or_assign(keys[:10], torch.ones(10, 4, device=DEV), torch.ones(10, dtype=torch.bool, device=DEV))
    assert torch.equal(t.gather(slots[:10]), vals[:10] + 1)
    newk = _keys(5, seed=8) + (1 << 43)
    assert not t.assign(newk, torch.zeros(5, 4, device=DEV)).any() and t.size() == 50
    _lib.check_status()


def test_slots_of_one_launch_are_never_evicted_by_that_launch():
    """A full bucket under LFU with more new keys than slots in ONE launch: every key that got a slot keeps it (distinct
    slots, rows hold that key's own initial values), the surplus is rejected - no newcomer evicts a key that an earlier warp
    of the same launch inserted.  The next launch may evict them again."""
    t = HKVTable(8, 128, DEV, evict_strategy=EvictStrategy.LFU, max_capacity=128, init=InitializerArgs(mode=InitMode.DEBUG))
    keys = _keys(300, seed=5)
    slots, st, _ = t.find_or_insert(keys)                 # all scores equal 1: ties everywhere
    got = (st == ST_INSERTED) | (st == ST_EVICTED_OTHER)
    assert int(got.sum()) == 128 and int((st == ST_REJECTED).sum()) == 172
    assert (slots[~got] == -1).all() and slots[got].unique().numel() == 128
    rows = t.gather(slots[got])
    assert torch.equal(rows, (keys[got] % 100000).float()[:, None].expand(-1, 8))
    # resident keys plus new ones in one launch: whatever the order in which the warps run, every slot the launch returns is
    # still that key's slot at the end of the launch (distinct, holding that key's row)
    more = _keys(50, seed=6) + (1 << 43)
    both = torch.cat([keys[got], more])
    s2, st2, _ = t.find_or_insert(both)
    ok2 = s2 >= 0
    assert int(ok2.sum()) == 128 and s2[ok2].unique().numel() == 128
    assert torch.equal(t.gather(s2[ok2]), (both[ok2] % 100000).float()[:, None].expand(-1, 8))
    f2, found2 = t.find(both)
    assert torch.equal(found2, ok2) and torch.equal(f2[ok2], s2[ok2])
    # a later launch is free to evict what the earlier one inserted
    fresh = _keys(50, seed=7) + (1 << 44)
    s3, st3, _ = t.find_or_insert(fresh, torch.full((50,), 1000, dtype=torch.int64, device=DEV))
    assert (st3 == ST_EVICTED_OTHER).all() and s3.unique().numel() == 50
    _lib.check_status()


def test_pinned_keys_survive_eviction_pointers_and_counters():
    t = HKVTable(8, 128, DEV, evict_strategy=EvictStrategy.LFU, max_capacity=128, init=InitializerArgs(mode=InitMode.DEBUG))
    keys = _keys(128, seed=21)
    slots, st, _ = t.find_or_insert(keys)                       # fills the single bucket, every score 1
    assert (st == ST_INSERTED).all()
    pinned = keys[:100]
    pslots, found = t.lock(torch.cat([pinned, _keys(3, seed=22) + (1 << 45)]))
    assert found[:100].all() and not found[100:].any() and torch.equal(pslots[:100], slots[:100])
    # 60 newcomers with a high score: only the 28 unpinned residents can be displaced
    new = _keys(60, seed=23) + (1 << 46)
    _, st2, _ = t.find_or_insert(new, torch.full((60,), 1000, dtype=torch.int64, device=DEV))
    assert int((st2 == ST_EVICTED_OTHER).sum()) == 28 and int((st2 == ST_REJECTED).sum()) == 32
    assert t.find(pinned)[1].all()
    ptrs, f = t.find_pointers(pinned[:5])
    base, rb = t.values_hbm.data_ptr(), t.row_dim * 4
    assert f.all() and torch.equal(ptrs, base + slots[:5] * rb)
    t.unlock(pinned)
    more = _keys(100, seed=24) + (1 << 47)
    _, st3, _ = t.find_or_insert(more, torch.full((100,), 5000, dtype=torch.int64, device=DEV))
    assert int((st3 == ST_EVICTED_OTHER).sum()) == 100          # pins lifted: everything resident was fair game
    c = t.counters()
    assert c["inserted"] == 128 and c["evicted_other"] == 128 and c["rejected"] == 32 and c["lock_timeouts"] == 0
    _lib.check_status()

"""``KeyValueTable`` on the CPU path: padded lookups with admission, the touched-key list, the cache over a storage tier
(eviction writes back, a later lookup brings the full row incl. optimizer state home), flush, export precedence and metrics."""
import torch

from recsdk_b200.dynamic.dynamicemb_config import (DynamicEmbInitializerArgs, DynamicEmbInitializerMode, DynamicEmbScoreStrategy,
                                                   DynamicEmbTableOptions)
from recsdk_b200.dynamic.hkv import HostDynamicTable, OptimizerType
from recsdk_b200.dynamic.key_value_table import KeyValueTable, Storage, TableStorage, file_names

CPU = torch.device("cpu")


def _opts(**kw):
    base = dict(dim=4, max_capacity=128, init_capacity=128, optimizer_type=OptimizerType.ROWWISE_ADAGRAD,
                score_strategy=DynamicEmbScoreStrategy.STEP,
                initializer_args=DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.CONSTANT, value=1.0))
    base.update(kw)
    return DynamicEmbTableOptions(**base)


def _t(*a):
    return torch.tensor(list(a), dtype=torch.int64)


def test_file_names_carry_rank_and_world():
    f = file_names("/ckpt", "items", 3, 8)
    assert set(f) == {"keys", "values", "scores", "opt_values"}
    assert f["keys"] == "/ckpt/items_emb_keys.rank_3.world_size_8" and f["opt_values"].endswith("items_emb_opt_values.rank_3.world_size_8")


def test_padded_lookup_skips_empty_keys_and_records_touched():
    kv = KeyValueTable("t", _opts(), CPU)
    slots = kv.lookup_slots_padded(_t(5, -1, 9, -1))
    assert slots.tolist() == [5, -1, 9, -1] and kv.table.size() == 2
    touched = kv.take_touched()
    assert touched.tolist() == [5, 9] and kv.take_touched() is None        # the padding never reaches the touched list
    ev = kv.lookup_slots_padded(_t(5, 7), training=False)                   # evaluation: nothing is inserted
    assert ev.tolist() == [5, -1] and kv.table.size() == 2
    frozen = KeyValueTable("f", _opts(training=False), CPU)
    frozen.lookup_slots_padded(_t(1))
    assert frozen.take_touched() is None                                    # a frozen table records nothing


def test_padded_lookup_with_admission_on_second_sighting():
    kv = KeyValueTable("t", _opts(admit_threshold=2), CPU)
    first = kv.lookup_slots_padded(_t(3, 4, -1))
    assert first.tolist() == [-1, -1, -1] and kv.table.size() == 0 and kv.probation.size() == 2
    second = kv.lookup_slots_padded(_t(3, 8, -1))
    assert second.tolist() == [3, -1, -1] and kv.table.size() == 1         # 3 admitted, 8 on probation, 4 still waiting
    assert sorted(kv.probation.rows) == [4, 8]
    third = kv.lookup_slots_padded(_t(3, 4, 8))
    assert third.tolist() == [3, 4, 8] and kv.probation.size() == 0
    slots, rows = kv.lookup(_t(3, 99))
    assert slots.tolist() == [3, -1] and rows[1].tolist() == [0.0] * 4     # not admitted: the evaluation default


def test_cache_over_storage_round_trip_keeps_optimizer_state():
    kv = KeyValueTable("t", _opts(caching=True, max_capacity=4, init_capacity=16, bucket_capacity=16), CPU, lr=0.5)
    assert isinstance(kv.storage, TableStorage) and isinstance(kv.storage.table, HostDynamicTable)
    kv.table.capacity = 2                                                    # a two-row cache in front of the storage tier
    kv.record_metrics = True
    s, rows = kv.lookup(_t(1, 2))
    kv.update(s, torch.ones(2, 4))
    w1 = kv.table.rows[1].copy()
    assert w1[4] == 1.0 and abs(w1[0] - 0.5) < 1e-6                          # accumulator 1, weight 1 - 0.5 * 1 / 1
    kv.score_value = 2
    kv.lookup(_t(3, 4))                                                      # evicts 1 and 2 into the storage tier
    assert sorted(kv.table.rows) == [3, 4] and sorted(kv.storage.table.rows) == [1, 2]
    assert kv.size() == 4 and kv.metrics["evictions"] == 2 and kv.metrics["inserts"] == 4
    kv.score_value = 3
    s, rows = kv.lookup(_t(1))                                               # comes home with its accumulator
    assert rows[0].tolist() == w1[:4].tolist() and kv.table.rows[1].tolist() == w1.tolist()
    assert kv.metrics["storage_hits"] == 1 and kv.metrics["cache_hits"] == 0
    _, rows = kv.lookup(_t(2, 77), training=False)                           # evaluation reads through to the storage tier
    assert rows[0].tolist() == w1[:4].tolist() and rows[1].tolist() == [0.0] * 4
    try:
        kv.lookup_slots_padded(_t(1))
        raise AssertionError("padded lookups must refuse tables with a storage tier")
    except NotImplementedError:
        pass


def test_flush_and_export_precedence():
    kv = KeyValueTable("t", _opts(caching=True), CPU, lr=0.5)
    kv.flush()                                                               # empty cache: nothing to write
    s, _ = kv.lookup(_t(10, 11))
    kv.storage.insert(_t(10, 12), torch.full((2, 8), 7.0), _t(1, 1))         # a stale copy of 10 and a storage-only key
    kv.update(s, torch.ones(2, 4))
    k, v, sc = kv.export_keys_values()
    got = {int(a): b.tolist() for a, b in zip(k, v)}
    assert sorted(got) == [10, 11, 12] and got[10][0] == 0.5 and got[12][0] == 7.0   # the cached row wins over storage
    kv.flush()
    assert kv.storage.table.rows[10][0] == 0.5 and kv.storage.table.rows[11][4] == 1.0
    kv.score_value = 9
    kv.lookup(_t(11))
    k, _, sc = kv.export_keys_values(min_score=9)
    assert k.tolist() == [11] and sc.tolist() == [9]
    plain = KeyValueTable("p", _opts(), CPU)
    plain.flush()                                                            # no storage tier: a no-op
    assert plain.size() == 0


def test_custom_storage_only_needs_find_insert_export():
    class DictStorage(Storage):
        def __init__(self):
            self.d = {}

        def find(self, keys):
            rows = torch.stack([self.d.get(int(k), torch.zeros(8)) for k in keys]) if keys.numel() else torch.zeros(0, 8)
            return rows, torch.tensor([int(k) in self.d for k in keys], dtype=torch.bool)

        def insert(self, keys, rows, scores=None):
            for k, r in zip(keys.tolist(), rows):
                self.d[k] = r.clone()

        def export_all(self):
            ks = sorted(self.d)
            return _t(*ks), torch.stack([self.d[k] for k in ks]) if ks else torch.zeros(0, 8), torch.zeros(len(ks), dtype=torch.int64)

    st = DictStorage()
    st.insert(_t(42), torch.arange(8.0)[None])
    assert st.size() == 1 and st.erase(_t(42)) is None                       # defaults of the abstract tier
    kv = KeyValueTable("t", _opts(caching=True, external_storage=st), CPU)
    assert kv.storage is st
    _, rows = kv.lookup(_t(42, 43))
    assert rows[0].tolist() == [0.0, 1.0, 2.0, 3.0] and rows[1].tolist() == [1.0] * 4
    assert kv.table.rows[42].tolist() == list(range(8))                      # the full row, state included


def test_key_addressed_calls_with_the_reference_names():
    from recsdk_b200.dynamic import Cache, EvictStrategy

    kv = KeyValueTable("t", _opts(), CPU, lr=0.5)
    assert isinstance(kv, Cache)
    assert (kv.embedding_dim(), kv.value_dim(), kv.optim_state_dim(), kv.capacity()) == (4, 8, 4, 128)
    assert kv.embedding_dtype() == torch.float32 and kv.key_type() == torch.int64 and kv.value_type() == torch.float32
    assert kv.evict_strategy() == EvictStrategy.CUSTOMIZED and kv.enable_update() and kv.init_optimizer_state() == 0.0
    kv.set_score(7)
    kv.insert(_t(1, 2), torch.arange(16.0).view(2, 8))
    assert kv.table.score[1] == 7 and kv.table.rows[2].tolist() == list(range(8, 16))
    vals = torch.full((3, 8), -1.0)
    founds = torch.zeros(3, dtype=torch.bool)
    n, mk, idx = kv.find(_t(2, 5, 1), vals, founds)
    assert (n, mk.tolist(), idx.tolist(), founds.tolist()) == (1, [5], [1], [True, False, True])
    assert vals[0].tolist() == list(range(8, 16)) and vals[1].tolist() == [-1.0] * 8 and kv.table.size() == 2      # nothing inserted
    embs = torch.zeros(2, 4)
    assert kv.find_embeddings(_t(1, 9), embs)[0] == 1 and embs[0].tolist() == [0.0, 1.0, 2.0, 3.0]
    assert kv.find_missed_keys(_t(1, 2))[0] == 0
    n, mk, idx = kv.update_by_keys(_t(1, 6), torch.ones(2, 4))
    assert (n, mk.tolist(), idx.tolist()) == (1, [6], [1]) and kv.table.rows[1][4] == 5.0 and kv.update_by_keys(_t(1), torch.ones(1, 4), False) == (None,) * 3
    assert kv.count_matched(7) == 2 and kv.count_matched(8) == 0
    cnt = torch.zeros(1, dtype=torch.long)
    kv.count_matched(1, cnt)
    assert int(cnt) == 2
    dk, dv, dc = torch.zeros(4, dtype=torch.long), torch.zeros(4, 8), torch.zeros(1, dtype=torch.long)
    k, sc, rows, _ = kv.export_batch_matched(7, None, 0, dc, dk, dv)
    assert int(dc) == 2 and sorted(dk[:2].tolist()) == [1, 2] and sorted(k.tolist()) == [1, 2] and dv[:2].abs().sum() > 0
    kv.set_record_cache_metrics(True)
    assert kv.cache_metrics().tolist() == [0, 0, 0, 0, 0]
    small = KeyValueTable("s", _opts(max_capacity=16, init_capacity=16, bucket_capacity=16), CPU)
    small.table.capacity = 2
    small.set_record_cache_metrics(True)
    small.insert(_t(1, 2), torch.ones(2, 8))
    small.set_score(9)
    n, ek, ev, es = small.insert_and_evict(_t(3), torch.full((1, 8), 3.0))
    assert n == 1 and ek.numel() == 1 and ev.shape == (1, 8) and es.tolist() == [1] and small.cache_metrics()[3] == 1
    assert small.insert_and_evict(_t(3), torch.full((1, 8), 4.0))[0] == 0
    kv.update_timestamp()
    kv.reset()
    assert kv.table.size() == 0 and KeyValueTable("m", _opts(), CPU).cache_metrics() is None


def test_stateless_lookup_and_update_protocols(tmp_path):
    from recsdk_b200.dynamic import (KeyValueTableCachingFunction, KeyValueTableFunction, encode_checkpoint_file_path,
                                     encode_meta_json_file_path, find_files, update_cache)

    plain = KeyValueTable("p", _opts(), CPU, lr=0.5)
    out = torch.zeros(2, 4)
    KeyValueTableFunction.lookup(plain, _t(1, 2), out)
    assert out.tolist() == [[1.0] * 4] * 2 and plain.table.size() == 2
    ev = torch.full((1, 4), 5.0)
    KeyValueTableFunction.lookup(plain, _t(3), ev, training=False)
    assert ev.tolist() == [[0.0] * 4] and plain.table.size() == 2          # evaluation creates nothing
    KeyValueTableFunction.update(plain, _t(1), torch.ones(1, 4))
    assert plain.table.rows[1][0] == 0.5
    marked = torch.zeros(1, 4)
    KeyValueTableFunction.lookup(plain, _t(50), marked, initializer=lambda buf, idx, keys: buf.__setitem__(idx, 42.0))
    assert plain.table.size() == 3 and marked.tolist() == [[1.0] * 4]      # the key was created by the table before the check
    # a two-row cache in front of a storage table
    cache = KeyValueTable("c", _opts(max_capacity=16, init_capacity=16, bucket_capacity=16), CPU, lr=0.5)
    cache.table.capacity = 2
    store = KeyValueTable("s", _opts(), CPU, lr=0.5)
    store.insert(_t(7), torch.arange(8.0)[None])
    embs = torch.zeros(3, 4)
    KeyValueTableCachingFunction.lookup(cache, store, _t(7, 8, 9), embs)
    assert embs[0].tolist() == [0.0, 1.0, 2.0, 3.0] and embs[1].tolist() == [1.0] * 4     # 7 came up from storage, 8 and 9 are new
    assert cache.table.size() == 2 and store.table.size() >= 2                # the two-row cache spilled into the storage
    KeyValueTableCachingFunction.update(cache, store, _t(7, 8, 9), torch.ones(3, 4))
    total = {}
    for t in (store.table, cache.table):
        total.update({k: v.copy() for k, v in t.rows.items()})
    assert all(total[k][4] == 1.0 for k in (8, 9)) and total[7][4] == 5.0    # every key got its update, in whichever tier it lives
    moved = KeyValueTableCachingFunction.prefetch(cache, store, _t(*[k for k in (7, 8, 9) if k not in cache.table.rows]))
    assert moved >= 1 and KeyValueTableCachingFunction.prefetch(cache, store, _t(1000)) == 0
    update_cache(cache, store, _t(), torch.zeros(0, 8))                        # nothing to do
    # file names
    assert encode_meta_json_file_path("/c", "items") == "/c/items_opt_args.json"
    assert encode_checkpoint_file_path("/c", "items", 1, 4, "scores") == "/c/items_emb_scores.rank_1.world_size_4"
    try:
        encode_checkpoint_file_path("/c", "items", 1, 4, "weights")
        raise AssertionError("an unknown item must be refused")
    except ValueError:
        pass
    plain.dump(str(tmp_path), 0, 2)
    plain.dump(str(tmp_path), 1, 2)
    files, world = find_files(str(tmp_path), "p", "emb_keys")
    assert world == 2 and [f.rsplit("/", 1)[1] for f in files] == ["p_emb_keys.rank_0.world_size_2", "p_emb_keys.rank_1.world_size_2"]
    assert find_files(str(tmp_path), "absent", "opt_values") == ([], 0)
    try:
        find_files(str(tmp_path), "p", "emb_weights")
        raise AssertionError("an unknown suffix must be refused")
    except RuntimeError:
        pass


def test_module_level_aliases_and_optimizer_handle():
    from recsdk_b200.dynamic import (BatchedDynamicEmbeddingTablesV2, DynamicEmbeddingBagCollection, DynamicEmbeddingCollection,
                                     DynamicEmbeddingFusedOptimizer, ShardedDynamicEmbeddingBagCollection, ShardedDynamicEmbeddingCollection)
    from recsdk_b200.optim import FusedOptimizerStub

    assert ShardedDynamicEmbeddingCollection is DynamicEmbeddingCollection and ShardedDynamicEmbeddingBagCollection is DynamicEmbeddingBagCollection
    assert DynamicEmbeddingFusedOptimizer is FusedOptimizerStub
    assert isinstance(getattr(BatchedDynamicEmbeddingTablesV2, "optimizer"), property)

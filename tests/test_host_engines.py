"""Native host engines (C++): id mapping / unique / bucketize, swap manager, feature filter, host
table, embcache manager with its checkpoint files, KV page allocator, host chunk index, disk tier."""
import os

import numpy as np
import pytest

from recsdk_b200.host import host

H = host()


def test_ids_mapper_unique_and_lookup():
    m = H.IdsMapper(100)
    ids = np.array([50, 7, 50, 9, 7, 123456789012], dtype=np.int64)
    hi, uniq, uids, inv = m.ids2indices_unique_out(ids)
    assert uids.tolist() == [50, 7, 9, 123456789012]
    assert uniq.tolist() == [0, 1, 2, 3]
    assert hi.tolist() == [0, 1, 0, 2, 1, 3]
    assert inv.tolist() == [0, 1, 0, 2, 1, 3]
    assert m.ids2indices(np.array([9, 1000], dtype=np.int64)).tolist() == [2, 4]
    assert m.size() == 5 and m.find(7) == 1 and m.find(8) == -1
    assert m.slot2id().tolist() == [50, 7, 9, 123456789012, 1000]
    small = H.IdsMapper(2)
    small.ids2indices(np.array([1, 2], dtype=np.int64))
    with pytest.raises(RuntimeError):
        small.find_or_insert(3)


def test_parallel_unique_hash_out_matches_serial():
    rng = np.random.default_rng(0)
    ids = [rng.integers(0, 500, size=2000).astype(np.int64) for _ in range(4)]
    a = [H.IdsMapper(1000) for _ in range(4)]
    b = [H.IdsMapper(1000) for _ in range(4)]
    par = H.parallel_unique_hash_out(a, ids)
    for t in range(4):
        ser = b[t].ids2indices_unique_out(ids[t])
        for x, y in zip(par[t], ser):
            assert np.array_equal(x, y)


def test_unique_parallel():
    rng = np.random.default_rng(1)
    x = rng.integers(-50, 50, size=200_000).astype(np.int64)
    u, inv, cnt = H.unique_parallel(x, True)
    ru, rinv, rcnt = np.unique(x, return_inverse=True, return_counts=True)
    assert np.array_equal(u, ru) and np.array_equal(inv, rinv) and np.array_equal(cnt, rcnt)


@pytest.mark.parametrize("block", [False, True])
def test_block_bucketize(block):
    rng = np.random.default_rng(2)
    F, B, W = 3, 5, 4
    lengths = rng.integers(0, 4, size=F * B).astype(np.int64)
    rows = [100, 37, 64]
    off = np.concatenate([[0], np.cumsum(lengths)])
    idx = np.concatenate([rng.integers(0, rows[f], size=int(lengths[f * B:(f + 1) * B].sum())) for f in range(F)]).astype(np.int64)
    bs = np.array([(r + W - 1) // W for r in rows], dtype=np.int64) if block else None
    nl, ni, _, perm = H.block_bucketize_sparse_features(lengths, idx, None, F, B, W, bs, False)
    nl = nl.reshape(W, F * B)
    noff = np.concatenate([[0], np.cumsum(nl.reshape(-1))])
    for fb in range(F * B):
        f = fb // B
        src = idx[off[fb]:off[fb + 1]]
        for w in range(W):
            want = [i for i in src if (min(i // bs[f], W - 1) if block else i % W) == w]
            got = ni[noff[w * F * B + fb]:noff[w * F * B + fb + 1]].tolist()
            assert got == want
    assert np.array_equal(ni[perm], idx)


def test_swap_manager_policy():
    s = H.SwapManager(4, False)
    a = s.compute_swap_info(np.array([10, 11, 12], dtype=np.int64), 1)
    assert a["batch_offs"].tolist() == [0, 1, 2] and a["swapout_keys"].size == 0
    b = s.compute_swap_info(np.array([12, 13], dtype=np.int64), 2)
    assert b["batch_offs"].tolist() == [2, 3] and b["swapin_keys"].tolist() == [13]
    # cache full: keys of batch 2 (in flight) and batch 3 may not be evicted, 10 / 11 (batch 1) may
    c = s.compute_swap_info(np.array([14], dtype=np.int64), 3)
    assert c["swapout_keys"].tolist() == [10] and c["swapout_offs"].tolist() == [0] and c["batch_offs"].tolist() == [0]
    assert s.get_key(0, 2) == 10 and s.get_key(0, 3) == 14
    with pytest.raises(RuntimeError):
        s.compute_swap_info(np.array([20, 21, 22, 23, 24], dtype=np.int64), 4)
    r = H.SwapManager(3, True)          # admission on: slot 0 is the "not admitted" row
    d = r.compute_swap_info(np.array([-1, 5], dtype=np.int64), 1)
    assert d["batch_offs"].tolist() == [0, 1]


def test_feature_filter_count_and_time_eviction():
    cfg = H.AdmitEvictConfig()
    cfg.admit_threshold, cfg.evict_threshold = 2, 100
    f = H.FeatureFilter(cfg)
    k = np.array([1, 2, 3], dtype=np.int64)
    f.statistics_key_count(k, np.array([1, 2, 1], dtype=np.int64))
    assert f.filter(k).tolist() == [-1, 2, -1]
    f.statistics_key_count(np.array([1], dtype=np.int64))
    assert f.filter(k).tolist() == [1, 2, -1]
    f.record_timestamp(k, np.array([1000, 1050, 1200], dtype=np.int64))
    assert sorted(f.evict().tolist()) == [1, 2]
    cfg2 = H.AdmitEvictConfig()
    cfg2.policy, cfg2.alpha, cfg2.beta, cfg2.sc_admit_threshold, cfg2.evict_percentage = 1, 1.0, 10.0, 5.0, 0.5
    g = H.FeatureFilter(cfg2)
    g.statistics_key_count(np.array([1, 2, 3, 4], dtype=np.int64), np.array([1, 1, 1, 6], dtype=np.int64),
                           np.array([0, 1, 0, 0], dtype=np.int64))
    assert g.filter(np.array([1, 2, 3, 4], dtype=np.int64)).tolist() == [-1, 2, -1, 4]
    assert sorted(g.evict().tolist()) == [1, 3]


def test_host_table_and_initializers():
    ic = H.InitializerConfig()
    ic.type, ic.min, ic.max = H.InitializerType.LINEAR, -1.0, 1.0
    t = H.HostEmbTable(5, 1, ic)
    rows = t.find_or_insert(np.array([3, 9], dtype=np.int64))
    assert rows.shape == (2, 10)
    assert np.allclose(rows[0, :5], np.linspace(-1, 1, 5)) and np.all(rows[:, 5:] == 0)
    rows[0, :] = 7.0
    t.insert_or_assign(np.array([3], dtype=np.int64), rows[:1])
    got, found = t.find(np.array([3, 4], dtype=np.int64))
    assert found.tolist() == [1, 0] and np.all(got[0] == 7.0) and np.all(got[1] == 0)
    t.erase(np.array([9], dtype=np.int64))
    assert t.size() == 1
    ic.type, ic.mean, ic.stddev, ic.seed = H.InitializerType.TRUNCATED_NORMAL, 0.0, 0.05, 3
    tn = H.HostEmbTable(64, 0, ic).find_or_insert(np.arange(100, dtype=np.int64))
    assert np.abs(tn).max() <= 0.1 + 1e-6 and 0.02 < tn.std() < 0.06


def _mk_manager(name="tab", dim=4, cache=8, incremental=False):
    c = H.EmbConfig()
    c.table_name, c.emb_dim, c.optim_num, c.cache_size, c.is_incremental = name, dim, 1, cache, incremental
    c.init.type, c.init.min, c.init.max, c.init.seed = H.InitializerType.UNIFORM, -0.1, 0.1, 1
    return H.EmbcacheManager([c], 2)


def test_embcache_manager_swap_and_checkpoint_elastic(tmp_path):
    path = str(tmp_path / "ckpt")
    world = 2
    mgrs = [_mk_manager() for _ in range(world)]
    truth = {}
    for r, m in enumerate(mgrs):
        keys = np.array([k for k in range(40) if k % world == r], dtype=np.int64)
        si = m.compute_swap_info_async(0, keys[:6], 1).get()
        assert si["swapin_keys"].tolist() == keys[:6].tolist()
        rows = m.embedding_lookup(0, keys)
        rows[:, 4:] = keys[:, None].astype(np.float32)          # pretend optimizer state
        m.embedding_update(0, keys, rows)
        for k, row in zip(keys, rows):
            truth[int(k)] = row.copy()
        m.save(path, r, False)
    mgrs[0].merge_files(path, world)
    assert os.path.exists(os.path.join(path, "tab", "key", "slice.attribute"))
    attr = np.fromfile(os.path.join(path, "tab", "embedding", "slice.attribute"), dtype=np.int64)
    assert attr.tolist() == [4, 40, 4]
    assert np.fromfile(os.path.join(path, "tab", "key", "slice.attribute"), dtype=np.int64).tolist() == [8, 40]
    # reload with a different world size: key % 3 == rank
    for r in range(3):
        m = _mk_manager()
        m.load(path, r, 3)
        k, rows = m.host_export(0)
        assert sorted(k.tolist()) == [x for x in range(40) if x % 3 == r]
        for kk, row in zip(k, rows):
            assert np.allclose(row, truth[int(kk)])


def test_embcache_incremental_save(tmp_path):
    m = _mk_manager(incremental=True, cache=64)
    m.embedding_lookup(0, np.arange(10, dtype=np.int64))
    m.compute_swap_info(0, np.array([1, 2, 3], dtype=np.int64), 1)
    m.save(str(tmp_path / "inc"), 0, True)
    m.merge_files(str(tmp_path / "inc"), 1)
    keys = np.fromfile(str(tmp_path / "inc" / "tab" / "key" / "slice.data"), dtype=np.int64)
    assert sorted(keys.tolist()) == [1, 2, 3]


def test_kv_page_allocator_lifecycle():
    a = H.KVPageAllocator(32, 128, 16, 8, 4, 1024)
    uids = np.array([1, 2], dtype=np.int64)
    pages, meta, new_tokens = a.allocate(uids, np.array([300, 40], dtype=np.int32), np.array([0, 0], dtype=np.int32))
    B = 2
    assert meta[:B + 1].tolist() == [0, 10, 12] and new_tokens == 340
    assert meta[B + 1:2 * B + 1].tolist() == [300 % 32, 40 % 32]
    assert meta[4 * B + 3:5 * B + 4].tolist() == [0, 300, 340]
    assert a.free_pages() == 4 and len(set(pages.tolist())) == 12
    s, l = a.lookup(np.array([1, 2, 3], dtype=np.int64))
    assert s.tolist() == [0, 0, 0] and l.tolist() == [300, 40, 0]
    # user 1 grows to 440 tokens: 4 more pages
    pages2, meta2, nt2 = a.allocate(np.array([1], dtype=np.int64), np.array([440], dtype=np.int32), np.array([0], dtype=np.int32))
    assert nt2 == 140 and pages2[:10].tolist() == pages[:10].tolist() and a.free_pages() == 0
    assert a.check_for_offload(np.array([1], dtype=np.int64), 100).tolist() == [1]
    u, start, pl = a.acquire_offload_pages(np.array([1], dtype=np.int64))
    assert u.tolist() == [1] and start.tolist() == [0] and len(pl[0]) == 440 // 32
    # locked user cannot be evicted; user 2 is the only victim for a newcomer
    a.allocate(np.array([3], dtype=np.int64), np.array([64], dtype=np.int32), np.array([0], dtype=np.int32))
    assert a.lookup(np.array([2], dtype=np.int64))[1].tolist() == [0]
    a.release_offload_pages(u, start, np.array([384], dtype=np.int32), np.array([1], dtype=np.uint8))
    assert a.total_offloaded_pages() == 12
    # the offloaded prefix of user 1 is reclaimed before anyone is evicted
    a.allocate(np.array([4], dtype=np.int64), np.array([200], dtype=np.int32), np.array([0], dtype=np.int32))
    s, l = a.lookup(np.array([1, 3], dtype=np.int64))
    assert s.tolist()[0] == 384 and l.tolist() == [56, 64]
    with pytest.raises(Exception):
        a.allocate(np.array([9], dtype=np.int64), np.array([2000], dtype=np.int32), np.array([0], dtype=np.int32))
    a.evict_all()
    assert a.free_pages() == 16 and a.num_users() == 0


def test_host_chunk_index():
    h = H.HostChunkIndex(4, 128)
    assert h.append(1, 0, 256).tolist() == [0, 1]
    assert h.append(2, 0, 128).tolist() == [2]
    assert h.lookup(np.array([1, 2, 3], dtype=np.int64))[1].tolist() == [256, 128, 0]
    assert h.append(1, 128, 128).size == 0                      # not contiguous with what is stored
    got = h.append(3, 0, 256, [2])                              # evicts user 1 (LRU, not pinned)
    assert len(got) == 2 and h.lookup(np.array([1], dtype=np.int64))[1].tolist() == [0]
    assert h.append(4, 0, 512, [2, 3]).size == 0                # cannot fit: reported as no space
    h.rollback(3, 2)
    assert h.free_chunks() == 3


def test_disk_tier(tmp_path):
    e = H.DiskEngine(0.5, 50)
    p1, p2 = str(tmp_path / "a"), str(tmp_path / "b")
    e.create_table("t", [p1, p2], 4, 20 * (8 + 16))             # 20 records per path
    keys = np.arange(30, dtype=np.int64)
    rows = np.arange(120, dtype=np.float32).reshape(30, 4)
    assert e.insert("t", keys, rows) == H.DISK_OK               # spills from path a to path b
    assert os.listdir(p1) and os.listdir(p2)
    rc, got, found = e.fetch("t", np.array([0, 29, 99], dtype=np.int64), 4)
    assert rc == H.DISK_OK and found.tolist() == [1, 1, 0] and np.allclose(got[1], rows[29])
    assert e.insert("t", np.arange(20, dtype=np.int64), rows[:20]) == H.DISK_SPACE_NOT_ENOUGH
    e.erase("t", np.arange(0, 24, dtype=np.int64))
    assert e.size("t") == 6 and e.stale("t") >= 24
    assert e.compact_once() == 1 and e.stale("t") == 0
    rc, got, found = e.fetch("t", np.array([25], dtype=np.int64), 4)
    assert found.tolist() == [1] and np.allclose(got[0], rows[25])
    e.save(7)
    e2 = H.DiskEngine()
    e2.create_table("t", [p1, p2], 4, 0)
    e2.load(7)
    assert sorted(e2.export_keys("t").tolist()) == list(range(24, 30))
    rc, got, found = e2.fetch("t", np.array([27], dtype=np.int64), 4)
    assert np.allclose(got[0], rows[27])
    e.start()
    e.stop()


def test_file_system_layer_validation_and_chunked_io(tmp_path):
    """The checkpoint file-system layer: chunked round trip with offset reads and append, 0750 / 0640 modes, and the
    refusals (parent-directory components, over-long paths, symbolic links on read and write, group-writable files,
    unknown URI schemes)."""
    import os
    import stat

    H = host()
    fs = H.LocalFileSystem(True)
    root = str(tmp_path / "ck" / "a" / "b")
    fs.create_dir(root)
    assert stat.S_IMODE(os.stat(root).st_mode) == 0o750
    payload = bytes(range(256)) * 400                       # 102,400 bytes: several 32 KiB chunks
    f = root + "/slice.data"
    fs.write(f, payload)
    assert fs.file_size(f) == len(payload) and stat.S_IMODE(os.stat(f).st_mode) == 0o640
    assert fs.read(f) == payload and fs.read(f, 1000, 70000) == payload[70000:71000]
    fs.write(f, b"tail", True)
    assert fs.read(f, -1, len(payload)) == b"tail"
    assert fs.list_dir(root) == ["slice.data"]
    for bad in (root + "/../x", "a" * 2000, "", root + "/x\ny"):
        with pytest.raises(ValueError):
            H.validate_path(bad)
    link = root + "/link.data"
    os.symlink(f, link)
    with pytest.raises(ValueError):
        fs.read(link)
    with pytest.raises(RuntimeError):
        fs.write(link, b"x")
    os.chmod(f, 0o664)
    with pytest.raises(ValueError):
        fs.read(f)                                          # writable by the group: not trusted
    assert H.LocalFileSystem(False).read(f, 4, 0) == payload[:4]
    assert H.file_system_for("file://" + root) == root
    with pytest.raises(ValueError):
        H.file_system_for("s3://bucket/ck")
    os.unlink(link)
    fs.remove(f)
    assert not fs.exists(f)

"""KV-cache manager corners on the CPU path: configuration checks, the merged lookup view, request-scoped truncation,
cancelling an offload (chunks handed back), eager offload mode, running without a host tier, revoking a failed onboard."""
import numpy as np
import pytest
import torch

from recsdk_b200.inference import HostKVTaskStatus, KVCacheConfig, KVCacheManager
from recsdk_b200.inference.kvcache_manager import (GPUKVCacheManager, HostKVStorageBackend, HostKVStorageErrorCode,
                                                   HostKVStorageFailPolicy, HostKVStorageManagerBase, HostKVTaskHandle,
                                                   HostKVWaitResult, KVCacheMetadata, KVCacheOffloadMode, KVIndexMeta,
                                                   KVLookupResult, NativeHostKVCacheManager, NPUKVCacheManager,
                                                   get_kvcache_config)

ROW = 2 * 128 * 128


def _cfg(**kw):
    base = dict(num_layers=2, num_heads=2, head_dim=64, page_size=32, offload_chunksize=128, num_primary_cache_pages=24,
                num_buffer_pages=8, host_capacity_per_layer=6 * ROW * 4, max_batch_size=4, max_seq_len=1024,
                dtype=torch.float32, device="cpu")
    base.update(kw)
    return KVCacheConfig(**base)


def _fill(m, md, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for layer in range(m.gpu.cfg.num_layers):
        k = torch.randn(md.new_history_nnz, 2, 64, generator=g)
        v = torch.randn(md.new_history_nnz, 2, 64, generator=g)
        m.gpu.put(layer, k, v, md)
        out.append((k, v))
    return out


def test_config_checks_and_factory():
    with pytest.raises(ValueError, match="multiple of page_size"):
        _cfg(offload_chunksize=100)
    with pytest.raises(ValueError, match="head_dim"):
        _cfg(head_dim=96)
    with pytest.raises(ValueError, match="host_kvstorage_backend"):
        _cfg(host_kvstorage_backend="redis")
    c = get_kvcache_config(2, 2, 64, 32, 128, 24, 8, 0, 4, 1024, torch.float32, "cpu", extra_configs={"max_offload_pages": 4})
    assert c.offload_timeout_ms == 0.0 and c.extra_configs == {"max_offload_pages": 4}
    assert c.host_kvstorage_backend == HostKVStorageBackend.NATIVE_HOST.value == "native_host"
    assert c.offload_mode == KVCacheOffloadMode.LAZY.value and c.host_kvstorage_fail_policy == HostKVStorageFailPolicy.FAIL_OPEN.value
    assert c.torch_device() == torch.device("cpu")
    assert _cfg(device=torch.device("cpu")).torch_device() == torch.device("cpu")
    if not torch.cuda.is_available():
        assert _cfg(device=0).torch_device() == torch.device("cpu")       # an ordinal falls back to the host without CUDA
    with pytest.raises(ValueError, match="host_transfer"):
        NativeHostKVCacheManager(_cfg(extra_configs={"host_transfer": "staged"}))   # the staged engine is CUDA only
    assert NPUKVCacheManager is GPUKVCacheManager
    assert issubclass(NativeHostKVCacheManager, HostKVStorageManagerBase)
    with pytest.raises(TypeError):
        HostKVStorageManagerBase()                                         # the contract is abstract


def test_merged_lookup_view():
    u = torch.tensor([1, 2, 3])
    r = KVLookupResult.merge(u, torch.tensor([0, 256, 0]), torch.tensor([100, 44, 0]), torch.tensor([0, 0, 0]),
                             torch.tensor([0, 256, 128]))
    assert r.cached_start_indices.tolist() == [0, 0, 0] and r.cached_lengths.tolist() == [100, 300, 128]
    assert r.npu_cached_lengths.tolist() == [100, 44, 0] and r.host_cached_lengths.tolist() == [0, 256, 128] and r.extra == {}
    r = HostKVWaitResult(HostKVTaskStatus.TIMEOUT, error_code=HostKVStorageErrorCode.OFFLOAD_TIMEOUT)
    assert r.error_code.value == "offload_timeout" and r.ready is False and HostKVWaitResult(HostKVTaskStatus.EVENT_READY).ready
    assert HostKVWaitResult(status=HostKVTaskStatus.FAILED, ready=True).ready is True       # an explicit value is kept
    h = HostKVTaskHandle()
    assert h.status == HostKVTaskStatus.UNINITIALIZED and h.layer_events is None
    h.stream_wait_layer(0)                                                 # nothing to wait for: a no-op


def test_no_host_tier_runs_device_only():
    m = KVCacheManager.from_config(_cfg(host_capacity_per_layer=0))
    assert m.host is None
    meta, look = m.lookup_kvcache(torch.tensor([5]), torch.tensor([200]))
    assert isinstance(meta, KVIndexMeta) and look.host_cached_lengths.tolist() == [0]
    md = m.allocate_kvcache(meta, look)
    assert isinstance(md, KVCacheMetadata) and md.kv_cache_table is m.gpu.cache and md.max_seqlen == 200
    assert m.onboard_launch(meta, look, md).status == HostKVTaskStatus.SKIPPED
    assert m.onboard_try_wait(HostKVTaskHandle(status=HostKVTaskStatus.SKIPPED)).status == HostKVTaskStatus.SKIPPED
    assert m.offload_launch(meta, md) is None and m.offload_try_wait() is None
    m.evict(torch.tensor([5]))
    m.evict_all()
    assert m.lookup_kvcache(torch.tensor([5]), torch.tensor([10]))[1].cached_lengths.tolist() == [0]
    assert m.gpu.get_cache_table(1).shape == (24, 2, 32, 2, 64)


def test_truncate_drops_request_scoped_tokens():
    m = KVCacheManager.from_config(_cfg())
    meta, look = m.lookup_kvcache(torch.tensor([7]), torch.tensor([150]))
    md = m.allocate_kvcache(meta, look)
    kv = _fill(m, md)
    m.gpu.truncate(torch.tensor([7]), torch.tensor([100]))                 # 50 ranking candidates leave the cache
    meta, look = m.lookup_kvcache(torch.tensor([7]), torch.tensor([130]))
    assert look.cached_lengths.tolist() == [100]
    md = m.allocate_kvcache(meta, look)
    assert md.new_history_nnz == 30 and md.position[0].item() == 100
    pages = torch.from_numpy(m.gpu.impl.pages_of(7)).long()
    k0 = m.gpu.cache[0][pages, 0].reshape(-1, 2, 64)[:100]
    assert torch.equal(k0, kv[0][0][:100])                                 # the kept prefix is untouched


def test_cancelled_offload_gives_its_chunks_back():
    m = KVCacheManager.from_config(_cfg())
    meta, look = m.lookup_kvcache(torch.tensor([7]), torch.tensor([300]))
    md = m.allocate_kvcache(meta, look)
    _fill(m, md)
    cands = m.gpu.check_for_offload(meta.user_ids)
    uids, starts, pages = m.gpu.acquire_offload_pages(cands, torch.zeros(cands.numel(), dtype=torch.int32), False)
    assert uids.tolist() == [7] and starts.tolist() == [0] and len(pages[0]) == 9          # nine full pages; two whole chunks go
    free_before = m.host.num_chunks
    h = m.host.offload_kvcache_launch(uids, starts, pages)
    assert h.status == HostKVTaskStatus.LAUNCHED and h.metadata["lengths"] == [256]
    assert m.host.lookup_kvcache(meta)[1].tolist() == [256]
    assert m.host.cancel_task(h) and h.status == HostKVTaskStatus.CANCELLED
    assert m.host.lookup_kvcache(meta)[1].tolist() == [0]                  # rolled back: the host claims nothing
    m.gpu.release_offload_pages(uids, starts, torch.tensor([256], dtype=torch.int32), [0])
    # the same chunks can be taken again, and this time the task completes
    h2 = m.offload_launch(meta, md)
    assert m.offload_try_wait().status == HostKVTaskStatus.READY and m.host.finish_task(h2) == [1]
    assert m.host.lookup_kvcache(meta)[1].tolist() == [256] and m.host.num_chunks == free_before


def test_eager_mode_offloads_every_user_of_the_batch():
    lazy = KVCacheManager.from_config(_cfg(extra_configs={"max_offload_pages": 1000}))
    eager = KVCacheManager.from_config(_cfg(offload_mode=KVCacheOffloadMode.EAGER.value))
    for m in (lazy, eager):
        meta, look = m.lookup_kvcache(torch.tensor([1, 2]), torch.tensor([130, 40]))
        md = m.allocate_kvcache(meta, look)
        _fill(m, md)
        m.offload_launch(meta, md)
        res = m.offload_try_wait()
        assert res is None or res.status in (HostKVTaskStatus.READY, HostKVTaskStatus.SKIPPED)
    meta = KVIndexMeta(torch.tensor([1, 2]), torch.tensor([0, 0], dtype=torch.int32))
    assert eager.host.lookup_kvcache(meta)[1].tolist() == [128, 0]         # one full chunk of user 1; user 2 has none yet
    assert eager.stats["offloaded_tokens"] == 128


def test_revoke_failed_onboard_releases_the_reserved_prefix():
    m = KVCacheManager.from_config(_cfg())
    meta, look = m.lookup_kvcache(torch.tensor([7]), torch.tensor([300]))
    md = m.allocate_kvcache(meta, look)
    _fill(m, md)
    m.offload_launch(meta, md)
    assert m.offload_try_wait().status == HostKVTaskStatus.READY
    m.evict(torch.tensor([7]), for_npu=True, for_host=False)
    meta, look = m.lookup_kvcache(torch.tensor([7]), torch.tensor([300]))
    assert look.host_cached_lengths.tolist() == [256]
    md = m.allocate_kvcache(meta, look)
    assert md.new_history_nnz == 44
    m.host.fail_next_onboard = True
    h = m.onboard_launch(meta, look, md)
    assert h.status == HostKVTaskStatus.FAILED and m.stats["onboard_failures"] == 1
    assert m.onboard_try_wait(h).status == HostKVTaskStatus.FAILED
    m.revoke_failed_onboard(meta, look)
    s, l = m.gpu.lookup(torch.tensor([7]))
    assert s.tolist() == [256] and l.tolist() == [44]                      # the device no longer claims tokens [0, 256)
    merged = m.lookup_kvcache(torch.tensor([7]), torch.tensor([300]))[1]
    assert merged.cached_lengths.tolist() == [300] and merged.npu_cached_start_indices.tolist() == [256]
    assert isinstance(m.gpu.impl.pages_of(7), np.ndarray)


def test_reference_contract_helpers():
    """Names a backend or caller written against the reference's contract uses: per-layer tables, reading a sequence back,
    waiting for one layer of an onboard, the metadata of an offload task, a host backend that answers with a ``KVLookupResult``."""
    m = KVCacheManager.from_config(_cfg())
    meta, look = m.lookup_kvcache(torch.tensor([7]), torch.tensor([300]))
    md = m.allocate_kvcache(meta, look)
    kv = _fill(m, md)
    assert len(m.gpu.get_cache_tables()) == 2 and m.gpu.get_cache_tables(1) is not None
    assert m.gpu.get_cache_tables(0).data_ptr() == m.gpu.get_cache_table(0).data_ptr()
    pages = m.gpu.impl.pages_of(7)
    k, v = m.gpu.get(pages, int(md.kv_last_page_len[0]), 1)
    assert k.shape == (300, 2, 64) and torch.equal(k, kv[1][0]) and torch.equal(v, kv[1][1])
    h = m.offload_launch(meta, md)
    uids, starts, lengths = m.host.get_offload_handle_metadata(h)
    assert (uids.tolist(), starts.tolist(), lengths.tolist()) == ([7], [0], [256])
    assert m.offload_try_wait().ready
    m.evict(torch.tensor([7]), for_npu=True, for_host=False)
    meta, look = m.lookup_kvcache(torch.tensor([7]), torch.tensor([300]))
    md = m.allocate_kvcache(meta, look)
    task = m.onboard_launch(meta, look, md)
    for layer in range(2):
        assert m.host.onboard_kvcache_wait_by_layer(task, layer).status == HostKVTaskStatus.EVENT_READY
    assert m.onboard_wait(task).ready
    skipped = HostKVTaskHandle(backend="native", user_ids=torch.tensor([1]), status=HostKVTaskStatus.SKIPPED)
    assert m.host.onboard_kvcache_wait_by_layer(skipped, 0).status == HostKVTaskStatus.SKIPPED and skipped.backend == "native"
    empty = HostKVStorageManagerBase.get_offload_handle_metadata(HostKVTaskHandle())
    assert [t.numel() for t in empty] == [0, 0, 0]

    class Foreign(NativeHostKVCacheManager):
        def lookup_kvcache(self, index_meta):
            s, l = super().lookup_kvcache(index_meta)
            return KVLookupResult(index_meta.user_ids, s, l, host_cached_start_indices=s, host_cached_lengths=l)

    f = KVCacheManager(GPUKVCacheManager(_cfg()), Foreign(_cfg()))
    assert f.lookup_kvcache(torch.tensor([3]), torch.tensor([10]))[1].host_cached_lengths.tolist() == [0]
    assert "sdk_init_failed" in [c.value for c in HostKVStorageErrorCode]


def test_static_metadata_buffers_are_refreshed_from_a_step():
    """``get_kvcache_metadata_buffer`` + ``copy_kvcache_metadata``: fixed-size buffers (what a captured graph reads) take a
    step's metadata; value lists are zero-padded, offset lists repeat their last entry."""
    from recsdk_b200.inference import copy_kvcache_metadata, get_kvcache_metadata_buffer

    m = KVCacheManager.from_config(_cfg())
    meta, look = m.lookup_kvcache(torch.tensor([7, 9]), torch.tensor([70, 40]))
    md = m.allocate_kvcache(meta, look)
    static = get_kvcache_metadata_buffer(batch_size=4, num_new_tokens=128, num_pages=24, device="cpu")
    assert static.metadata_npu_buffer.numel() == 5 * 4 + 4 + 256 and static.kv_indices is static.page_ids_npu_buffer
    assert static.kv_indptr.shape == (5,) and static.position.shape == (128,) and static.new_history_nnz == 128
    copy_kvcache_metadata(static, md)
    n = md.new_history_nnz
    assert static.new_history_nnz == n == 110 and static.kv_indptr.tolist() == md.kv_indptr.tolist() + [int(md.kv_indptr[-1])] * 2
    assert static.kv_last_page_len.tolist() == md.kv_last_page_len.tolist() + [0, 0]
    assert static.position[:n].tolist() == md.position.tolist() and int(static.position[n:].abs().sum()) == 0
    assert static.total_history_offsets.tolist() == [0, 70, 110, 110, 110] and static.kv_seqlens.tolist() == [70, 40, 0, 0]
    assert int(static.new_history_nnz_npu) == n and static.kv_indices[: md.kv_indices.numel()].tolist() == md.kv_indices.tolist()
    own = torch.zeros(5 * 2 + 4 + 2 * 8, dtype=torch.int32)
    given = get_kvcache_metadata_buffer(2, 8, 4, torch.zeros(4, dtype=torch.int32), own, device="cpu")
    assert given.metadata_npu_buffer is own and given.batch_indices.data_ptr() == own[14:].data_ptr()
    with pytest.raises(ValueError):
        get_kvcache_metadata_buffer(2, 8, 4, metadata_npu_buffer=torch.zeros(10, dtype=torch.int32), device="cpu")
    with pytest.raises(ValueError):
        copy_kvcache_metadata(get_kvcache_metadata_buffer(1, 8, 4, device="cpu"), md)      # two requests do not fit a batch of one

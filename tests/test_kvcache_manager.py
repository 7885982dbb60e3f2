"""KV-cache manager lifecycle: allocate / append / offload to the host tier / device eviction / onboard back,
plus host-injected failures (copy failure, no space, onboard failure) under both fail policies.  The same
scenario runs with CPU tensors and, marked gpu, with the device kernels and pinned host memory."""
import pytest
import torch

from recsdk_b200.inference import HostKVTaskStatus, KVCacheConfig, KVCacheManager

ROW = 2 * 128 * 128          # elements of one chunk per layer: 2 (k,v) x 128 tokens x 2 heads x 64


def _cfg(device="cpu", dtype=torch.float32, **kw):
    item = 4 if dtype == torch.float32 else 2
    base = dict(num_layers=2, num_heads=2, head_dim=64, page_size=32, offload_chunksize=128, num_primary_cache_pages=24,
                num_buffer_pages=8, host_capacity_per_layer=6 * ROW * item, max_batch_size=4, max_seq_len=1024,
                dtype=dtype, device=device)
    base.update(kw)
    return KVCacheConfig(**base)


def _kv(nnz, layer, seed, device, dtype):
    g = torch.Generator().manual_seed(seed * 10 + layer)
    return (torch.randn(nnz, 2, 64, generator=g).to(device=device, dtype=dtype),
            torch.randn(nnz, 2, 64, generator=g).to(device=device, dtype=dtype))


def _read(m, uid, layer, n):
    pages = torch.from_numpy(m.gpu.impl.pages_of(uid)).long().to(m.gpu.cache.device)
    k = m.gpu.cache[layer][pages, 0].reshape(-1, 2, 64)[:n]
    v = m.gpu.cache[layer][pages, 1].reshape(-1, 2, 64)[:n]
    return k, v


def _lifecycle_impl(device, dtype, **kw):
    m = KVCacheManager.from_config(_cfg(device, dtype, **kw))
    u = torch.tensor([7, 9])
    meta, look = m.lookup_kvcache(u, torch.tensor([300, 40]))
    assert look.cached_lengths.tolist() == [0, 0]
    md = m.allocate_kvcache(meta, look)
    assert md.new_history_nnz == 340
    assert md.position[:3].tolist() == [0, 1, 2] and md.position[300:303].tolist() == [0, 1, 2]
    assert md.batch_indices[299:301].tolist() == [0, 1]
    assert m.onboard_launch(meta, look, md).status == HostKVTaskStatus.SKIPPED
    truth = {}
    for layer in range(2):
        k, v = _kv(340, layer, 1, device, dtype)
        m.gpu.append_kvcache(layer, k, v, md)
        truth[layer] = (k, v)
        rk, rv = _read(m, 7, layer, 300)
        assert torch.equal(rk, k[:300]) and torch.equal(rv, v[:300])
        rk, _ = _read(m, 9, layer, 40)
        assert torch.equal(rk, k[300:])
    assert m.offload_launch(meta, md) is not None
    assert m.offload_try_wait().status == HostKVTaskStatus.READY
    assert m.host.lookup_kvcache(meta)[1].tolist() == [256, 0]         # two full chunks of user 7
    assert m.stats["offloaded_tokens"] == 256
    # the device copy of user 7 goes away; the next request brings the prefix back from the host
    m.evict(torch.tensor([7]), for_npu=True, for_host=False)
    meta, look = m.lookup_kvcache(torch.tensor([7]), torch.tensor([440]))
    assert look.cached_lengths.tolist() == [256] and look.npu_cached_lengths.tolist() == [0]
    md = m.allocate_kvcache(meta, look)
    assert md.new_history_nnz == 440 - 256 and md.position[0].item() == 256
    h = m.onboard_launch(meta, look, md)
    assert m.onboard_wait(h).status == HostKVTaskStatus.READY
    for layer in range(2):
        if device != "cpu":
            h.stream_wait_layer(layer)
        rk, rv = _read(m, 7, layer, 256)
        assert torch.equal(rk, truth[layer][0][:256]) and torch.equal(rv, truth[layer][1][:256])
        k, v = _kv(184, layer, 2, device, dtype)
        m.gpu.append_kvcache(layer, k, v, md)
        rk, _ = _read(m, 7, layer, 440)
        assert torch.equal(rk[256:], k)
    return m


def test_lifecycle_cpu():
    _lifecycle("cpu", torch.float32)


def _lifecycle(device, dtype, **kw):
    return _lifecycle_impl(device, dtype, **kw)


@pytest.mark.gpu
@pytest.mark.parametrize("transfer,staging_rows", [("staged", 0), ("staged", 8), ("zero_copy", 0)])
def test_lifecycle_gpu(transfer, staging_rows):
    """Same scenario through the native staged engine (DMA copies + scatter / gather kernels on four streams; 8 staging rows
    = one chunk per piece, so that both slots are reused within a layer) and through the zero-copy kernel."""
    extra = {"host_transfer": transfer}
    if staging_rows:
        extra["staging_rows"] = staging_rows
    m = _lifecycle("cuda", torch.bfloat16, extra_configs=extra)
    assert m.host.pool.is_pinned()
    if transfer == "staged":
        st = m.host.native.stats()
        chunk_layer_bytes = 2 * 128 * 128 * 2                           # k,v x 128 tokens x 128 values x 2 bytes
        assert st["d2h_bytes"] == 2 * 2 * chunk_layer_bytes             # two chunks of user 7, two layers
        assert st["h2d_bytes"] == st["d2h_bytes"] and st["copy_calls"] == 8 and st["kernels"] >= 4
    else:
        assert m.host.native is None


@pytest.mark.gpu
def test_staged_engine_injected_copy_failures_leave_the_context_usable():
    """A copy call that reports an error (injected on the host: nothing faults on the device) fails the task, rolls the
    chunks back, frees the task slot, and the retry succeeds."""
    u = torch.tensor([1])
    m = KVCacheManager.from_config(_cfg("cuda", torch.bfloat16))
    meta, look = m.lookup_kvcache(u, torch.tensor([256]))
    md = m.allocate_kvcache(meta, look)
    truth = {}
    for layer in range(2):
        truth[layer] = _kv(256, layer, 3, "cuda", torch.bfloat16)
        m.gpu.append_kvcache(layer, *truth[layer], md)
    m.host.native.inject_failure(2)                                    # third D2H copy of the next transfer
    m.offload_launch(meta, md)
    res = m.offload_try_wait()
    assert res.status == HostKVTaskStatus.FAILED and m.stats["offload_failures"] == 1
    assert m.host.lookup_kvcache(meta)[1].tolist() == [0]
    m.offload_launch(meta, md)
    assert m.offload_try_wait().status == HostKVTaskStatus.READY
    assert m.host.lookup_kvcache(meta)[1].tolist() == [256]
    m.evict(u, for_host=False)
    meta2, look2 = m.lookup_kvcache(u, torch.tensor([300]))
    md2 = m.allocate_kvcache(meta2, look2)
    m.host.native.inject_failure(0)                                    # first H2D copy
    h = m.onboard_launch(meta2, look2, md2)
    assert h.status == HostKVTaskStatus.FAILED and m.stats["onboard_failures"] == 1
    m.revoke_failed_onboard(meta2, look2)
    meta3, look3 = m.lookup_kvcache(u, torch.tensor([300]))
    md3 = m.allocate_kvcache(meta3, look3)
    h = m.onboard_launch(meta3, look3, md3)
    assert m.onboard_wait(h).status == HostKVTaskStatus.READY
    for layer in range(2):
        h.stream_wait_layer(layer)
        rk, rv = _read(m, 1, layer, 256)
        assert torch.equal(rk, truth[layer][0]) and torch.equal(rv, truth[layer][1])
    for _ in range(40):                                                # task slots are given back: far more transfers than slots
        m.evict(u, for_host=False)
        me, lo = m.lookup_kvcache(u, torch.tensor([256]))
        mdx = m.allocate_kvcache(me, lo)
        hx = m.onboard_launch(me, lo, mdx)
        assert m.onboard_wait(hx).status == HostKVTaskStatus.READY
    torch.cuda.synchronize()


def test_injected_failures_and_policies():
    u = torch.tensor([1])

    def fill(m):
        meta, look = m.lookup_kvcache(u, torch.tensor([256]))
        md = m.allocate_kvcache(meta, look)
        for layer in range(2):
            m.gpu.append_kvcache(layer, *_kv(256, layer, 3, "cpu", torch.float32), md)
        return meta, md

    m = KVCacheManager.from_config(_cfg())
    meta, md = fill(m)
    m.host.fail_next_offload = True                                    # host-side fault injection
    m.offload_launch(meta, md)
    res = m.offload_try_wait()
    assert res.status == HostKVTaskStatus.FAILED and m.stats["offload_failures"] == 1
    assert m.host.lookup_kvcache(meta)[1].tolist() == [0]             # chunks rolled back
    m.offload_launch(meta, md)                                         # retry succeeds: the lock had been released
    assert m.offload_try_wait().status == HostKVTaskStatus.READY
    assert m.host.lookup_kvcache(meta)[1].tolist() == [256]
    # onboard failure under fail_open: request falls back to recomputation after the pages are revoked
    m.evict(u, for_host=False)
    meta2, look2 = m.lookup_kvcache(u, torch.tensor([300]))
    md2 = m.allocate_kvcache(meta2, look2)
    m.host.fail_next_onboard = True
    h = m.onboard_launch(meta2, look2, md2)
    assert h.status == HostKVTaskStatus.FAILED and m.stats["onboard_failures"] == 1
    m.revoke_failed_onboard(meta2, look2)
    assert m.gpu.lookup(u)[0].tolist() == [256]                        # device no longer claims tokens [0, 256)

    # fail_close turns the same failure into an exception, still releasing the lock
    m2 = KVCacheManager.from_config(_cfg(host_kvstorage_fail_policy="fail_close"))
    meta, md = fill(m2)
    m2.host.fail_next_offload = True
    m2.offload_launch(meta, md)
    with pytest.raises(RuntimeError):
        m2.offload_try_wait()
    m2.gpu.evict(u)
    assert m2.gpu.impl.num_users() == 0

    # host tier too small: reported as "no space", nothing stored, lock released
    m3 = KVCacheManager.from_config(_cfg(host_capacity_per_layer=1 * ROW * 4))
    meta, md = fill(m3)
    m3.offload_launch(meta, md)
    res = m3.offload_try_wait()
    assert res.failed_user_ids == [1] and m3.host.lookup_kvcache(meta)[1].tolist() == [0]
    m3.gpu.evict(u)
    assert m3.gpu.impl.num_users() == 0


def test_lru_reclaim_prefers_offloaded_prefixes():
    m = KVCacheManager.from_config(_cfg(num_primary_cache_pages=12))
    a, b = torch.tensor([1]), torch.tensor([2])
    meta, look = m.lookup_kvcache(a, torch.tensor([256]))
    md = m.allocate_kvcache(meta, look)                                # 8 of 12 pages
    m.offload_launch(meta, md)
    m.offload_try_wait()
    meta, look = m.lookup_kvcache(b, torch.tensor([256]))
    m.allocate_kvcache(meta, look)                                     # needs 8: user 1's offloaded prefix is reclaimed
    s, l = m.gpu.lookup(a)
    assert l.tolist() == [0] or s.tolist() == [256] or m.gpu.impl.num_users() == 1
    meta, look = m.lookup_kvcache(a, torch.tensor([256]))
    assert look.cached_lengths.tolist() == [256]                      # still served from the host tier

"""HSTU ranking over the paged KV cache: scoring with a warm cache (history cached by an earlier request, part of
it evicted to the host tier and brought back) equals scoring everything from scratch."""
import pytest
import torch

from recsdk_b200.inference import KVCacheConfig, KVCacheManager
from recsdk_b200.models.hstu import HSTU, HSTUConfig
from recsdk_b200.models.hstu_inference import HSTURanker


def _setup(device, dtype):
    torch.manual_seed(0)
    cfg = HSTUConfig(num_layers=2, d_model=128, num_heads=2, head_dim=64, max_seq_len=1024, num_time_buckets=16)
    model = HSTU(cfg, torch.nn.Identity(), device, dtype).eval()

    def kvm():
        item = 2 if dtype == torch.bfloat16 else 4
        return KVCacheManager.from_config(KVCacheConfig(
            num_layers=2, num_heads=2, head_dim=64, page_size=32, offload_chunksize=64, num_primary_cache_pages=64,
            num_buffer_pages=16, host_capacity_per_layer=16 * 2 * 64 * 128 * item, max_batch_size=4, max_seq_len=1024,
            dtype=dtype, device=device))
    return cfg, model, kvm


def _run(device, dtype, tol):
    cfg, model, kvm = _setup(device, dtype)
    g = torch.Generator().manual_seed(1)
    users = torch.tensor([3, 5])
    hist1, hist2, ncand = torch.tensor([150, 70]), torch.tensor([200, 100]), torch.tensor([7, 4])
    full = [torch.randn(int(h), cfg.d_model, generator=g) * 0.5 for h in hist2]
    cands = [torch.randn(int(n), cfg.d_model, generator=g) * 0.5 for n in ncand]
    ts_hist = [torch.sort(torch.randint(0, 100000, (int(h),), generator=g)).values.float() for h in hist2]

    def pack(lo, hi, with_c):
        xs, ts = [], []
        for b in range(2):
            xs.append(full[b][int(lo[b]):int(hi[b])])
            if with_c:
                xs.append(cands[b])
        return torch.cat(xs).to(device=device, dtype=dtype)

    def tstamps(hi, nc):
        out = []
        for b in range(2):
            out.append(ts_hist[b][: int(hi[b])])
            out.append(ts_hist[b][int(hi[b]) - 1].repeat(int(nc[b])) + 1)
        return torch.cat(out).to(device)

    zero = torch.zeros(2, dtype=torch.long)
    # cold: everything in one request
    cold = HSTURanker(model, kvm())
    ref = cold.rank(users, hist2, ncand, pack(zero, hist2, True), tstamps(hist2, ncand)).float().cpu()
    # warm: first request caches hist1 (no candidates), user 3's device copy is dropped, second sends only the tail
    kv = kvm()
    warm = HSTURanker(model, kv)
    none = torch.zeros(2, dtype=torch.long)
    warm.rank(users, hist1, none, pack(zero, hist1, False), tstamps(hist1, none))
    kv.offload_try_wait()
    assert kv.host.lookup_kvcache(kv.host.build_index_meta(users, hist1))[1].tolist() == [128, 64]
    kv.evict(torch.tensor([3]), for_npu=True, for_host=False)
    cached = warm.plan(users, hist2)
    assert cached.tolist() == [128, 70]
    got = warm.rank(users, hist2, ncand, pack(cached, hist2, True), tstamps(hist2, ncand)).float().cpu()
    assert kv.stats["onboarded_tokens"] == 128
    assert got.shape == (11,)
    assert torch.allclose(got, ref, atol=tol, rtol=tol), (got - ref).abs().max()
    # candidates left the cache again
    assert kv.gpu.lookup(users)[1].tolist() == [200, 100]


def test_warm_equals_cold_cpu():
    _run("cpu", torch.float32, 1e-4)


@pytest.mark.gpu
def test_warm_equals_cold_gpu():
    _run("cuda", torch.bfloat16, 3e-2)

"""KV-cache manager lifecycle of one user over two requests (the worked example of the reference's
``inference/kvcache_manager/docs/codeview.md``: page 32, chunk 128): request 1 caches 300 tokens, the two full chunks are
offloaded to the host tier, the device copy is evicted, request 2 (440 tokens) brings the 256-token prefix back from the
host while the model only computes the 184 new tokens.

    python examples/kvcache_lifecycle.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from recsdk_b200.inference import HostKVTaskStatus, KVCacheConfig, KVCacheManager  # noqa: E402


def main() -> int:
    cuda = torch.cuda.is_available()
    device, dtype = ("cuda", torch.bfloat16) if cuda else ("cpu", torch.float32)
    item = 2 if cuda else 4
    L, H, D = 2, 2, 64
    cfg = KVCacheConfig(num_layers=L, num_heads=H, head_dim=D, page_size=32, offload_chunksize=128, num_primary_cache_pages=24,
                        num_buffer_pages=8, host_capacity_per_layer=6 * 2 * 128 * H * D * item, max_batch_size=4, max_seq_len=1024,
                        dtype=dtype, device=device)
    m = KVCacheManager.from_config(cfg)
    user = torch.tensor([7])

    # ---- request 1: 300 tokens, nothing cached
    meta, look = m.lookup_kvcache(user, torch.tensor([300]))
    md = m.allocate_kvcache(meta, look)                               # pages for 300 tokens, packed metadata on the device
    assert m.onboard_launch(meta, look, md).status == HostKVTaskStatus.SKIPPED
    for layer in range(L):
        k = torch.randn(md.new_history_nnz, H, D, device=device, dtype=dtype)
        v = torch.randn(md.new_history_nnz, H, D, device=device, dtype=dtype)
        m.gpu.append_kvcache(layer, k, v, md)                         # ... the layer's paged attention would run here
    m.offload_launch(meta, md)                                        # full chunks that only live on the device -> host tier
    print("offload:", m.offload_try_wait().status.value, "- host now holds", m.host.lookup_kvcache(meta)[1].tolist(), "tokens")

    # ---- the device needs room: the user's pages go away, the host copy stays
    m.evict(user, for_npu=True, for_host=False)

    # ---- request 2: 440 tokens, 256 of them come back from the host
    meta, look = m.lookup_kvcache(user, torch.tensor([440]))
    md = m.allocate_kvcache(meta, look)
    handle = m.onboard_launch(meta, look, md)                         # host -> device, layer by layer, on side streams
    for layer in range(L):
        if cuda:
            handle.stream_wait_layer(layer)                           # only this layer's rows have to be there
        k = torch.randn(md.new_history_nnz, H, D, device=device, dtype=dtype)
        v = torch.randn(md.new_history_nnz, H, D, device=device, dtype=dtype)
        m.gpu.append_kvcache(layer, k, v, md)
    status = m.onboard_wait(handle).status
    print("request 2: cached %d, computed %d new tokens, onboard %s" % (int(look.cached_lengths[0]), md.new_history_nnz, status.value))
    return md.new_history_nnz


if __name__ == "__main__":
    main()

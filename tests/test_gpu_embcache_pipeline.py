"""The asynchronous embcache pipeline on the GPU: results equal the synchronous swap, host updates go through pinned
staging buffers, and the swap traffic of batch i+1 (memcpy stream) overlaps the forward / backward of batch i."""
import numpy as np
import pytest
import torch

from recsdk_b200.embcache import (EmbCacheEmbeddingBagCollection, EmbCacheEmbeddingBagConfig,
                                  EmbCacheShardedEmbeddingBagCollection, EmbCacheTrainPipelineSparseDist)
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


class _Batch:
    def __init__(self, k):
        self.sparse_features = k

    def to(self, device, non_blocking=False):
        return _Batch(self.sparse_features.to(device, non_blocking=non_blocking))

    def record_stream(self, stream):
        self.sparse_features.record_stream(stream)


class _Model(torch.nn.Module):
    def __init__(self, emb, width, burn=0):
        super().__init__()
        self.emb, self.burn = emb, burn
        self.w = torch.nn.Parameter(torch.randn(width, generator=torch.Generator().manual_seed(9)).to(DEV))
        self.a = torch.randn(2048, 2048, device=DEV)

    def forward(self, batch):
        x = self.emb(batch.sparse_features).values()
        loss = (x * self.w).sum(dim=1).pow(2).mean()
        for _ in range(self.burn):                        # dense work standing in for the rest of the model
            loss = loss + (self.a @ self.a).mean() * 0.0
        return loss, loss.detach()


def _make(rows, dim, cache, B, hot, burn=0):
    tabs = [EmbCacheEmbeddingBagConfig(num_embeddings=rows, embedding_dim=dim, name="t0", feature_names=["f0"]),
            EmbCacheEmbeddingBagConfig(num_embeddings=rows, embedding_dim=dim, name="t1", feature_names=["f1", "f2"])]
    ebc = EmbCacheEmbeddingBagCollection(tabs, 1, B, [hot, hot], device=DEV, embedding_optimizer_cls=torch.optim.Adagrad)
    emb = EmbCacheShardedEmbeddingBagCollection(ebc, ShardingEnv(1, 0, None), DEV, ebc.optimizer_spec(lr=0.1), cache_rows=cache)
    return _Model(emb, 3 * dim, burn)


def _batches(n, B, rows, seed, max_len=3):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        lens = torch.randint(1, max_len + 1, (3 * B,), generator=g)
        vals = torch.randint(0, rows, (int(lens.sum()),), generator=g)
        out.append(_Batch(KeyedJaggedTensor(["f0", "f1", "f2"], vals, lengths=lens).pin_memory()))
    return out


def _run(async_swap, steps=10):
    model = _make(rows=400, dim=16, cache=[120, 240], B=16, hot=3)
    opt = torch.optim.SGD([model.w], lr=0.01)
    pipe = EmbCacheTrainPipelineSparseDist(model, opt, "cpu", DEV, return_loss=True)
    assert pipe._async
    pipe._async = async_swap
    data = iter(_batches(steps, 16, 400, seed=3))
    losses = [float(pipe.progress(data)[0]) for _ in range(steps)]
    torch.cuda.synchronize()
    rows = model.emb.host_rows("t1", list(range(400)))
    return losses, rows, model.emb.stats


def test_async_swap_equals_synchronous_swap():
    la, ra, sa = _run(True)
    lb, rb, sb = _run(False)
    assert sa["swap_out"] > 0 and sa == sb
    assert la == lb                                        # same kernels in the same order on the same rows: bit-equal
    assert torch.equal(ra, rb)


def test_swap_traffic_overlaps_compute():
    """Device-side evidence of the overlap: with a dense model part that outlasts the host-side planning, the swap traffic
    of batch i+1 (memcpy stream: gather, D2H, H2D, scatter) runs while the compute stream is still inside step i, and is
    over before step i ends - the compute stream meets the memcpy stream only at the lookup of the next step."""
    B, rows, dim, steps = 2048, 200_000, 64, 10
    model = _make(rows=rows, dim=dim, cache=[3 * 3 * B, 2 * 3 * 3 * B], B=B, hot=3, burn=400)
    model.emb.record_timing = True
    opt = torch.optim.SGD([model.w], lr=0.01)
    pipe = EmbCacheTrainPipelineSparseDist(model, opt, "cpu", DEV, return_loss=True)
    assert pipe._async
    data = iter(_batches(steps + 1, B, rows, seed=5))
    begin, end = [], []
    for _ in range(steps):
        b = torch.cuda.Event(enable_timing=True)
        b.record()
        pipe.progress(data)                     # enqueues step i, then plans and enqueues the swap of batch i+1
        e = torch.cuda.Event(enable_timing=True)
        e.record()                              # compute stream: end of step i (the fetch adds nothing to this stream)
        begin.append(b)
        end.append(e)
    torch.cuda.synchronize()
    assert model.emb.stats["swap_out"] > 0
    spans = {b: (t0, t1) for b, t0, t1 in model.emb.swap_events}      # keyed by swap_step (1 = first batch)
    hidden = 0
    for i in range(3, steps - 1):               # steady state: the cache is full, every batch swaps
        t0, t1 = spans[i + 2]                   # the swap of batch i+1, planned during step i
        step_ms = begin[i].elapsed_time(end[i])
        swap_ms = t0.elapsed_time(t1)
        started_inside = begin[i].elapsed_time(t0) >= 0.0 and t0.elapsed_time(end[i]) > 0.0
        ended_inside = t1.elapsed_time(end[i]) > 0.0
        print("step %d: compute %.2f ms, swap of the next batch %.2f ms, inside the step: begin %s end %s"
              % (i, step_ms, swap_ms, started_inside, ended_inside))
        hidden += int(started_inside and ended_inside)
    assert hidden >= (steps - 4) - 1, hidden   # every steady-state swap (one straggler allowed) ran beside compute

"""The pipelines emit profiler ranges under the stage names of the reference's pipelines, so a trace of a migrated job
reads the same (reference: ``hybrid_train_pipeline.py:282-521``, ``torchrec_embcache/distributed/train_pipeline.py``)."""
import torch
from torch.profiler import ProfilerActivity, profile

from recsdk_b200.embcache import (EmbCacheEmbeddingBagCollection, EmbCacheEmbeddingBagConfig, EmbCacheShardedEmbeddingBagCollection,
                                  EmbCacheTrainPipelineSparseDist)
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.parallel.train_pipeline import TrainPipelineBase
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor


class _B:
    def __init__(self, k):
        self.sparse_features = k

    def to(self, device, non_blocking=False):
        return self


def _names(prof):
    return {e.name for e in prof.events() if e.name.startswith("## ")}


def test_base_pipeline_ranges():
    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.l = torch.nn.Linear(4, 1)

        def forward(self, b):
            loss = self.l(b.x).pow(2).mean()
            return loss, loss.detach()

    class XB:
        def __init__(self):
            self.x = torch.randn(8, 4)

        def to(self, device, non_blocking=False):
            return self

    m = M()
    pipe = TrainPipelineBase(m, torch.optim.SGD(m.parameters(), lr=0.1), torch.device("cpu"))
    with profile(activities=[ProfilerActivity.CPU]) as prof:
        pipe.progress(iter([XB()]))
    assert {"## zero_grad ##", "## forward ##", "## backward ##", "## optimizer ##"} <= _names(prof)


def test_embcache_pipeline_ranges():
    tables = [EmbCacheEmbeddingBagConfig(num_embeddings=100, embedding_dim=8, name="t0", feature_names=["f0"])]
    ebc = EmbCacheEmbeddingBagCollection(tables, 1, 4, [2], device="cpu")
    emb = EmbCacheShardedEmbeddingBagCollection(ebc, ShardingEnv(1, 0, None), "cpu", ebc.optimizer_spec(lr=0.1), cache_rows=[16])

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = emb
            self.w = torch.nn.Parameter(torch.ones(8))

        def forward(self, b):
            loss = (self.emb(b.sparse_features).values() * self.w).sum()
            return loss, loss.detach()

    m = M()
    g = torch.Generator().manual_seed(0)
    data = iter([_B(KeyedJaggedTensor(["f0"], torch.randint(0, 50, (8,), generator=g), lengths=torch.full((4,), 2)))
                 for _ in range(3)])
    pipe = EmbCacheTrainPipelineSparseDist(m, torch.optim.SGD([m.w], lr=0.1), "cpu", "cpu", evict_step_interval=None)
    with profile(activities=[ProfilerActivity.CPU]) as prof:
        for _ in range(3):
            pipe.progress(data)
    assert {"## get_next_batch ##", "## copy_batch_to_gpu ##", "## zero_grad ##", "## forward ##", "## backward ##",
            "## optimizer ##"} <= _names(prof)

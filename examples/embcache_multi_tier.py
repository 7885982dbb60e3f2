"""Multi-tier embedding tables: a small device cache in front of a large host table, rows swapped in and out by the
pipeline one batch ahead of the compute, feature admission, save and (incremental) load
(user flow of the reference's ``torchrec_embcache`` package: ``distributed/embedding_bag.py:229-258`` module,
``distributed/train_pipeline.py:226-293`` pipeline, ``saver.py:31-171``).

    python examples/embcache_multi_tier.py
"""
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from recsdk_b200.embcache import (AdmitAndEvictConfig, EmbCacheEmbeddingBagCollection, EmbCacheEmbeddingBagConfig,  # noqa: E402
                                  EmbCacheShardedEmbeddingBagCollection, EmbCacheTrainPipelineSparseDist, Saver)
from recsdk_b200.parallel.comm import ShardingEnv  # noqa: E402
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor  # noqa: E402


class Batch:
    def __init__(self, sparse_features):
        self.sparse_features = sparse_features

    def to(self, device, non_blocking=False):
        return Batch(self.sparse_features.to(device)) if torch.device(device).type != "cpu" else self

    def record_stream(self, stream):
        pass

    def pin_memory(self):
        return self


class Model(torch.nn.Module):
    def __init__(self, emb, width):
        super().__init__()
        self.emb = emb
        self.w = torch.nn.Parameter(torch.randn(width, generator=torch.Generator().manual_seed(9)) * 0.1)

    def forward(self, batch):
        pooled = self.emb(batch.sparse_features).values().float()
        loss = (pooled * self.w.to(pooled.device)).sum(dim=1).pow(2).mean()
        return loss, loss.detach()


def main() -> float:
    device = "cuda" if torch.cuda.is_available() else "cpu"
    B = 16
    tables = [EmbCacheEmbeddingBagConfig(num_embeddings=100_000, embedding_dim=8, name="t0", feature_names=["f0"],
                                         admit_and_evict_config=AdmitAndEvictConfig(admit_threshold=2, not_admitted_default_value=0.0)),
              EmbCacheEmbeddingBagConfig(num_embeddings=50_000, embedding_dim=16, name="t1", feature_names=["f1", "f2"])]
    ebc = EmbCacheEmbeddingBagCollection(tables, 1, B, [3, 3], device=device)
    # device cache of 256 / 512 rows in front of host tables of 100,000 / 50,000 rows
    emb = EmbCacheShardedEmbeddingBagCollection(ebc, ShardingEnv(1, 0, None), device, ebc.optimizer_spec(lr=0.1), cache_rows=[256, 512])
    model = Model(emb, 8 + 16 + 16)
    opt = torch.optim.SGD([model.w], lr=0.01)
    pipe = EmbCacheTrainPipelineSparseDist(model, opt, "cpu", device, return_loss=True)

    g = torch.Generator().manual_seed(1)

    def batch():
        lens = torch.randint(1, 4, (3 * B,), generator=g)
        return Batch(KeyedJaggedTensor(["f0", "f1", "f2"], torch.randint(0, 2000, (int(lens.sum()),), generator=g), lengths=lens))

    data = iter([batch() for _ in range(20)])
    loss = None
    for step in range(20):
        loss, _ = pipe.progress(data)
    with tempfile.TemporaryDirectory() as d:
        saver = Saver()
        saver.save(emb, os.path.join(d, "ckpt"))
        latest = Saver.get_latest_load_path(os.path.join(d, "ckpt")) or os.path.join(d, "ckpt")
        ebc2 = EmbCacheEmbeddingBagCollection(tables, 1, B, [3, 3], device=device)
        emb2 = EmbCacheShardedEmbeddingBagCollection(ebc2, ShardingEnv(1, 0, None), device, ebc2.optimizer_spec(lr=0.1), cache_rows=[256, 512])
        saver.load(emb2, latest)
    print("loss after 20 pipelined steps: %.5f; checkpoint written and loaded into a fresh module" % float(loss))
    return float(loss)


if __name__ == "__main__":
    main()

"""Multi-tier embedding tables: device-memory cache of hot rows over a host-DRAM table, admission / eviction."""
from .configs import (POLICY_COUNT, POLICY_SHOW_CLICK, AdmitAndEvictConfig, AdmitAndEvictPolicyType, EmbCacheEmbeddingBagConfig, EmbCacheEmbeddingConfig,
                      InitializerType, ShowClickParams)
from .embedding_bag import (CacheKernelView, EmbCacheEmbeddingBagCollection, EmbCacheEmbeddingBagCollectionSharder,
                            EmbCacheHashTable, EmbCacheShardedEmbeddingBagCollection, calculate_caches)
from .embedding import EmbCacheEmbeddingCollection, EmbCacheEmbeddingCollectionSharder, EmbCacheShardedEmbeddingCollection
from .restore import RestoreTask, restore, restore_async
from .saver import Saver
from .train_pipeline import EmbCacheTrainPipelineSparseDist

__all__ = ["POLICY_COUNT", "POLICY_SHOW_CLICK", "AdmitAndEvictConfig", "AdmitAndEvictPolicyType", "EmbCacheEmbeddingBagConfig", "EmbCacheEmbeddingConfig",
           "InitializerType", "ShowClickParams", "EmbCacheEmbeddingBagCollection", "EmbCacheEmbeddingBagCollectionSharder",
           "EmbCacheShardedEmbeddingBagCollection", "calculate_caches", "EmbCacheEmbeddingCollection", "EmbCacheEmbeddingCollectionSharder",
           "EmbCacheShardedEmbeddingCollection", "Saver", "EmbCacheTrainPipelineSparseDist", "RestoreTask", "restore", "restore_async", "CacheKernelView", "EmbCacheHashTable"]

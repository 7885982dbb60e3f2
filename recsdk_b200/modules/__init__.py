"""Embedding table configurations and the unsharded collections (plain and hash-mapped)."""
from .embedding_configs import (BaseEmbeddingConfig, DataType, EmbeddingBagConfig, EmbeddingConfig, PoolingType, data_type_to_dtype,
                                dtype_to_data_type, validate_hash_table_config)
from .embedding_modules import EmbeddingBagCollection, EmbeddingCollection, TableDict
from .ids_process import BucketParams, HashMapBase, IdsMapper, block_bucketize_sparse_features_cpu
from .hash_embeddingbag import EvictStrategy, HashEmbeddingBagCollection, HashEmbeddingBagConfig, HashTableOption, HybridHashTable

__all__ = ["BaseEmbeddingConfig", "DataType", "EmbeddingBagConfig", "EmbeddingConfig", "PoolingType", "data_type_to_dtype",
           "dtype_to_data_type", "validate_hash_table_config", "EmbeddingBagCollection", "EmbeddingCollection", "TableDict", "EvictStrategy",
           "HashEmbeddingBagCollection", "HashEmbeddingBagConfig", "HashTableOption", "HybridHashTable", "BucketParams", "HashMapBase", "IdsMapper",
           "block_bucketize_sparse_features_cpu"]

"""Dynamic (hash-table backed) embeddings: the ``dynamic_emb`` API surface on the GPU hash table."""
from .batched_dynamicemb_table import BatchedDynamicEmbeddingTablesV2
from .dump_load import DynamicEmbDump, DynamicEmbLoad, get_score, incremental_dump, set_score
from .dynamicemb_config import (DynamicEmbCheckMode, DynamicEmbInitializerArgs, DynamicEmbInitializerMode,
                                DynamicEmbPoolingMode, DynamicEmbScoreStrategy, DynamicEmbTableOptions, EmbOptimType,
                                convert_optimizer_type, get_constraint_capacity)
from .embedding import DynamicEmbeddingBagCollection, DynamicEmbeddingCollection
from .hkv import EvictStrategy, HKVTable, HostDynamicTable, InitializerArgs, InitMode, OptimizerType
from .key_value_table import DiskStorage, KeyValueTable, Storage, TableStorage
from .planner import (DynamicEmbeddingBagCollectionSharder, DynamicEmbeddingCollectionSharder, DynamicEmbeddingEnumerator,
                      DynamicEmbeddingShardingPlanner, DynamicEmbParameterConstraints, DynamicEmbParameterSharding, ShardingOption)
from .construct_twin_module import ConstructTwinModule, StaticTwin, generate_sparse_feature

__version__ = "v25.09"          # the API level of the dynamic-embedding surface this package follows

__all__ = [
    "DynamicEmbeddingEnumerator", "ShardingOption", "ConstructTwinModule", "StaticTwin", "generate_sparse_feature",
    "BatchedDynamicEmbeddingTablesV2", "DynamicEmbDump", "DynamicEmbLoad", "get_score", "incremental_dump", "set_score",
    "DynamicEmbCheckMode", "DynamicEmbInitializerArgs", "DynamicEmbInitializerMode", "DynamicEmbPoolingMode",
    "DynamicEmbScoreStrategy", "DynamicEmbTableOptions", "EmbOptimType", "convert_optimizer_type",
    "get_constraint_capacity", "DynamicEmbeddingBagCollection", "DynamicEmbeddingCollection", "EvictStrategy", "HKVTable",
    "HostDynamicTable", "InitializerArgs", "InitMode", "OptimizerType", "DiskStorage", "KeyValueTable", "Storage",
    "TableStorage", "DynamicEmbeddingBagCollectionSharder", "DynamicEmbeddingCollectionSharder", "DynamicEmbeddingShardingPlanner",
    "DynamicEmbParameterConstraints", "DynamicEmbParameterSharding",
]

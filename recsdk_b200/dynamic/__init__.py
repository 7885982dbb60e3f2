"""Dynamic (hash-table backed) embeddings: the ``dynamic_emb`` API surface on the GPU hash table."""
from .batched_dynamicemb_table import (BatchedDynamicEmbeddingTablesV2, DynamicEmbeddingBagFunction, DynamicEmbeddingFunctionV2,
                                       dynamicemb_prefetch)
from .dump_load import (DynamicEmbDump, DynamicEmbLoad, check_emb_collection_modules, find_dynamic_modules, find_sharded_modules,
                        get_dynamic_emb_module, get_score, incremental_dump, set_score)
from .dynamicemb_config import (DynamicEmbCheckMode, DynamicEmbInitializerArgs, DynamicEmbInitializerMode,
                                DynamicEmbPoolingMode, DynamicEmbScoreStrategy, DynamicEmbTableOptions, EmbOptimType,
                                convert_optimizer_type, get_constraint_capacity, aligned_capacity_per_rank, DistType,
                                DynamicEmbDataType, DynamicEmbEvictStrategy, create_dynamicemb_table, dtype_to_bytes, dyn_emb_to_torch,
                                get_optimizer_state_dim, next_power_of_2, torch_to_dyn_emb, validate_initializer_args)
from .embedding import DynamicEmbeddingBagCollection, DynamicEmbeddingCollection
from .hkv import EvictStrategy, HKVTable, HostDynamicTable, InitializerArgs, InitMode, OptimizerType
from .key_value_table import (Cache, DiskStorage, KeyValueTable, KeyValueTableCachingFunction, KeyValueTableFunction, Storage, TableStorage,
                              encode_checkpoint_file_path, encode_meta_json_file_path, find_files, update_cache)
from .planner import (DynamicEmbeddingBagCollectionSharder, DynamicEmbeddingCollectionSharder, DynamicEmbeddingEnumerator,
                      DynamicEmbeddingShardingPlanner, DynamicEmbParameterConstraints, DynamicEmbParameterSharding, ShardingOption)
from .construct_twin_module import ConstructTwinModule, StaticTwin, generate_sparse_feature
from .initializers import (BaseDynamicEmbInitializer, ConstantInitializer, DebugInitializer, NormalInitializer, TruncatedNormalInitializer,
                           UniformInitializer, create_initializer)
from .optimizers import (AdagradDynamicEmbeddingOptimizer, AdagradDynamicEmbeddingOptimizerV2, AdamDynamicEmbeddingOptimizer,
                         AdamDynamicEmbeddingOptimizerV2, BaseDynamicEmbeddingOptimizer, BaseDynamicEmbeddingOptimizerV2, OptimizerArgs,
                         RowWiseAdagradDynamicEmbeddingOptimizer, RowWiseAdagradDynamicEmbeddingOptimizerV2, SGDDynamicEmbeddingOptimizer,
                         SGDDynamicEmbeddingOptimizerV2, create_optimizer, get_required_arg, string_to_opt_type)

# names of the reference's sharded modules and of its no-op fused optimizer handle (the update runs inside the backward)
ShardedDynamicEmbeddingCollection = DynamicEmbeddingCollection
ShardedDynamicEmbeddingBagCollection = DynamicEmbeddingBagCollection
from ..optim import FusedOptimizerStub as DynamicEmbeddingFusedOptimizer  # noqa: E402

__version__ = "v25.09"          # the API level of the dynamic-embedding surface this package follows

__all__ = [
    "BaseDynamicEmbInitializer", "ConstantInitializer", "DebugInitializer", "NormalInitializer", "TruncatedNormalInitializer",
    "UniformInitializer", "create_initializer", "AdagradDynamicEmbeddingOptimizer", "AdagradDynamicEmbeddingOptimizerV2",
    "AdamDynamicEmbeddingOptimizer", "AdamDynamicEmbeddingOptimizerV2", "BaseDynamicEmbeddingOptimizer", "BaseDynamicEmbeddingOptimizerV2",
    "OptimizerArgs", "RowWiseAdagradDynamicEmbeddingOptimizer", "RowWiseAdagradDynamicEmbeddingOptimizerV2", "SGDDynamicEmbeddingOptimizer",
    "SGDDynamicEmbeddingOptimizerV2", "create_optimizer", "get_required_arg", "string_to_opt_type",
    "DynamicEmbeddingBagFunction", "DynamicEmbeddingFunctionV2", "dynamicemb_prefetch", "check_emb_collection_modules", "find_dynamic_modules",
    "find_sharded_modules", "get_dynamic_emb_module", "Cache", "KeyValueTableCachingFunction", "KeyValueTableFunction", "encode_checkpoint_file_path", "encode_meta_json_file_path", "find_files",
    "update_cache", "ShardedDynamicEmbeddingCollection", "ShardedDynamicEmbeddingBagCollection", "DynamicEmbeddingFusedOptimizer",
    "aligned_capacity_per_rank", "DistType", "DynamicEmbDataType", "DynamicEmbEvictStrategy", "create_dynamicemb_table", "dtype_to_bytes",
    "dyn_emb_to_torch", "get_optimizer_state_dim", "next_power_of_2", "torch_to_dyn_emb", "validate_initializer_args",
    "DynamicEmbeddingEnumerator", "ShardingOption", "ConstructTwinModule", "StaticTwin", "generate_sparse_feature",
    "BatchedDynamicEmbeddingTablesV2", "DynamicEmbDump", "DynamicEmbLoad", "get_score", "incremental_dump", "set_score",
    "DynamicEmbCheckMode", "DynamicEmbInitializerArgs", "DynamicEmbInitializerMode", "DynamicEmbPoolingMode",
    "DynamicEmbScoreStrategy", "DynamicEmbTableOptions", "EmbOptimType", "convert_optimizer_type",
    "get_constraint_capacity", "DynamicEmbeddingBagCollection", "DynamicEmbeddingCollection", "EvictStrategy", "HKVTable",
    "HostDynamicTable", "InitializerArgs", "InitMode", "OptimizerType", "DiskStorage", "KeyValueTable", "Storage",
    "TableStorage", "DynamicEmbeddingBagCollectionSharder", "DynamicEmbeddingCollectionSharder", "DynamicEmbeddingShardingPlanner",
    "DynamicEmbParameterConstraints", "DynamicEmbParameterSharding",
]

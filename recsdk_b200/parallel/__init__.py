"""Sharding, planning, collectives and training pipelines."""
from .comm import PeerGroup, ShardingEnv
from .embeddingbag import ParameterSharding, ShardedEmbeddingBagCollection
from .collective_embeddingbag import CollectiveShardedEmbeddingBagCollection
from .hybrid import (HybridEmbeddingBagCollectionSharder, HybridHashEmbeddingBagCollectionSharder, HybridPipelineContext,
                     HybridShardedEmbeddingBagCollection, HybridShardedHashEmbeddingBagCollection, HybridStage, HybridTrainPipelineContext,
                     HybridTrainPipelineSparseDist, TaskType, get_default_hybrid_sharders)
from .lccl import lccl_all_to_all, lccl_all_uss, lccl_gather_all, unsorted_segment_sum
from .model_parallel import DistributedModelParallel
from .planner import EmbeddingShardingPlanner, ParameterConstraints, ShardingPlan, Topology
from .train_pipeline import TrainPipelineBase, TrainPipelineSparseDist

__all__ = ["PeerGroup", "ShardingEnv", "ParameterSharding", "ShardedEmbeddingBagCollection", "CollectiveShardedEmbeddingBagCollection",
           "HybridEmbeddingBagCollectionSharder", "HybridHashEmbeddingBagCollectionSharder", "HybridTrainPipelineSparseDist",
           "HybridPipelineContext", "HybridShardedEmbeddingBagCollection", "HybridShardedHashEmbeddingBagCollection", "HybridStage",
           "HybridTrainPipelineContext", "TaskType", "get_default_hybrid_sharders", "DistributedModelParallel", "EmbeddingShardingPlanner", "ParameterConstraints", "ShardingPlan",
           "Topology", "TrainPipelineBase", "TrainPipelineSparseDist", "lccl_all_to_all", "lccl_all_uss", "lccl_gather_all",
           "unsorted_segment_sum"]

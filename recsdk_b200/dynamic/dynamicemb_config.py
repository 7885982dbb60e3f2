"""Options of dynamic (hash-table backed) embedding tables.

Field names and defaults follow the reference (``dynamic_emb/distributed/dynamicemb_config.py:56-546``):
``DynamicEmbTableOptions`` user fields (training, initializer_args, eval_initializer_args, init_capacity ->
power of two, max_load_factor 0.5, score_strategy, bucket_capacity 128 in [16, 1024] and a power of two,
safe_check_mode, global_hbm_for_values, caching, external_storage, index_type) and the context fields
filled in by the planner / sharder (dim, max_capacity, evict_strategy, local_hbm_for_values, optimizer_type...).
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Any, Optional

import torch

from .hkv import EvictStrategy, InitializerArgs, InitMode, OptimizerType


class DynamicEmbInitializerMode(enum.Enum):
    NORMAL = "normal"
    TRUNCATED_NORMAL = "truncated_normal"
    UNIFORM = "uniform"
    CONSTANT = "constant"
    DEBUG = "debug"


class DynamicEmbScoreStrategy(enum.IntEnum):
    TIMESTAMP = 0     # LRU: device timestamp on every access
    STEP = 1          # customized: global step counter
    CUSTOMIZED = 2    # customized: user-set score (set_score)
    LFU = 3           # access count


class DynamicEmbCheckMode(enum.IntEnum):
    ERROR = 0
    WARNING = 1
    IGNORE = 2


class DynamicEmbPoolingMode(enum.IntEnum):
    SUM = 0
    MEAN = 1
    NONE = 2


class EmbOptimType(enum.Enum):
    SGD = "sgd"
    EXACT_SGD = "exact_sgd"
    ADAM = "adam"
    EXACT_ADAGRAD = "exact_adagrad"
    EXACT_ROWWISE_ADAGRAD = "exact_row_wise_adagrad"
    ADAMW = "adamw"
    LARS_SGD = "lars_sgd"
    PARTIAL_ROWWISE_ADAM = "partial_row_wise_adam"


def convert_optimizer_type(t: EmbOptimType) -> OptimizerType:
    """ADAMW / LARS / partial row-wise Adam are rejected, as in the reference's optimizer factory."""
    m = {EmbOptimType.SGD: OptimizerType.SGD, EmbOptimType.EXACT_SGD: OptimizerType.SGD, EmbOptimType.ADAM: OptimizerType.ADAM,
         EmbOptimType.EXACT_ADAGRAD: OptimizerType.ADAGRAD, EmbOptimType.EXACT_ROWWISE_ADAGRAD: OptimizerType.ROWWISE_ADAGRAD}
    if t not in m:
        raise ValueError("optimizer %s is not supported by dynamic embedding tables" % t)
    return m[t]


_MODE = {DynamicEmbInitializerMode.NORMAL: InitMode.NORMAL, DynamicEmbInitializerMode.TRUNCATED_NORMAL: InitMode.TRUNCATED_NORMAL,
         DynamicEmbInitializerMode.UNIFORM: InitMode.UNIFORM, DynamicEmbInitializerMode.CONSTANT: InitMode.CONSTANT,
         DynamicEmbInitializerMode.DEBUG: InitMode.DEBUG}


@dataclasses.dataclass
class DynamicEmbInitializerArgs:
    mode: DynamicEmbInitializerMode = DynamicEmbInitializerMode.UNIFORM
    mean: float = 0.0
    std_dev: float = 1.0
    lower: Optional[float] = None
    upper: Optional[float] = None
    value: float = 0.0

    def to_native(self, num_embeddings_hint: int = 0, seed: int = 0) -> InitializerArgs:
        lo, hi = self.lower, self.upper
        if lo is None or hi is None:
            b = (1.0 / max(num_embeddings_hint, 1)) ** 0.5 if num_embeddings_hint else 0.01
            lo, hi = (-b if lo is None else lo), (b if hi is None else hi)
        return InitializerArgs(mode=_MODE[self.mode], lower=lo, upper=hi, mean=self.mean, std_dev=self.std_dev,
                               value=self.value, seed=seed)


def _pow2_ceil(x: int) -> int:
    p = 1
    while p < x:
        p <<= 1
    return p


@dataclasses.dataclass
class DynamicEmbTableOptions:
    # ---- user fields
    training: bool = True
    initializer_args: DynamicEmbInitializerArgs = dataclasses.field(default_factory=DynamicEmbInitializerArgs)
    eval_initializer_args: DynamicEmbInitializerArgs = dataclasses.field(
        default_factory=lambda: DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.CONSTANT, value=0.0))
    init_capacity: Optional[int] = None
    max_load_factor: float = 0.5
    score_strategy: DynamicEmbScoreStrategy = DynamicEmbScoreStrategy.TIMESTAMP
    bucket_capacity: int = 128
    safe_check_mode: DynamicEmbCheckMode = DynamicEmbCheckMode.IGNORE
    global_hbm_for_values: int = 0
    caching: bool = False
    external_storage: Any = None
    index_type: torch.dtype = torch.int64
    admit_threshold: int = 0          # > 0: a key becomes resident on its admit_threshold-th sighting
    # ---- context fields (planner / sharder)
    score_type: torch.dtype = torch.int64
    embedding_dtype: torch.dtype = torch.float32
    dim: int = 0
    max_capacity: int = 0
    evict_strategy: Optional[EvictStrategy] = None
    local_hbm_for_values: int = 0
    num_aligned_embedding_per_rank: int = 0
    device_id: int = -1
    optimizer_type: OptimizerType = OptimizerType.SGD
    block_size: int = 128
    io_block_size: int = 1024
    io_by_cpu: bool = False
    use_constant_memory: bool = False
    reserved_key_start_bit: int = 0
    num_of_buckets_per_alloc: int = 1

    def __post_init__(self) -> None:
        if self.eval_initializer_args.mode != DynamicEmbInitializerMode.CONSTANT:
            raise ValueError("eval_initializer_args supports CONSTANT only")
        if not (16 <= self.bucket_capacity <= 1024) or self.bucket_capacity & (self.bucket_capacity - 1):
            raise ValueError("bucket_capacity must be a power of two in [16, 1024]")
        if not (0.0 < self.max_load_factor <= 1.0):
            raise ValueError("max_load_factor must be in (0, 1]")
        if self.index_type not in (torch.int64, torch.uint64):
            raise ValueError("index_type must be int64 or uint64")
        if self.init_capacity is not None:
            self.init_capacity = _pow2_ceil(max(int(self.init_capacity), self.bucket_capacity))
        if self.evict_strategy is None:
            self.evict_strategy = {DynamicEmbScoreStrategy.TIMESTAMP: EvictStrategy.LRU,
                                   DynamicEmbScoreStrategy.STEP: EvictStrategy.CUSTOMIZED,
                                   DynamicEmbScoreStrategy.CUSTOMIZED: EvictStrategy.CUSTOMIZED,
                                   DynamicEmbScoreStrategy.LFU: EvictStrategy.LFU}[self.score_strategy]

    def grouping_key(self):
        """Tables with equal (training, caching, external_storage, index_type) may share one batched module."""
        return (self.training, self.caching, id(self.external_storage) if self.external_storage is not None else None,
                self.index_type)


def get_constraint_capacity(num_embeddings: int, world_size: int, bucket_capacity: int = 128) -> int:
    """Rows per rank, aligned up to a power of two and at least one bucket
    (``dynamic_emb/distributed/planner/planners.py:63-77``)."""
    per_rank = (num_embeddings + world_size - 1) // world_size
    return max(bucket_capacity, _pow2_ceil(per_rank))

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

    def as_ctype(self) -> InitializerArgs:
        """The native form with the reference's defaults for open bounds (0 and 1; ``dynamicemb_config.py:203-211``)."""
        return InitializerArgs(mode=_MODE[self.mode], lower=self.lower if self.lower else 0.0, upper=self.upper if self.upper else 1.0,
                               mean=self.mean, std_dev=self.std_dev, value=self.value)


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

    def get_grouped_key(self):
        return {"training": self.training, "caching": self.caching, "external_storage": self.external_storage,
                "index_type": self.index_type}

    def __hash__(self):
        return hash((self.training, self.caching, id(self.external_storage) if self.external_storage is not None else None,
                     self.index_type))

    def grouping_key(self):
        """Tables with equal (training, caching, external_storage, index_type) may share one batched module."""
        return (self.training, self.caching, id(self.external_storage) if self.external_storage is not None else None,
                self.index_type)


def aligned_capacity_per_rank(num_embeddings: int, world_size: int, bucket_capacity: int = 128) -> int:
    """Rows per rank, aligned up to a power of two and at least one bucket
    (``dynamic_emb/distributed/planner/planners.py:63-77``)."""
    per_rank = (num_embeddings + world_size - 1) // world_size
    return max(bucket_capacity, _pow2_ceil(per_rank))


# ----------------------------------------------------------------------------------------------------------------------
# Helpers with the reference's names (``dynamicemb_config.py:56-146``, ``:456-546``)
# ----------------------------------------------------------------------------------------------------------------------
class DynamicEmbDataType(enum.Enum):
    Float32 = "float32"
    BFloat16 = "bfloat16"
    Float16 = "float16"
    Int64 = "int64"
    UInt64 = "uint64"
    Int32 = "int32"
    Size_t = "size_t"


_DE_TO_TORCH = {DynamicEmbDataType.Float32: torch.float32, DynamicEmbDataType.BFloat16: torch.bfloat16, DynamicEmbDataType.Float16: torch.float16,
                DynamicEmbDataType.Int64: torch.int64, DynamicEmbDataType.UInt64: torch.uint64, DynamicEmbDataType.Int32: torch.int32,
                DynamicEmbDataType.Size_t: torch.int64}


def dyn_emb_to_torch(data_type: DynamicEmbDataType) -> torch.dtype:
    if data_type not in _DE_TO_TORCH:
        raise ValueError("Unsupported DynamicEmbDataType: %s" % (data_type,))
    return _DE_TO_TORCH[data_type]


def torch_to_dyn_emb(torch_dtype: torch.dtype) -> DynamicEmbDataType:
    for k, v in _DE_TO_TORCH.items():
        if v == torch_dtype and k is not DynamicEmbDataType.Size_t:
            return k
    raise ValueError("Unsupported torch dtype: %s" % (torch_dtype,))


def dtype_to_bytes(dtype: torch.dtype) -> int:
    if dtype == torch.bool:
        return 1
    try:
        return torch.empty(0, dtype=dtype).element_size()
    except (TypeError, RuntimeError) as e:
        raise ValueError("Unsupported dtype: %s" % (dtype,)) from e


class DynamicEmbEvictStrategy(enum.Enum):
    LRU = EvictStrategy.LRU
    LFU = EvictStrategy.LFU
    EPOCH_LRU = EvictStrategy.EPOCH_LRU
    EPOCH_LFU = EvictStrategy.EPOCH_LFU
    CUSTOMIZED = EvictStrategy.CUSTOMIZED


class DistType(enum.Enum):
    CONTINUOUS = "continuous"
    ROUNDROBIN = "roundrobin"


def next_power_of_2(n: int) -> int:
    return 1 if n <= 0 else _pow2_ceil(int(n))


def get_optimizer_state_dim(optimizer_type: OptimizerType, dim: int, dtype: torch.dtype = torch.float32) -> int:
    """Optimizer-state elements behind the embedding in a row: Adam 2 x dim, Adagrad dim, row-wise Adagrad 16 bytes."""
    optimizer_type = OptimizerType(optimizer_type)
    if optimizer_type == OptimizerType.ROWWISE_ADAGRAD:
        return 16 // dtype_to_bytes(dtype)
    if optimizer_type == OptimizerType.ADAM:
        return dim * 2
    if optimizer_type == OptimizerType.ADAGRAD:
        return dim
    return 0


def validate_initializer_args(initializer_args: DynamicEmbInitializerArgs, eb_config=None) -> None:
    """Fill the open bounds of a uniform initialiser: ``+-sqrt(1 / num_embeddings)`` with a table config, else ``[0, 1]``."""
    if initializer_args.mode == DynamicEmbInitializerMode.UNIFORM:
        b = (1.0 / eb_config.num_embeddings) ** 0.5 if eb_config is not None else None
        if initializer_args.lower is None:
            initializer_args.lower = -b if b is not None else 0.0
        if initializer_args.upper is None:
            initializer_args.upper = b if b is not None else 1.0


def get_constraint_capacity(memory_bytes: int, dtype: torch.dtype, dim: int, optimizer_type: OptimizerType, bucket_capacity: int) -> int:
    """Rows (embedding + optimizer state) that fit into ``memory_bytes``, rounded down to whole buckets; at least one bucket
    must fit (``dynamicemb_config.py:531-546`` of the reference)."""
    per_row = (dim + get_optimizer_state_dim(optimizer_type, dim, dtype)) * dtype_to_bytes(dtype)
    if memory_bytes < bucket_capacity * per_row:
        raise ValueError("reserved bytes %d are less than the size of one bucket %d" % (memory_bytes, bucket_capacity * per_row))
    return (memory_bytes // per_row // bucket_capacity) * bucket_capacity


def create_dynamicemb_table(table_options: DynamicEmbTableOptions, device: Optional[torch.device] = None, seed: int = 0):
    """The table handle of one set of options: the device hash table on CUDA (``device`` or ``device_id``), the
    dictionary-backed table otherwise.  A table that is not trained keeps no optimizer state
    (``dynamicemb_config.py:481-505`` of the reference)."""
    from .hkv import HKVTable, HostDynamicTable

    o = table_options
    if o.dim <= 0:
        raise ValueError("table options need dim > 0 (a context field the planner / sharder fills in)")
    opt = OptimizerType(o.optimizer_type) if o.training else OptimizerType.SGD
    cap = o.init_capacity or o.max_capacity or 1024
    max_cap = max(o.max_capacity or cap, cap)
    init = o.initializer_args.to_native(max_cap, seed)
    if device is None:
        device = torch.device("cuda", o.device_id) if (o.device_id >= 0 and torch.cuda.is_available()) else torch.device("cpu")
    device = torch.device(device)
    kw = dict(optimizer=opt, evict_strategy=o.evict_strategy, init=init)
    if device.type == "cuda":
        hbm_rows = None
        if o.local_hbm_for_values > 0:
            hbm_rows = max(128, int(o.local_hbm_for_values // (4 * (o.dim + opt_state_dim_of(opt, o.dim)))))
        return HKVTable(o.dim, cap, device, max_capacity=max_cap, max_load_factor=o.max_load_factor, hbm_rows=hbm_rows, **kw)
    return HostDynamicTable(o.dim, max_cap, **kw)


def opt_state_dim_of(opt: OptimizerType, dim: int) -> int:
    from .hkv import opt_state_dim

    return opt_state_dim(opt, dim)

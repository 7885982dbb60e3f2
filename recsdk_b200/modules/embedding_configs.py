"""Embedding table configuration dataclasses (TorchRec-compatible field names) and the validation
limits of the reference's hash tables (``hybrid_torchrec/constants.py:8-16``,
``hybrid_torchrec/modules/hash_embeddingbag.py:95-201``).
"""
from __future__ import annotations

import enum
import re
from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch


class PoolingType(enum.Enum):
    SUM = "SUM"
    MEAN = "MEAN"
    NONE = "NONE"


class DataType(enum.Enum):
    FP32 = "FP32"
    FP16 = "FP16"
    BF16 = "BF16"


_DT_TO_TORCH = {DataType.FP32: torch.float32, DataType.FP16: torch.float16, DataType.BF16: torch.bfloat16}


def data_type_to_dtype(dt: DataType) -> torch.dtype:
    return _DT_TO_TORCH[dt]


def dtype_to_data_type(dt: torch.dtype) -> DataType:
    for k, v in _DT_TO_TORCH.items():
        if v == dt:
            return k
    raise ValueError("unsupported embedding dtype %s" % dt)


@dataclass
class BaseEmbeddingConfig:
    num_embeddings: int
    embedding_dim: int
    name: str = ""
    data_type: DataType = DataType.FP32
    feature_names: List[str] = field(default_factory=list)
    weight_init_max: Optional[float] = None
    weight_init_min: Optional[float] = None
    init_fn: Optional[Callable[[torch.Tensor], Optional[torch.Tensor]]] = None

    def get_weight_init_max(self) -> float:
        if self.weight_init_max is None:
            return (1.0 / self.num_embeddings) ** 0.5
        return self.weight_init_max

    def get_weight_init_min(self) -> float:
        if self.weight_init_min is None:
            return -((1.0 / self.num_embeddings) ** 0.5)
        return self.weight_init_min

    def num_features(self) -> int:
        return len(self.feature_names)

    def __post_init__(self) -> None:
        if not self.feature_names:
            self.feature_names = [self.name]


@dataclass
class EmbeddingBagConfig(BaseEmbeddingConfig):
    pooling: PoolingType = PoolingType.SUM


@dataclass
class EmbeddingConfig(BaseEmbeddingConfig):
    pass


# limits of the hash-table variants -------------------------------------------------------------
MAX_EMBEDDING_DIM = 4096
MIN_EMBEDDING_DIM = 8
EMBEDDING_DIM_ALIGN = 8
MAX_NUM_EMBEDDINGS = 1_000_000_000
MAX_TABLES = 1024
_NAME_RE = re.compile(r"^[A-Za-z0-9_\-\.]{1,128}$")


def validate_hash_table_config(cfg: BaseEmbeddingConfig) -> None:
    """Checks applied to ``HashEmbeddingBagConfig`` tables: name charset/length, dim in [8, 4096] and a
    multiple of 8, rows in [1, 1e9], fp32 storage."""
    if not isinstance(cfg.name, str) or not _NAME_RE.match(cfg.name):
        raise ValueError("invalid table name %r" % (cfg.name,))
    if not (MIN_EMBEDDING_DIM <= cfg.embedding_dim <= MAX_EMBEDDING_DIM) or cfg.embedding_dim % EMBEDDING_DIM_ALIGN:
        raise ValueError("embedding_dim must be a multiple of %d in [%d, %d], got %d"
                         % (EMBEDDING_DIM_ALIGN, MIN_EMBEDDING_DIM, MAX_EMBEDDING_DIM, cfg.embedding_dim))
    if not (1 <= cfg.num_embeddings <= MAX_NUM_EMBEDDINGS):
        raise ValueError("num_embeddings must be in [1, %d], got %d" % (MAX_NUM_EMBEDDINGS, cfg.num_embeddings))
    if cfg.data_type != DataType.FP32:
        raise ValueError("hash embedding tables are fp32 only")
    for f in cfg.feature_names:
        if not isinstance(f, str) or not _NAME_RE.match(f):
            raise ValueError("invalid feature name %r" % (f,))

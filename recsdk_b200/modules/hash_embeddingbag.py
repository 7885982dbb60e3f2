"""``HashEmbeddingBagCollection``: embedding bags whose tables are addressed by raw 64-bit ids.

Each table owns a native ``IdsMapper`` (C++ open-addressing map) that assigns dense slots to ids in
first-seen order; the lookup then runs on slots.  Config validation follows the reference
(``hybrid_torchrec/modules/hash_embeddingbag.py:95-201,276-362``; limits ``constants.py:8-16``):
table/feature name charset, dim in [8, 4096] and a multiple of 8, at most 1e9 rows, fp32 storage,
pooling SUM / MEAN, ``is_weighted=False``.
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

from ..host import host
from ..sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor
from .embedding_configs import EmbeddingBagConfig, PoolingType, validate_hash_table_config
from .embedding_modules import EmbeddingBagCollection, TableDict, _init_table


class EvictStrategy(enum.Enum):
    kLru = 0
    kLfu = 1
    kEpochLru = 2
    kEpochLfu = 3
    kCustomized = 4


@dataclasses.dataclass
class HashTableOption:
    init_capacity: int = 0
    max_capacity: int = 0
    max_npu_memory_for_vectors: int = 0
    max_bucket_size: int = 128
    dim: int = 64
    max_load_factor: float = 0.5
    block_size: int = 128
    io_block_size: int = 1024
    device_id: int = -1
    io_by_cpu: bool = False


@dataclasses.dataclass
class HashEmbeddingBagConfig(EmbeddingBagConfig):
    """Same fields as ``EmbeddingBagConfig``; ``num_embeddings`` is the slot capacity of the table."""


class HybridHashTable(nn.Module):
    """One hash table: slot-addressed weight + the id -> slot mapper."""

    def __init__(self, cfg: EmbeddingBagConfig, device: torch.device) -> None:
        super().__init__()
        self.cfg = cfg
        self.weight = nn.Parameter(torch.empty(cfg.num_embeddings, cfg.embedding_dim, device=device))
        _init_table(self.weight.data, cfg)
        self.mapper = host().IdsMapper(cfg.num_embeddings) if device.type != "meta" else None

    def slots(self, ids: torch.Tensor) -> torch.Tensor:
        out = self.mapper.ids2indices(ids.detach().cpu().numpy().astype(np.int64))
        return torch.from_numpy(out).to(ids.device)


class HashEmbeddingBagCollection(EmbeddingBagCollection):
    def __init__(self, tables: List[EmbeddingBagConfig], is_weighted: bool = False,
                 device: Optional[torch.device] = None) -> None:
        if is_weighted:
            raise ValueError("HashEmbeddingBagCollection does not support weighted features")
        if not tables:
            raise ValueError("tables must not be empty")
        for t in tables:
            validate_hash_table_config(t)
            if t.pooling not in (PoolingType.SUM, PoolingType.MEAN, PoolingType.NONE):
                raise ValueError("unsupported pooling %s" % t.pooling)
        nn.Module.__init__(self)
        self._configs = list(tables)
        self._is_weighted = False
        self._device = torch.device(device) if device is not None else torch.device("cpu")
        self.embedding_bags = TableDict()
        self._feature_names, self._feature_table = [], []
        seen = set()
        for cfg in self._configs:
            if cfg.name in seen:
                raise ValueError("duplicate table name %s" % cfg.name)
            seen.add(cfg.name)
            self.embedding_bags[cfg.name] = HybridHashTable(cfg, self._device)
            for f in cfg.feature_names:
                self._feature_names.append(f)
                self._feature_table.append(cfg.name)
        self._cfg_by_name = {c.name: c for c in self._configs}

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        outs, dims = [], []
        fd = features.to_dict()
        for fname, tname in zip(self._feature_names, self._feature_table):
            cfg = self._cfg_by_name[tname]
            jt = fd[fname]
            table: HybridHashTable = self.embedding_bags[tname]  # type: ignore[assignment]
            slots = table.slots(jt.values())
            mode = "sum" if cfg.pooling == PoolingType.SUM else "mean"
            outs.append(F.embedding_bag(slots, table.weight, jt.offsets()[:-1], mode=mode))
            dims.append(cfg.embedding_dim)
        return KeyedTensor(self._feature_names, dims, torch.cat(outs, dim=1))

"""Unsharded ``EmbeddingBagCollection`` / ``EmbeddingCollection`` (TorchRec-compatible surface).

These are the modules a user builds (possibly on the ``meta`` device) before
``DistributedModelParallel`` replaces them by their sharded, fused counterparts.  Their own forward
is the plain PyTorch implementation (``F.embedding_bag`` / ``F.embedding``) and serves as the golden
model in the tests, like the reference's CPU golden (``hybrid_torchrec/test/st/
test_hybrid_hash_embeddingbag.py:127-225``).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor
from .embedding_configs import EmbeddingBagConfig, EmbeddingConfig, PoolingType, data_type_to_dtype


class TableDict(nn.ModuleDict):
    """``nn.ModuleDict`` for per-table holders that accepts every table name.  The stock container refuses keys that are
    also names of its own methods (``items``, ``keys``, ``values``, ``pop`` ...), and ``items`` is what recommendation
    models call their largest table.  Entries are reached by subscript (``d["items"]``), the ``state_dict`` prefix is the
    table name as usual; attribute access keeps meaning the container's method."""

    def __setitem__(self, key: str, module: nn.Module) -> None:
        if not isinstance(key, str) or not key or "." in key:
            raise KeyError("table name must be a non-empty string without '.', got %r" % (key,))
        if not isinstance(module, nn.Module):
            raise TypeError("%s is not a Module" % type(module).__name__)
        self._modules[key] = module


def _init_table(w: torch.Tensor, cfg) -> None:
    if w.device.type == "meta":
        return
    with torch.no_grad():
        if cfg.init_fn is not None:
            cfg.init_fn(w)
        else:
            w.uniform_(cfg.get_weight_init_min(), cfg.get_weight_init_max())


class EmbeddingBagCollection(nn.Module):
    def __init__(self, tables: List[EmbeddingBagConfig], is_weighted: bool = False,
                 device: Optional[torch.device] = None) -> None:
        super().__init__()
        self._configs = list(tables)
        self._is_weighted = is_weighted
        self._device = torch.device(device) if device is not None else torch.device("cpu")
        self.embedding_bags = TableDict()
        names = set()
        self._feature_names: List[str] = []
        self._feature_table: List[str] = []
        for cfg in self._configs:
            if cfg.name in names:
                raise ValueError("duplicate table name %s" % cfg.name)
            names.add(cfg.name)
            holder = nn.Module()
            holder.weight = nn.Parameter(torch.empty(cfg.num_embeddings, cfg.embedding_dim,
                                                     dtype=data_type_to_dtype(cfg.data_type), device=self._device))
            _init_table(holder.weight.data, cfg)
            self.embedding_bags[cfg.name] = holder
            for f in cfg.feature_names:
                self._feature_names.append(f)
                self._feature_table.append(cfg.name)
        self._cfg_by_name = {c.name: c for c in self._configs}

    def embedding_bag_configs(self) -> List[EmbeddingBagConfig]:
        return self._configs

    def is_weighted(self) -> bool:
        return self._is_weighted

    def is_meta(self) -> bool:
        return self._device.type == "meta"

    @property
    def device(self) -> torch.device:
        return self._device

    def reset_parameters(self) -> None:
        for cfg in self._configs:
            _init_table(self.embedding_bags[cfg.name].weight.data, cfg)

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        outs, dims = [], []
        fd = features.to_dict()
        for fname, tname in zip(self._feature_names, self._feature_table):
            cfg = self._cfg_by_name[tname]
            jt = fd[fname]
            w = self.embedding_bags[tname].weight
            mode = "sum" if cfg.pooling == PoolingType.SUM else "mean"
            psw = jt.weights_or_none() if self._is_weighted else None
            out = F.embedding_bag(jt.values().long(), w, jt.offsets()[:-1], mode=mode, per_sample_weights=psw,
                                  include_last_offset=False)
            outs.append(out)
            dims.append(cfg.embedding_dim)
        return KeyedTensor(self._feature_names, dims, torch.cat(outs, dim=1))


class EmbeddingCollection(nn.Module):
    """Sequence (non-pooled) embeddings: ``forward(kjt) -> Dict[feature, JaggedTensor]``."""

    def __init__(self, tables: List[EmbeddingConfig], device: Optional[torch.device] = None,
                 need_indices: bool = False) -> None:
        super().__init__()
        self._configs = list(tables)
        self._device = torch.device(device) if device is not None else torch.device("cpu")
        self._need_indices = need_indices
        self.embeddings = TableDict()
        self._feature_names: List[str] = []
        self._feature_table: List[str] = []
        dims = {c.embedding_dim for c in self._configs}
        if len(dims) > 1:
            raise ValueError("EmbeddingCollection tables must share embedding_dim")
        self._dim = dims.pop() if dims else 0
        for cfg in self._configs:
            holder = nn.Module()
            holder.weight = nn.Parameter(torch.empty(cfg.num_embeddings, cfg.embedding_dim,
                                                     dtype=data_type_to_dtype(cfg.data_type), device=self._device))
            _init_table(holder.weight.data, cfg)
            self.embeddings[cfg.name] = holder
            for f in cfg.feature_names:
                self._feature_names.append(f)
                self._feature_table.append(cfg.name)

    def embedding_configs(self) -> List[EmbeddingConfig]:
        return self._configs

    def embedding_dim(self) -> int:
        return self._dim

    def is_meta(self) -> bool:
        return self._device.type == "meta"

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        out: Dict[str, JaggedTensor] = {}
        fd = features.to_dict()
        for fname, tname in zip(self._feature_names, self._feature_table):
            jt = fd[fname]
            emb = F.embedding(jt.values().long(), self.embeddings[tname].weight)
            out[fname] = JaggedTensor(emb, lengths=jt.lengths(), weights=jt.values() if self._need_indices else None)
        return out

"""One ``EmbeddingBagCollection`` whose tables differ in storage dtype or pooling, on the fused backend.

A fused ``ShardedEmbeddingBagCollection`` keeps all its tables in one flat buffer of one dtype and pools them the same
way.  A collection that mixes fp32 and fp16 tables, or SUM and MEAN pooling, is split here into one fused collection per
(dtype, pooling) group; ``forward`` routes every group's features to its collection and puts the pooled columns back in
the order of the original features, so the model sees one ``KeyedTensor`` as before.  The sub-collections are ordinary
submodules: the optimizer, the gradient join, checkpoints and the status watch find them like any other sharded
collection.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
from torch import nn

from ..modules.embedding_configs import EmbeddingBagConfig
from ..modules.embedding_modules import TableDict
from ..ops import embedding_ops as E
from ..sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor
from .comm import PeerGroup, ShardingEnv
from .embeddingbag import ParameterSharding, ShardedEmbeddingBagCollection


def group_key(t: EmbeddingBagConfig) -> Tuple[object, object]:
    return (t.data_type, t.pooling)


def needs_grouping(tables: List[EmbeddingBagConfig]) -> bool:
    return len({group_key(t) for t in tables}) > 1


class GroupedShardedEmbeddingBagCollection(nn.Module):
    split_dist = False      # every group runs its own exchange inside ``forward``

    def __init__(self, tables: List[EmbeddingBagConfig], plan: Dict[str, ParameterSharding], env: ShardingEnv,
                 device: torch.device, optimizer_spec: Optional[E.OptimizerSpec] = None, peer: Optional[PeerGroup] = None,
                 out_dtype: torch.dtype = torch.bfloat16, max_local_batch: int = 0, one_hot: bool = False,
                 init_weights: bool = True) -> None:
        super().__init__()
        self.tables = list(tables)
        self.feature_names: List[str] = [f for t in tables for f in t.feature_names]
        self.feature_dims: List[int] = [t.embedding_dim for t in tables for _ in t.feature_names]
        order: List[Tuple[object, object]] = []
        members: Dict[Tuple[object, object], List[EmbeddingBagConfig]] = {}
        for t in tables:
            k = group_key(t)
            if k not in members:
                members[k] = []
                order.append(k)
            members[k].append(t)
        self.groups = nn.ModuleList()
        self._group_features: List[List[int]] = []            # positions (in the original feature order) of each group's features
        pos = {f: i for i, f in enumerate(self.feature_names)}
        for k in order:
            sub = members[k]
            self.groups.append(ShardedEmbeddingBagCollection(
                sub, {t.name: plan[t.name] for t in sub if t.name in plan}, env, device, optimizer_spec, peer=peer,
                out_dtype=out_dtype, max_local_batch=max_local_batch, one_hot=one_hot, init_weights=init_weights))
            self._group_features.append([pos[f] for t in sub for f in t.feature_names])
        # column ranges of the original features inside the concatenation of the groups' outputs
        cat_order = [i for g in self._group_features for i in g]
        col, start_of = 0, {}
        for i in cat_order:
            start_of[i] = col
            col += self.feature_dims[i]
        idx = []
        for i in range(len(self.feature_names)):
            idx.extend(range(start_of[i], start_of[i] + self.feature_dims[i]))
        self._identity = idx == list(range(col))
        self.register_buffer("_col_index", torch.tensor(idx, dtype=torch.int64, device=device), persistent=False)
        self.embedding_bags = TableDict()
        for g in self.groups:
            for name, holder in g.embedding_bags.items():
                self.embedding_bags[name] = holder

    # ------------------------------------------------------------------ module surface
    def embedding_bag_configs(self) -> List[EmbeddingBagConfig]:
        return self.tables

    def pooled_dim(self) -> int:
        return sum(self.feature_dims)

    def reset_parameters(self, seed: int = 0) -> None:
        for i, g in enumerate(self.groups):
            g.reset_parameters(seed=seed + 7919 * i)

    def load_from_unsharded(self, ebc: nn.Module) -> None:
        for g in self.groups:
            g.load_from_unsharded(ebc)

    def full_table(self, name: str) -> torch.Tensor:
        for g in self.groups:
            if name in g.embedding_bags:
                return g.full_table(name)
        raise KeyError(name)

    def table_weight(self, name: str) -> torch.Tensor:
        return self.embedding_bags[name].weight

    def join_exchange(self) -> None:
        for g in self.groups:
            g.join_exchange()

    # ------------------------------------------------------------------ forward
    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        assert features.keys() == self.feature_names, "feature order must match the table configs"
        outs = []
        for g, feats in zip(self.groups, self._group_features):
            contiguous = feats == list(range(feats[0], feats[-1] + 1))
            if contiguous and len(self.groups) > 1:
                segs = [feats[0], len(feats), len(self.feature_names) - feats[-1] - 1]
                parts = features.split([s for s in segs if s > 0])
                sub = parts[1 if feats[0] > 0 else 0]
            else:
                sub = features.permute(feats)
            if getattr(features, "one_hot", False):
                sub.one_hot = True
            outs.append(g(sub).values())
        cat = outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)
        if not self._identity:
            cat = cat.index_select(1, self._col_index)
        return KeyedTensor(self.feature_names, self.feature_dims, cat)

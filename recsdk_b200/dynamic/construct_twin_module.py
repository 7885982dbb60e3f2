"""Twin models for equivalence tests: a dynamic (hash-table) embedding collection and a plain static one that start from
the same rows and are trained with the same sparse optimizer, so their outputs and updated rows can be compared step by step
(dynamic_emb ``distributed/construct_twin_module.py:56-96`` feature generator, ``:168-434`` ``ConstructTwinModule`` of the
reference; there the static twin is a TorchRec model with a fused optimizer, here it is the unsharded
``EmbeddingCollection`` plus the row-sparse update below).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..modules.embedding_configs import EmbeddingConfig
from ..modules.embedding_modules import EmbeddingCollection
from ..ops.mxrec_tbe import apply_rows
from ..ops import embedding_ops as E
from ..parallel.comm import ShardingEnv
from ..sparse.jagged_tensor import KeyedJaggedTensor
from .dynamicemb_config import DynamicEmbTableOptions
from .embedding import DynamicEmbeddingCollection
from .hkv import OptimizerType, opt_state_dim

_KIND = {OptimizerType.SGD: E.OPT_SGD, OptimizerType.ROWWISE_ADAGRAD: E.OPT_ROWWISE_ADAGRAD, OptimizerType.ADAGRAD: E.OPT_ADAGRAD,
         OptimizerType.ADAM: E.OPT_ADAM}


def generate_sparse_feature(feature_names: List[str], num_embeddings_list: List[int], local_batch_size: int, lookup_iter: int = 0,
                            device: Optional[torch.device] = None) -> Tuple[KeyedJaggedTensor, torch.Tensor]:
    """One id per sample and feature, walking the id space: iteration ``i`` looks up ids ``i*B .. (i+1)*B - 1`` of every
    table (ids past a table's size fall back to 1).  Returns the KJT and its flat ids."""
    start = lookup_iter * local_batch_size
    base = torch.arange(start, start + local_batch_size, dtype=torch.int64)
    ids = torch.cat([torch.where(base >= n, torch.ones_like(base), base) for n in num_embeddings_list])
    lengths = torch.ones(ids.numel(), dtype=torch.int64)
    if device is not None:
        ids, lengths = ids.to(device), lengths.to(device)
    return KeyedJaggedTensor(keys=list(feature_names), values=ids, lengths=lengths), ids


class StaticTwin(nn.Module):
    """Static tables with the dynamic table's update rule applied to the rows a step touched (``step()`` after ``backward()``)."""

    def __init__(self, configs: List[EmbeddingConfig], device: torch.device, optimizer_type: OptimizerType, hp: Dict[str, float],
                 initial_accumulator_value: float = 0.0) -> None:
        super().__init__()
        self.ec = EmbeddingCollection(configs, device=device)
        self.kind, self.hp, self._steps = _KIND[OptimizerType(optimizer_type)], dict(hp), 0
        self.state1: Dict[str, torch.Tensor] = {}
        self.state2: Dict[str, torch.Tensor] = {}
        for c in configs:
            w = self.ec.embeddings[c.name].weight
            if self.kind == E.OPT_ROWWISE_ADAGRAD:
                self.state1[c.name] = torch.full((w.shape[0],), float(initial_accumulator_value), device=device)
            elif self.kind == E.OPT_ADAGRAD:
                self.state1[c.name] = torch.full_like(w, float(initial_accumulator_value), dtype=torch.float32)
            elif self.kind == E.OPT_ADAM:
                self.state1[c.name], self.state2[c.name] = torch.zeros_like(w, dtype=torch.float32), torch.zeros_like(w, dtype=torch.float32)

    def forward(self, features: KeyedJaggedTensor):
        return self.ec(features)

    @torch.no_grad()
    def step(self) -> None:
        self._steps += 1
        hp = dict(self.hp, iter=self._steps)
        for name, holder in self.ec.embeddings.items():
            w = holder.weight
            if w.grad is None:
                continue
            rows = torch.nonzero(w.grad.abs().sum(dim=1) > 0).flatten()
            if rows.numel():
                apply_rows(self.kind, w.data, rows, w.grad[rows].float(), self.state1.get(name), self.state2.get(name), hp)
            w.grad = None

    def set_optimizer_step(self, step: int) -> None:
        self._steps = int(step)


class ConstructTwinModule:
    """``init_twin_embedding_model()`` builds both models and copies every row of the static twin that this rank owns
    (``id % world_size == rank``) into the dynamic table, optimizer state at its initial value."""

    def __init__(self, table_num: int, dims: List[int], num_embeddings: List[int], multi_hot_sizes: Optional[List[int]] = None,
                 batch_size: int = 65536, output_dtype: torch.dtype = torch.float32, fwd_a2a_precision: Any = None,
                 bwd_a2a_precision: Any = None, optimizer_kwargs: Optional[Dict[str, Any]] = None,
                 init_fn: Optional[Callable[[torch.Tensor], Optional[torch.Tensor]]] = None, rank: int = 0, world_size: int = 1,
                 scale_factor: int = 2, env: Optional[ShardingEnv] = None, device: Optional[torch.device] = None) -> None:
        self._table_num, self._dims, self._num_embeddings = table_num, list(dims), list(num_embeddings)
        self._multi_hot_sizes = list(multi_hot_sizes) if multi_hot_sizes is not None else [1] * table_num
        self._batch_size, self._output_dtype = batch_size, output_dtype
        self._optimizer_kwargs = dict(optimizer_kwargs or {})
        self._init_fn, self._rank, self._world_size, self._scale_factor = init_fn, rank, world_size, scale_factor
        self._env = env or ShardingEnv(world_size, rank, None)
        self._device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self._table_names = [f"t_{t}" for t in range(table_num)]
        self._feature_names = [f"f_{t}" for t in range(table_num)]
        self._dynamicemb_model: Optional[DynamicEmbeddingCollection] = None
        self._torchrec_model: Optional[StaticTwin] = None

    def _optimizer(self) -> Tuple[OptimizerType, Dict[str, float], float]:
        kw = self._optimizer_kwargs
        opt = OptimizerType(kw.get("optimizer", OptimizerType.ROWWISE_ADAGRAD))
        hp = {"lr": float(kw.get("learning_rate", 0.01)), "eps": float(kw.get("eps", 1e-8)), "beta1": float(kw.get("beta1", 0.9)),
              "beta2": float(kw.get("beta2", 0.999)), "weight_decay": float(kw.get("weight_decay", 0.0))}
        return opt, hp, float(kw.get("initial_accumulator_value", 0.0))

    def _construct_dynamicemb_module(self) -> None:
        opt, hp, acc0 = self._optimizer()
        configs = [EmbeddingConfig(name=self._table_names[i], embedding_dim=self._dims[i], feature_names=[self._feature_names[i]],
                                   num_embeddings=self._num_embeddings[i] * self._scale_factor) for i in range(self._table_num)]
        options = {n: DynamicEmbTableOptions() for n in self._table_names}
        self._dynamicemb_model = DynamicEmbeddingCollection(
            configs, options, env=self._env, device=self._device, optimizer_type=opt, learning_rate=hp["lr"], eps=hp["eps"],
            betas=(hp["beta1"], hp["beta2"]), weight_decay=hp["weight_decay"], output_dtype=self._output_dtype)

    def _construct_torchrec_module(self) -> None:
        opt, hp, acc0 = self._optimizer()
        configs = [EmbeddingConfig(name=self._table_names[i], embedding_dim=self._dims[i], feature_names=[self._feature_names[i]],
                                   num_embeddings=self._num_embeddings[i]) for i in range(self._table_num)]
        self._torchrec_model = StaticTwin(configs, self._device, opt, hp, acc0)
        if self._init_fn is not None:
            with torch.no_grad():
                for holder in self._torchrec_model.ec.embeddings.values():
                    r = self._init_fn(holder.weight.data)
                    if r is not None:
                        holder.weight.data.copy_(r)

    def init_twin_embedding_model(self) -> None:
        self._construct_dynamicemb_module()
        self._construct_torchrec_module()
        opt, _, acc0 = self._optimizer()
        for i, name in enumerate(self._table_names):
            w = self._torchrec_model.ec.embeddings[name].weight.data.float()
            ids = torch.arange(w.shape[0], dtype=torch.int64, device=w.device)
            mine = ids % self._world_size == self._rank
            kv = self._dynamicemb_model.table(name)
            sd = opt_state_dim(opt, self._dims[i])
            fill = acc0 if opt in (OptimizerType.ADAGRAD, OptimizerType.ROWWISE_ADAGRAD) else 0.0
            rows = torch.cat([w[mine], torch.full((int(mine.sum()), sd), fill, device=w.device)], dim=1).contiguous()
            table = kv.table
            table.reserve(max(table.capacity, 2 * int(mine.sum())))
            table.insert_and_evict(ids[mine].to(table.device), rows.to(table.device))
        self._torchrec_model.set_optimizer_step(0)

    @property
    def dynamicemb_model(self) -> DynamicEmbeddingCollection:
        return self._dynamicemb_model

    @property
    def torchrec_model(self) -> StaticTwin:
        return self._torchrec_model

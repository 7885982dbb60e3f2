"""``BatchedDynamicEmbeddingTablesV2``: N dynamic tables behind one module, sequence (EC) or pooled (EBC).

Forward per table: de-duplicate the ids (sort + run-length encode on the GPU), ``find_or_insert`` (train) or
``find`` (eval) the unique keys, gather their rows and expand them back (EC) or pool them per bag (EBC).
Backward: reduce the gradients per unique key and run the fused optimizer on the row pointers - the update
happens inside backward, the module's optimizer ``step`` is a no-op.  Structure after
``dynamic_emb/distributed/batched_dynamicemb_table.py:490-1267`` and ``batched_dynamicemb_function.py:53-469``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
from torch import nn

from .dynamicemb_config import DynamicEmbPoolingMode, DynamicEmbScoreStrategy, DynamicEmbTableOptions
from .key_value_table import KeyValueTable


def _unique(ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return torch.unique(ids, return_inverse=True)


class _DynamicLookupFn(torch.autograd.Function):
    """ids of ONE table -> rows per id; sparse update in backward."""

    @staticmethod
    def forward(ctx, anchor: torch.Tensor, table: KeyValueTable, ids: torch.Tensor, training: bool):
        uniq, inv = _unique(ids)
        slots, rows = table.lookup(uniq, training)
        ctx.table, ctx.training = table, training
        ctx.save_for_backward(slots, inv)
        ctx.n_unique = uniq.numel()
        return rows[inv]

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        slots, inv = ctx.saved_tensors
        if ctx.training and ctx.n_unique:
            red = torch.zeros(ctx.n_unique, g.shape[1], dtype=torch.float32, device=g.device)
            red.index_add_(0, inv, g.float())                 # reduce_grads: one row per unique key
            ctx.table.update(slots, red)
        return None, None, None, None


class BatchedDynamicEmbeddingTablesV2(nn.Module):
    def __init__(self, table_options: List[DynamicEmbTableOptions], table_names: List[str],
                 pooling_mode: DynamicEmbPoolingMode = DynamicEmbPoolingMode.NONE,
                 output_dtype: torch.dtype = torch.float32, device: Optional[torch.device] = None,
                 feature_table_map: Optional[List[int]] = None, learning_rate: float = 0.01, eps: float = 1e-8,
                 betas=(0.9, 0.999), weight_decay: float = 0.0, initial_accumulator_value: float = 0.0, seed: int = 0) -> None:
        super().__init__()
        assert len(table_options) == len(table_names)
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda" if torch.cuda.is_available() else "cpu")
        self.table_names = list(table_names)
        self.pooling_mode = DynamicEmbPoolingMode(pooling_mode)
        self.output_dtype = output_dtype
        self.feature_table_map = list(range(len(table_names))) if feature_table_map is None else list(feature_table_map)
        self.tables: List[KeyValueTable] = [
            KeyValueTable(n, o, self.device, lr=learning_rate, eps=eps, betas=betas, weight_decay=weight_decay,
                          seed=seed + 7919 * i, initial_accumulator_value=initial_accumulator_value)
            for i, (n, o) in enumerate(zip(table_names, table_options))]
        self.dims = [o.dim for o in table_options]
        self._anchor = nn.Parameter(torch.zeros(1, device=self.device))
        self._anchor._in_backward_optimizers = True  # type: ignore[attr-defined]
        self._global_step = 0

    # ---------------------------------------------------------------- scores
    def _update_score(self) -> None:
        """STEP tables count steps; CUSTOMIZED tables keep what ``set_score`` stored; TIMESTAMP / LFU tables are
        scored by the kernels (``batched_dynamicemb_table.py:1032-1091``)."""
        self._global_step += 1
        for t in self.tables:
            if t.options.score_strategy == DynamicEmbScoreStrategy.STEP:
                t.score_value = self._global_step

    def set_score(self, named: Dict[str, int]) -> None:
        for t in self.tables:
            if t.name in named:
                t.score_value = int(named[t.name])

    def get_score(self) -> Dict[str, int]:
        return {t.name: int(t.score_value) for t in self.tables}

    def set_learning_rate(self, lr: float) -> None:
        for t in self.tables:
            t.lr = lr

    # ---------------------------------------------------------------- forward
    def forward(self, indices: torch.Tensor, offsets: torch.Tensor, feature_splits: List[int], batch_size: int):
        """``indices`` [nnz] ids of all features (feature-major), ``offsets`` [F*B+1] bag offsets,
        ``feature_splits[f]`` = number of ids of feature ``f``.
        EC (pooling NONE): -> [nnz, D]; EBC: -> [B, sum(D_f)]."""
        if self.training:
            self._update_score()
        outs = []
        start = 0
        F = len(self.feature_table_map)
        for f in range(F):
            n = feature_splits[f]
            tab = self.tables[self.feature_table_map[f]]
            ids = indices[start:start + n]
            rows = _DynamicLookupFn.apply(self._anchor, tab, ids, self.training)
            if self.pooling_mode == DynamicEmbPoolingMode.NONE:
                outs.append(rows)
            else:
                off = offsets[f * batch_size:(f + 1) * batch_size + 1] - start
                lengths = off[1:] - off[:-1]
                bag = torch.repeat_interleave(torch.arange(batch_size, device=rows.device), lengths)
                pooled = torch.zeros(batch_size, rows.shape[1], dtype=rows.dtype, device=rows.device).index_add_(0, bag, rows)
                if self.pooling_mode == DynamicEmbPoolingMode.MEAN:
                    pooled = pooled / lengths.clamp(min=1).to(pooled.dtype)[:, None]
                outs.append(pooled)
            start += n
        if self.pooling_mode == DynamicEmbPoolingMode.NONE:
            return torch.cat(outs, dim=0).to(self.output_dtype)
        return torch.cat(outs, dim=1).to(self.output_dtype)

    # ---------------------------------------------------------------- persistence
    def dump(self, save_dir: str, rank: int = 0, world: int = 1, optim: bool = True,
             table_names: Optional[List[str]] = None) -> None:
        for t in self.tables:
            if table_names is None or t.name in table_names:
                t.dump(save_dir, rank, world, optim)

    def load(self, save_dir: str, rank: int = 0, world: int = 1, optim: bool = True,
             table_names: Optional[List[str]] = None) -> Dict[str, int]:
        return {t.name: t.load(save_dir, rank, world, optim) for t in self.tables
                if table_names is None or t.name in table_names}

    def incremental_dump(self, score_threshold: Dict[str, int]):
        """-> ({table: (keys, values)}, {table: current score}) for entries whose score >= threshold."""
        out, cur = {}, {}
        for t in self.tables:
            thr = score_threshold.get(t.name, 0) if isinstance(score_threshold, dict) else int(score_threshold)
            k, v, _s = t.export_keys_values(min_score=thr)
            out[t.name] = (k, v[:, : t.dim].contiguous())
            cur[t.name] = int(t.score_value)
        return out, cur

    def export_keys_values(self, name: str):
        t = self.tables[self.table_names.index(name)]
        k, v, s = t.export_keys_values()
        return k, v[:, : t.dim], s

    def flush(self) -> None:
        for t in self.tables:
            t.flush()

    def set_record_cache_metrics(self, on: bool) -> None:
        for t in self.tables:
            t.record_metrics = on

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


_SORTED_REDUCE_MIN_IDS = int(__import__("os").environ.get("RECSDK_B200_SORTED_REDUCE_MIN_IDS", "65536"))


class _DynamicPooledLookupFn(torch.autograd.Function):
    """ids of ONE feature with bag offsets -> pooled rows ``[B, D]``; the per-id rows are never materialised: the pooled
    gather reads the unique rows through the inverse index, the backward adds each bag's gradient to its unique rows
    with 16-byte vector reductions, then the fused optimizer runs on the unique rows."""

    @staticmethod
    def forward(ctx, anchor: torch.Tensor, table: KeyValueTable, ids: torch.Tensor, offsets: torch.Tensor, batch: int, mean: bool,
                training: bool, out_dtype: torch.dtype):
        """``ids`` / ``offsets`` may span several features of the table (``offsets`` has ``F * batch + 1`` entries,
        feature-major); the result is ``[batch, F * D]`` with feature ``f`` in columns ``[f * D, (f + 1) * D)``."""
        from ..ops import _lib

        uniq, inv = _unique(ids)
        slots, rows = table.lookup(uniq, training)
        rows = rows.float().contiguous()
        D = rows.shape[1]
        offsets = offsets.to(torch.int64).contiguous()
        bags = offsets.numel() - 1
        F = bags // batch
        if rows.is_cuda and D % 4 == 0:
            out = torch.empty(batch, F * D, dtype=out_dtype, device=rows.device)
            rc = _lib.lib().rb_pooled_gather(rows.data_ptr(), inv.data_ptr(), offsets.data_ptr(), bags, batch, D, int(mean), out.data_ptr(),
                                             _lib.dtype_code(out_dtype), out.stride(0), _lib.stream_ptr(rows.device))
            _lib.check(rc, "rb_pooled_gather")
        else:
            lengths = offsets[1:] - offsets[:-1]
            bag = torch.repeat_interleave(torch.arange(bags, device=rows.device), lengths)
            out = torch.zeros(bags, D, dtype=torch.float32, device=rows.device).index_add_(0, bag, rows[inv])
            if mean:
                out = out / lengths.clamp(min=1).to(out.dtype)[:, None]
            out = out.view(F, batch, D).permute(1, 0, 2).reshape(batch, F * D).to(out_dtype)
        ctx.table, ctx.training, ctx.mean, ctx.batch = table, training, mean, batch
        ctx.save_for_backward(slots, inv, offsets)
        ctx.n_unique, ctx.D = uniq.numel(), D
        return out

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        from ..ops import _lib

        slots, inv, offsets = ctx.saved_tensors
        if ctx.training and ctx.n_unique:
            red = torch.zeros(ctx.n_unique, ctx.D, dtype=torch.float32, device=g.device)
            bags = offsets.numel() - 1
            n = inv.numel()
            if g.is_cuda and ctx.D % 4 == 0 and g.stride(1) == 1 and n >= _SORTED_REDUCE_MIN_IDS and bags < (1 << 31):
                # large batches: sort the (unique row, bag) pairs by row and sum runs, so a hot row costs one reduction per
                # 64 ids instead of one per id and rows used by few bags are written without atomics
                from ..ops.sparse_ops import _ws

                dev = g.device
                L = _lib.lib()
                lengths = offsets[1:] - offsets[:-1]
                bag_of = torch.repeat_interleave(torch.arange(bags, dtype=torch.int32, device=dev), lengths, output_size=n)
                keys_sorted = _ws(dev, "pool_keys", n, torch.int64)
                bags_sorted = _ws(dev, "pool_bags", n, torch.int32)
                tb = int(L.rb_sort_segments_temp_bytes(n))
                temp = _ws(dev, "pool_sort_tmp", tb, torch.uint8)
                st = _lib.stream_ptr(dev)
                rc = L.rb_sort_pairs_i64_i32(inv.data_ptr(), bag_of.data_ptr(), n, max(1, int(ctx.n_unique).bit_length()),
                                             keys_sorted.data_ptr(), bags_sorted.data_ptr(), temp.data_ptr(), tb, st)
                _lib.check(rc, "rb_sort_pairs_i64_i32")
                rc = L.rb_pooled_segment_add(g.data_ptr(), _lib.dtype_code(g.dtype), g.stride(0), keys_sorted.data_ptr(),
                                             bags_sorted.data_ptr(), offsets.data_ptr(), n, ctx.batch, ctx.D, int(ctx.mean),
                                             red.data_ptr(), st)
                _lib.check(rc, "rb_pooled_segment_add")
            elif g.is_cuda and ctx.D % 4 == 0 and g.stride(1) == 1:
                rc = _lib.lib().rb_pooled_scatter_add(g.data_ptr(), _lib.dtype_code(g.dtype), g.stride(0), inv.data_ptr(), offsets.data_ptr(),
                                                      bags, ctx.batch, ctx.D, int(ctx.mean), red.data_ptr(), _lib.stream_ptr(g.device))
                _lib.check(rc, "rb_pooled_scatter_add")
            else:
                lengths = offsets[1:] - offsets[:-1]
                bag = torch.repeat_interleave(torch.arange(bags, device=g.device), lengths)
                gg = g.float().view(ctx.batch, bags // ctx.batch, ctx.D).permute(1, 0, 2).reshape(bags, ctx.D)
                if ctx.mean:
                    gg = gg / lengths.clamp(min=1).to(gg.dtype)[:, None]
                red.index_add_(0, inv, gg[bag])
            ctx.table.update(slots, red)
        return (None,) * 8


# the reference's names of the two autograd functions (``batched_dynamicemb_function.py:53-213`` pooled, ``:342-432`` sequence)
DynamicEmbeddingFunctionV2 = _DynamicLookupFn
DynamicEmbeddingBagFunction = _DynamicPooledLookupFn


def dynamicemb_prefetch(module: "BatchedDynamicEmbeddingTablesV2", indices: torch.Tensor, offsets: torch.Tensor, forward_stream=None) -> None:
    """Function form of ``module.prefetch`` (``batched_dynamicemb_function.py:284-325`` of the reference)."""
    module.prefetch(indices, offsets, forward_stream)


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
        self._enable_prefetch = False
        self.num_prefetch_ahead = 0
        self.prefetch_stream: Optional["torch.cuda.Stream"] = None
        self._caching = any(t.storage is not None for t in self.tables)

    # ---------------------------------------------------------------- accessors of the reference module
    @property
    def caches(self) -> List[KeyValueTable]:
        """Tables that front a storage tier (their device table is the cache)."""
        return [t for t in self.tables if t.storage is not None]

    @property
    def optimizer(self):
        """Row-level optimizer object with this module's current hyper-parameters (learning rate, eps, betas, weight decay,
        iterations): the handle the reference exposes for exporting / restoring optimizer arguments."""
        from .optimizers import OptimizerArgs, create_optimizer

        t = self.tables[0]
        opt = create_optimizer(t.optimizer, OptimizerArgs(learning_rate=t.lr, weight_decay=t.weight_decay, eps=t.eps, beta1=t.betas[0],
                                                          beta2=t.betas[1], initial_accumulator_value=float(t._init.state_init)))
        opt._iterations = int(t._step)
        return opt

    def split_embedding_weights(self) -> List[torch.Tensor]:
        """One ``[live rows, dim]`` tensor per table (a snapshot: dynamic tables have no fixed weight matrix)."""
        return [self.export_keys_values(n)[1] for n in self.table_names]

    def reset_cache_states(self) -> None:
        """Write the cached rows back and zero the cache metrics."""
        self.flush()
        for t in self.tables:
            for k in t.metrics:
                t.metrics[k] = 0

    # ---------------------------------------------------------------- memory report
    def memory_report(self) -> List[Dict[str, object]]:
        """Per table: capacity, live rows, and the bytes its rows take in total / on the device / on the host, split into
        embedding and optimizer state - what the reference prints at construction (``_print_memory_consume``,
        ``batched_dynamicemb_table.py:272-363``)."""
        out = []
        for t in self.tables:
            tab = t.table
            cap = int(getattr(tab, "capacity", 0) or 0)
            hbm_rows = int(getattr(tab, "hbm_rows", cap) if getattr(tab, "hbm_rows", None) is not None else cap)
            hbm_rows = min(hbm_rows, cap)
            host_rows = cap - hbm_rows
            eb, sb = 4 * t.dim, 4 * t.state_dim

            def split(rows: int) -> Dict[str, int]:
                return {"total": rows * (eb + sb), "embedding": rows * eb, "optim_state": rows * sb}

            out.append({"table": t.name, "dim": t.dim, "optim_state_dim": t.state_dim, "capacity": cap,
                        "size": int(t.table.size()) if hasattr(t.table, "size") else 0,
                        "total_bytes": split(cap), "hbm_bytes": split(hbm_rows), "host_bytes": split(host_rows),
                        "index_bytes": cap * (8 + 8 + 1 + 4) + (cap // 128) * 4,      # keys, scores, digests, stamps, bucket locks
                        "storage_tier": type(t.storage).__name__ if t.storage is not None else None})
        return out

    def print_memory_consume(self) -> str:
        rows = self.memory_report()
        unit, name = (1 << 20, "MB") if any(r["total_bytes"]["total"] >= (1 << 20) for r in rows) else (1 << 10, "KB")
        head = "%-20s %14s %14s %14s %14s" % ("table (%s)" % name, "total", "hbm", "host", "index")
        lines = [head] + ["%-20s %14d %14d %14d %14d" % (r["table"], r["total_bytes"]["total"] // unit, r["hbm_bytes"]["total"] // unit,
                                                         r["host_bytes"]["total"] // unit, r["index_bytes"] // unit) for r in rows]
        text = "\n".join(lines)
        print(text)
        return text

    # ---------------------------------------------------------------- prefetch
    @property
    def enable_prefetch(self) -> bool:
        return self._enable_prefetch

    @enable_prefetch.setter
    def enable_prefetch(self, value: bool) -> None:
        self._enable_prefetch = bool(value)
        self.num_prefetch_ahead = 0

    def prefetch(self, indices: torch.Tensor, offsets: torch.Tensor, forward_stream=None,
                 batch_size_per_feature_per_rank=None, feature_splits: Optional[List[int]] = None) -> None:
        """Bring the rows of a coming batch from the storage tier into the device cache ahead of its ``forward`` (sequence
        embeddings only, as in the reference: ``batched_dynamicemb_table.py:940-1001``).  Runs on the caller's current
        stream, which must differ from ``forward_stream``; ``forward`` then finds its keys resident.  ``feature_splits``
        gives the ids per feature when several tables share the module (default: all ids belong to table 0's features in
        order of ``feature_table_map`` with equal bags)."""
        if self.pooling_mode != DynamicEmbPoolingMode.NONE:
            raise RuntimeError("only support prefetch for sequence embedding.")
        if not self._enable_prefetch:
            raise RuntimeError("Prefetch is not enabled.")
        if indices.is_cuda and forward_stream is not None:
            cur = torch.cuda.current_stream(indices.device)
            if self.prefetch_stream is None:
                self.prefetch_stream = cur
            if cur == forward_stream:
                raise RuntimeError("prefetch_stream and forward_stream should not be the same stream.")
            indices.record_stream(cur)
            offsets.record_stream(cur)
        self.num_prefetch_ahead += 1
        if not self._caching:
            return                                       # nothing below the device table: prefetch has nothing to move
        F = len(self.feature_table_map)
        if feature_splits is None:
            if F == 1:
                feature_splits = [indices.numel()]
            else:
                B = (offsets.numel() - 1) // F
                feature_splits = [int(offsets[(f + 1) * B] - offsets[f * B]) for f in range(F)]
        start = 0
        by_table: Dict[int, List[torch.Tensor]] = {}
        for f, n in enumerate(feature_splits):
            by_table.setdefault(self.feature_table_map[f], []).append(indices[start:start + n])
            start += n
        for ti, parts in by_table.items():
            t = self.tables[ti]
            if t.storage is None:
                continue
            keys = torch.unique(torch.cat(parts) if len(parts) > 1 else parts[0])
            if self.training and t.options.score_strategy == DynamicEmbScoreStrategy.STEP:
                # rows touched by a prefetch carry the score of the step that will use them
                saved, t.score_value = t.score_value, self._global_step + self.num_prefetch_ahead
                t._caching_lookup(keys.to(self.device).long())
                t.score_value = saved
            else:
                t._caching_lookup(keys.to(self.device).long())

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
        if self._enable_prefetch and self.num_prefetch_ahead > 0:
            self.num_prefetch_ahead -= 1
        F = len(self.feature_table_map)
        starts = [0] * (F + 1)
        for f in range(F):
            starts[f + 1] = starts[f] + feature_splits[f]
        by_table: Dict[int, List[int]] = {}
        for f, ti in enumerate(self.feature_table_map):
            by_table.setdefault(ti, []).append(f)
        outs: List[Optional[torch.Tensor]] = [None] * F
        pooled = self.pooling_mode != DynamicEmbPoolingMode.NONE
        # ONE unique / lookup / update per table and step: the features that share a table are looked up together, so a
        # growing or evicting table never invalidates slots that another feature of the same step still holds, and the
        # optimizer steps once per table
        for ti, feats in by_table.items():
            tab = self.tables[ti]
            adjacent = feats == list(range(feats[0], feats[-1] + 1))
            if adjacent:
                ids = indices[starts[feats[0]]:starts[feats[-1] + 1]]
            else:
                ids = torch.cat([indices[starts[f]:starts[f + 1]] for f in feats])
            if not pooled:
                rows = _DynamicLookupFn.apply(self._anchor, tab, ids, self.training)
                pos = 0
                for f in feats:
                    outs[f] = rows[pos:pos + feature_splits[f]]
                    pos += feature_splits[f]
                continue
            if adjacent:
                off = offsets[feats[0] * batch_size:(feats[-1] + 1) * batch_size + 1] - starts[feats[0]]
            else:
                lens = torch.cat([offsets[f * batch_size + 1:(f + 1) * batch_size + 1] - offsets[f * batch_size:(f + 1) * batch_size]
                                  for f in feats])
                off = torch.cat([lens.new_zeros(1), lens.cumsum(0)])
            out = _DynamicPooledLookupFn.apply(self._anchor, tab, ids, off, batch_size,
                                               self.pooling_mode == DynamicEmbPoolingMode.MEAN, self.training, self.output_dtype)
            D = self.dims[ti]
            for k, f in enumerate(feats):
                outs[f] = out[:, k * D:(k + 1) * D]
        if not pooled:
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

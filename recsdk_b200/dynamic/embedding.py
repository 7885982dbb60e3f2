"""Dynamic (hash-table backed) embedding collections, row-wise sharded by ``key % world_size``.

``DynamicEmbeddingCollection`` returns per-id embeddings (sequence), ``DynamicEmbeddingBagCollection``
pooled ones.  Flow per step (``dynamic_emb/distributed/embedding.py:143-336``, ``sharding/rw_sharding.py:153-263``):
optional local de-duplication of the ids, bucketise by owner (round robin), all-to-all of counts and ids,
owner-side ``find_or_insert`` + gather in ``BatchedDynamicEmbeddingTablesV2``, all-to-all of the rows back,
restore the original order (and pool per bag for the bag collection).  Backward runs the same exchange in
reverse and the fused optimizer on the owner.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..modules.embedding_configs import BaseEmbeddingConfig, PoolingType
from ..parallel.collective_embeddingbag import _AllToAll
from ..parallel.comm import ShardingEnv
from ..sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor
from .batched_dynamicemb_table import BatchedDynamicEmbeddingTablesV2
from .dynamicemb_config import DynamicEmbPoolingMode, DynamicEmbTableOptions, get_constraint_capacity
from .hkv import OptimizerType


class _ShardedDynamicBase(nn.Module):
    def __init__(self, tables: List[BaseEmbeddingConfig], options: Dict[str, DynamicEmbTableOptions],
                 env: Optional[ShardingEnv] = None, device: Optional[torch.device] = None,
                 optimizer_type: OptimizerType = OptimizerType.ROWWISE_ADAGRAD, learning_rate: float = 0.01,
                 eps: float = 1e-8, betas=(0.9, 0.999), weight_decay: float = 0.0, use_index_dedup: bool = False,
                 output_dtype: torch.dtype = torch.float32, seed: int = 0) -> None:
        super().__init__()
        self.env = env or ShardingEnv(1, 0, None)
        self.world, self.rank, self.pg = self.env.world_size, self.env.rank, self.env.process_group
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.configs = list(tables)
        self.use_index_dedup = use_index_dedup
        self.feature_names: List[str] = []
        self.feature_table: List[int] = []
        opts = []
        for ti, t in enumerate(tables):
            o = options.get(t.name) or DynamicEmbTableOptions()
            o.dim = t.embedding_dim
            o.optimizer_type = optimizer_type
            cap = get_constraint_capacity(t.num_embeddings, self.world, o.bucket_capacity)
            o.max_capacity = o.max_capacity or cap
            o.num_aligned_embedding_per_rank = cap
            if o.init_capacity is None:
                o.init_capacity = min(o.max_capacity, max(o.bucket_capacity, 1024))
            opts.append(o)
            for f in t.feature_names:
                self.feature_names.append(f)
                self.feature_table.append(ti)
        self.dims = [t.embedding_dim for t in tables]
        self.lookup = BatchedDynamicEmbeddingTablesV2(
            opts, [t.name for t in tables], DynamicEmbPoolingMode.NONE, torch.float32, self.device, self.feature_table,
            learning_rate, eps, betas, weight_decay, seed=seed)
        self.output_dtype = output_dtype

    # -- rows for every id of the local KJT, in the KJT's own order: [nnz, D] ------------------------
    def _sequence_rows(self, features: KeyedJaggedTensor) -> torch.Tensor:
        assert features.keys() == self.feature_names
        F = len(self.feature_names)
        ids = features.values().to(self.device).long()
        lpk = features.length_per_key()
        if self.world == 1:
            return self.lookup(ids, None, lpk, features.stride())
        W = self.world
        feat = torch.repeat_interleave(torch.arange(F, device=ids.device), torch.tensor(lpk, device=ids.device))
        inv_dedup = None
        if self.use_index_dedup:
            # ids are feature-major, so the (feature, id) pairs de-duplicate with one 1-D unique per feature (a row-wise
            # unique over pairs is far slower and this needs no assumption about the key range)
            us, invs, fs, start, base = [], [], [], 0, 0
            for f, n in enumerate(lpk):
                u, inv = torch.unique(ids[start:start + n], return_inverse=True)
                us.append(u)
                invs.append(inv + base)
                fs.append(torch.full((u.numel(),), f, dtype=feat.dtype, device=ids.device))
                base += u.numel()
                start += n
            ids, inv_dedup, feat = torch.cat(us), torch.cat(invs), torch.cat(fs)
        dest = torch.remainder(ids, W)
        order = torch.argsort(dest * F + feat, stable=True)            # (destination, feature)-major
        send_ids = ids[order]
        counts = torch.bincount(dest * F + feat, minlength=W * F).view(W, F)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts.contiguous(), group=self.pg)
        in_splits = counts.sum(1).tolist()
        both = torch.cat([recv_counts.sum(1), recv_counts.sum(0)]).tolist()      # one host read for both split lists
        out_splits, feature_splits = both[:W], both[W:]
        recv_ids = send_ids.new_empty(int(sum(out_splits)))
        dist.all_to_all_single(recv_ids, send_ids, out_splits, in_splits, group=self.pg)
        # owner side: regroup (source, feature) -> feature-major for the batched lookup
        rc = recv_counts.view(-1)
        seg_feat = torch.arange(F, device=ids.device).repeat(W)
        elem_feat = torch.repeat_interleave(seg_feat, rc)
        to_fm = torch.argsort(elem_feat, stable=True)
        splits = feature_splits
        rows_fm = self.lookup(recv_ids[to_fm], None, splits, 0)
        rows_sf = torch.empty_like(rows_fm)
        rows_sf[to_fm] = rows_fm                                        # differentiable scatter back
        back = _AllToAll.apply(rows_sf, in_splits, out_splits, self.pg)
        rows = torch.empty_like(back)
        rows[order] = back
        if inv_dedup is not None:
            rows = rows[inv_dedup]
        return rows

    # -- persistence / scores -----------------------------------------------------------------------
    def dump(self, save_dir: str, optim: bool = True, table_names=None) -> None:
        self.lookup.dump(save_dir, self.rank, self.world, optim, table_names)

    def load(self, save_dir: str, optim: bool = True, table_names=None):
        return self.lookup.load(save_dir, self.rank, self.world, optim, table_names)

    def table(self, name: str):
        return self.lookup.tables[self.lookup.table_names.index(name)]


class DynamicEmbeddingCollection(_ShardedDynamicBase):
    def embedding_configs(self):
        return self.configs

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        rows = self._sequence_rows(features).to(self.output_dtype)
        out: Dict[str, JaggedTensor] = {}
        B, start = features.stride(), 0
        lens = features.lengths().to(self.device)
        for f, (name, n) in enumerate(zip(self.feature_names, features.length_per_key())):
            out[name] = JaggedTensor(rows[start:start + n], lengths=lens[f * B:(f + 1) * B])
            start += n
        return out


class DynamicEmbeddingBagCollection(_ShardedDynamicBase):
    def embedding_bag_configs(self):
        return self.configs

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        if self.world == 1:
            return self._forward_local(features)
        rows = self._sequence_rows(features)
        B = features.stride()
        lens = features.lengths().to(self.device)
        outs, start = [], 0
        for f, n in enumerate(features.length_per_key()):
            cfg = self.configs[self.feature_table[f]]
            ln = lens[f * B:(f + 1) * B]
            bag = torch.repeat_interleave(torch.arange(B, device=rows.device), ln)
            r = rows[start:start + n]
            pooled = torch.zeros(B, r.shape[1], dtype=r.dtype, device=r.device).index_add_(0, bag, r)
            if getattr(cfg, "pooling", PoolingType.SUM) == PoolingType.MEAN:
                pooled = pooled / ln.clamp(min=1).to(pooled.dtype)[:, None]
            outs.append(pooled)
            start += n
        feature_dims = [self.dims[t] for t in self.feature_table]
        return KeyedTensor(self.feature_names, feature_dims, torch.cat(outs, dim=1).to(self.output_dtype))

    def _forward_local(self, features: KeyedJaggedTensor) -> KeyedTensor:
        """One rank: pool straight from the unique rows (no per-id row tensor)."""
        from .batched_dynamicemb_table import _DynamicPooledLookupFn

        assert features.keys() == self.feature_names
        B = features.stride()
        ids = features.values().to(self.device).long()
        offsets = features.offsets().to(self.device).long()
        lk = self.lookup
        if lk.training:
            lk._update_score()
        # features of one table are adjacent in the key order: one unique / lookup / pooled gather per table
        outs, start, f = [], 0, 0
        lpk = features.length_per_key()
        F = len(self.feature_names)
        while f < F:
            ti = self.feature_table[f]
            f1 = f
            while f1 < F and self.feature_table[f1] == ti:
                f1 += 1
            n = sum(lpk[f:f1])
            cfg = self.configs[ti]
            off = offsets[f * B:f1 * B + 1] - start
            mean = getattr(cfg, "pooling", PoolingType.SUM) == PoolingType.MEAN
            outs.append(_DynamicPooledLookupFn.apply(lk._anchor, lk.tables[ti], ids[start:start + n], off, B, mean, lk.training,
                                                     self.output_dtype))
            start += n
            f = f1
        feature_dims = [self.dims[t] for t in self.feature_table]
        return KeyedTensor(self.feature_names, feature_dims, torch.cat(outs, dim=1))

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
from .dynamicemb_config import DynamicEmbPoolingMode, DynamicEmbTableOptions, aligned_capacity_per_rank
from .hkv import OptimizerType


class _ShardedDynamicBase(nn.Module):
    def __init__(self, tables: List[BaseEmbeddingConfig], options: Dict[str, DynamicEmbTableOptions],
                 env: Optional[ShardingEnv] = None, device: Optional[torch.device] = None,
                 optimizer_type: OptimizerType = OptimizerType.ROWWISE_ADAGRAD, learning_rate: float = 0.01,
                 eps: float = 1e-8, betas=(0.9, 0.999), weight_decay: float = 0.0, use_index_dedup: bool = False,
                 output_dtype: torch.dtype = torch.float32, seed: int = 0, peer=None, max_ids_per_rank: int = 0,
                 backend: Optional[str] = None) -> None:
        """``backend``: ``"fused"`` (push exchange over NVLink peer memory; CUDA with more than one rank, the default there)
        or ``"collective"`` (``torch.distributed`` all-to-all; any device).  ``max_ids_per_rank`` bounds the ids one rank
        sends per table and step on the fused backend (0: 1.5 x the largest first batch over all ranks)."""
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
            cap = aligned_capacity_per_rank(t.num_embeddings, self.world, o.bucket_capacity)
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
        self.max_ids_per_rank = int(max_ids_per_rank)
        cuda_multi = self.world > 1 and self.device.type == "cuda"
        self.backend = backend or ("fused" if cuda_multi and all(t.storage is None for t in self.lookup.tables)
                                   and all(d % 8 == 0 for d in self.dims) else "collective")
        if self.backend == "fused" and not cuda_multi:
            self.backend = "collective"
        self.peer = peer
        self._exchanges: Dict[int, object] = {}
        if self.backend == "fused" and self.peer is None:
            from ..parallel.comm import PeerGroup

            self.peer = PeerGroup(self.pg, self.device)

    # -- table groups: features of one table are adjacent in the key order -------------------------------
    def _groups(self, lpk: List[int]):
        """-> [(table index, first feature, one-past-last feature, first id, number of ids)]"""
        out, f, start, F = [], 0, 0, len(self.feature_names)
        while f < F:
            ti, f1 = self.feature_table[f], f
            while f1 < F and self.feature_table[f1] == ti:
                f1 += 1
            n = sum(lpk[f:f1])
            out.append((ti, f, f1, start, n))
            start += n
            f = f1
        tabs = [g[0] for g in out]
        if len(set(tabs)) != len(tabs):
            raise ValueError("features of one table must be adjacent in the feature order")
        return out

    def _exchange(self, ti: int, n: int):
        """The fused exchange of table ``ti``, created on first use (a collective set-up step: every rank arrives here
        with the same table at its first batch)."""
        ex = self._exchanges.get(ti)
        if ex is None:
            from .fused_exchange import FusedDynamicExchange, owned_capacity

            cap_n = self.max_ids_per_rank
            if not cap_n:
                t = torch.tensor([n], dtype=torch.int64, device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.pg)
                cap_n = int(int(t[0]) * 1.5) + 1024
            cap_n = (cap_n + 7) // 8 * 8
            ex = FusedDynamicExchange(self.peer, self.lookup.tables[ti], self.device, cap_n,
                                      owned_capacity(cap_n, self.world), self.output_dtype)
            self._exchanges[ti] = ex
        if n > ex.px.nnz_cap:
            raise ValueError("table %s: %d ids in one batch, the exchange was sized for %d (max_ids_per_rank)"
                             % (self.lookup.table_names[ti], n, ex.px.nnz_cap))
        return ex

    def _fused_sequence_rows(self, features: KeyedJaggedTensor) -> torch.Tensor:
        from .fused_exchange import _FusedRowsFn

        ids = features.values().to(self.device).long().contiguous()
        lk = self.lookup
        if lk.training:
            lk._update_score()
        outs = []
        for ti, _f0, _f1, start, n in self._groups(features.length_per_key()):
            ex = self._exchange(ti, n)
            outs.append(_FusedRowsFn.apply(lk._anchor, ex, ids[start:start + n], lk.training))
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=0)

    # -- rows for every id of the local KJT, in the KJT's own order: [nnz, D] ------------------------
    def _sequence_rows(self, features: KeyedJaggedTensor) -> torch.Tensor:
        assert features.keys() == self.feature_names
        F = len(self.feature_names)
        ids = features.values().to(self.device).long()
        lpk = features.length_per_key()
        if self.world == 1:
            return self.lookup(ids, None, lpk, features.stride())
        if self.backend == "fused":
            return self._fused_sequence_rows(features)
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
        if self.backend == "fused":
            return self._forward_fused(features)
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

    def _forward_fused(self, features: KeyedJaggedTensor) -> KeyedTensor:
        """Several ranks on CUDA: one push exchange per table, pooled on the requesting GPU from the received rows."""
        from .fused_exchange import _FusedPooledFn

        assert features.keys() == self.feature_names
        B = features.stride()
        ids = features.values().to(self.device).long().contiguous()
        offsets = features.offsets().to(self.device).long()
        lk = self.lookup
        if lk.training:
            lk._update_score()
        outs = []
        for ti, f0, f1, start, n in self._groups(features.length_per_key()):
            ex = self._exchange(ti, n)
            off = (offsets[f0 * B:f1 * B + 1] - start).contiguous()
            mean = getattr(self.configs[ti], "pooling", PoolingType.SUM) == PoolingType.MEAN
            outs.append(_FusedPooledFn.apply(lk._anchor, ex, ids[start:start + n], off, f1 - f0, B, mean, lk.training,
                                             self.output_dtype))
        feature_dims = [self.dims[t] for t in self.feature_table]
        return KeyedTensor(self.feature_names, feature_dims, outs[0] if len(outs) == 1 else torch.cat(outs, dim=1))

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

"""Sequence (non-pooled) multi-tier embeddings: ``EmbCacheEmbeddingCollection`` and its sharded form.

Same tiers and swap as the bag collection (``embedding_bag.py``); the output is one row per id, returned to the rank
that owns the sample in the sample's own order: ``forward(kjt) -> Dict[feature, JaggedTensor]``.
Reference: ``torchrec_embcache/distributed/embedding.py:184-306`` (module), ``:309-919`` (sharded module, not-admitted
ids ``:587-625``), ``sharding/rw_sequence_sharding.py:34-104``.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import embedding_ops as E
from ..parallel.collective_embeddingbag import _AllToAll
from ..parallel.comm import ShardingEnv
from ..sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor
from .configs import EmbCacheEmbeddingConfig
from .embedding_bag import EmbCacheEmbeddingBagCollection, EmbCacheShardedEmbeddingBagCollection


class EmbCacheEmbeddingCollection(EmbCacheEmbeddingBagCollection):
    def __init__(self, tables: List[EmbCacheEmbeddingConfig], world_size: int, batch_size: int, multi_hot_sizes: List[int],
                 need_accumulate_offset: bool = True, device=None, embedding_optimizer_cls=torch.optim.Adagrad) -> None:
        super().__init__(tables, world_size, batch_size, multi_hot_sizes, False, need_accumulate_offset, device, embedding_optimizer_cls)
        if len({t.embedding_dim for t in tables}) > 1:
            raise ValueError("EmbCacheEmbeddingCollection tables must share embedding_dim")

    def embedding_configs(self):
        return self.tables

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        if self._sharded is None:
            self._sharded = EmbCacheShardedEmbeddingCollection(self, ShardingEnv(1, 0, None), self.device, self.optimizer_spec())
        return self._sharded(features)


class _SeqLookup(torch.autograd.Function):
    """Rows of several cache tables for a list of (table, slot) pairs; the sparse update happens in backward."""

    @staticmethod
    def forward(ctx, anchor, mod, table_of: torch.Tensor, slots: torch.Tensor):
        D = mod.tables[0].embedding_dim
        out = torch.zeros(slots.numel(), D, dtype=torch.float32, device=slots.device)
        for ti, t in enumerate(mod.tables):
            sel = (table_of == ti).nonzero(as_tuple=True)[0]
            if sel.numel():
                out[sel] = mod.embedding_bags[t.name].weight.data.float().index_select(0, slots[sel])
        ctx.mod = mod
        ctx.save_for_backward(table_of, slots)
        return out

    @staticmethod
    def backward(ctx, g):
        table_of, slots = ctx.saved_tensors
        for ti in range(len(ctx.mod.tables)):
            sel = (table_of == ti).nonzero(as_tuple=True)[0]
            if sel.numel():
                ctx.mod._apply_update(ti, slots[sel], g[sel])
        return None, None, None, None


def local_unique_kjt(features: KeyedJaggedTensor) -> Tuple[KeyedJaggedTensor, torch.Tensor]:
    """Every feature's ids de-duplicated over the local batch: -> (KJT of the unique ids - all of a feature's ids sit in its
    first bag -, index of every original id in the reduced value list).  Host tensors."""
    F, B = len(features.keys()), features.stride()
    values = features.values().cpu().long()
    lpk = features.length_per_key()
    lengths = torch.zeros(F * B, dtype=torch.int64)
    uniq, inv, start, base = [], [], 0, 0
    for f, n in enumerate(lpk):
        u, i = torch.unique(values[start:start + n], return_inverse=True)
        uniq.append(u)
        inv.append(i + base)
        lengths[f * B] = u.numel()
        base += u.numel()
        start += n
    reduced = KeyedJaggedTensor(features.keys(), torch.cat(uniq) if uniq else values, lengths=lengths, stride=B)
    return reduced, (torch.cat(inv) if inv else torch.zeros(0, dtype=torch.int64))


class EmbCacheShardedEmbeddingCollection(EmbCacheShardedEmbeddingBagCollection):
    def __init__(self, module: EmbCacheEmbeddingBagCollection, env: ShardingEnv, device, optimizer_spec: Optional[E.OptimizerSpec] = None,
                 cache_rows: Optional[List[int]] = None, threads: int = 4) -> None:
        super().__init__(module, env, device, optimizer_spec, cache_rows, threads)
        self._perm: Dict[int, torch.Tensor] = {}
        self._sent: Dict[int, List[int]] = {}
        # DO_EC_LOCAL_UNIQUE (true / 1 / yes): every feature's ids are de-duplicated on the sending rank before the id
        # exchange, so an id that occurs many times in the local batch crosses the network once, is swapped in once and its
        # row comes back once (sequence embeddings only: torchrec_embcache/distributed/sharding/rw_sharding.py:109-111)
        self.do_local_unique = os.environ.get("DO_EC_LOCAL_UNIQUE", "False").lower() in ("true", "1", "yes")

    def _bucketize(self, features: KeyedJaggedTensor):
        if self.do_local_unique:
            reduced, inv = local_unique_kjt(features)
            nl, ni, perm_r = super()._bucketize(reduced)
            perm = perm_r[inv]                                 # bucket order of the unique ids -> every original position
        else:
            nl, ni, perm = super()._bucketize(features)
        self._perm[id(features)] = perm
        self._sent[id(features)] = nl.sum(dim=1).tolist()
        return nl, ni, perm

    def prefetch_async(self, features_dev: KeyedJaggedTensor, features_host: KeyedJaggedTensor) -> None:
        super().prefetch_async(features_dev, features_host)
        ctx = self._prepared[id(features_dev)]
        self._prepared[id(features_dev)] = ctx[:4] + (self._perm.pop(id(features_host)), ctx[4])
        self._sent[id(features_dev)] = self._sent.pop(id(features_host))

    def _prepare(self, features: KeyedJaggedTensor):
        ctx = super()._prepare(features)
        return ctx + (self._perm.pop(id(features)),)

    def forward(self, features: KeyedJaggedTensor) -> Dict[str, JaggedTensor]:
        ctx = self._prepared.pop(id(features), None)
        ev = None
        if ctx is None:
            lengths, slots, B, orig, perm = self._prepare(features)
        else:
            lengths, slots, B, orig, perm, ev = ctx
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
        self._step += 1
        W, F, _ = lengths.shape
        per_seg = lengths.sum(dim=2).reshape(-1)                                  # ids per (source, feature)
        seg_table = torch.tensor([self.feature_table[f] for f in range(F)] * W, device=slots.device)
        table_of = torch.repeat_interleave(seg_table, per_seg.to(slots.device))
        rows = _SeqLookup.apply(self._anchor, self, table_of, slots)
        if self.world > 1:
            to_src = lengths.view(W, -1).sum(dim=1).tolist()                      # what each source sent here
            mine = features.lengths().view(F, B)
            # what this rank sent to each owner = what comes back from it
            sent = self._sent_counts(features)
            rows = _AllToAll.apply(rows, sent, to_src, self.pg)
        rows = rows[perm.to(rows.device)]                                         # bucket order -> the KJT's own order
        out: Dict[str, JaggedTensor] = {}
        start = 0
        lens = features.lengths().to(self.device)
        for f, (name, n) in enumerate(zip(self.feature_names, features.length_per_key())):
            out[name] = JaggedTensor(rows[start:start + n].to(self.out_dtype), lengths=lens[f * B:(f + 1) * B])
            start += n
        return out

    def _sent_counts(self, features: KeyedJaggedTensor) -> List[int]:
        sent = self._sent.pop(id(features), None)              # recorded when the batch was bucketized
        if sent is not None:
            return sent
        dest = torch.remainder(features.values().cpu().long(), self.world)
        return torch.bincount(dest, minlength=self.world).tolist()


class EmbCacheEmbeddingCollectionSharder:
    def __init__(self, cpu_device=None, cpu_env: Optional[ShardingEnv] = None, npu_device=None, npu_env: Optional[ShardingEnv] = None,
                 fused_params: Optional[dict] = None, qcomm_codecs_registry=None) -> None:
        self.device, self.env = npu_device, npu_env
        self.fused_params = dict(fused_params or {})

    def sharding_types(self, compute_device_type: str = "cuda") -> List[str]:
        return ["row_wise"]

    @property
    def module_type(self):
        return EmbCacheEmbeddingCollection

    def shard(self, module: EmbCacheEmbeddingCollection, params=None, env: Optional[ShardingEnv] = None, device=None):
        spec = module.optimizer_spec(**{k: v for k, v in self.fused_params.items() if k in ("lr", "eps", "beta1", "beta2", "weight_decay")})
        return EmbCacheShardedEmbeddingCollection(module, env or self.env or ShardingEnv(1, 0, None),
                                                  device or self.device or module.device, spec)

"""``KeyValueTable``: one dynamic embedding table with its optional tiers.

* plain:     one ``HKVTable`` (values in HBM, optionally spilling into pinned host DRAM that the kernels
             address directly - ``local_hbm_for_values`` decides how many rows stay in HBM);
* caching:   a small HBM ``HKVTable`` in front of a ``Storage`` (a host-resident table or an external
             storage such as the disk tier): misses are fetched from storage, inserted into the cache and
             whatever the cache evicts is written back;
* admission: a key becomes resident on its ``admit_threshold``-th sighting (probation counters live in a
             value-less LFU table); until then lookups return the default value and updates are dropped.

No per-table host synchronisation happens on the plain training path (the reference syncs with
``.item()`` several times per table per step, ``dynamic_emb/distributed/key_value_table.py:260-261,282,355``).
Storage / cache interfaces follow ``dynamic_emb/distributed/types.py:51-227``; file formats follow
``key_value_table.py:385-415,565-575`` and ``batched_dynamicemb_table.py:176-184``.
"""
from __future__ import annotations

import abc
import json
import os
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .dynamicemb_config import DynamicEmbScoreStrategy, DynamicEmbTableOptions
from .hkv import (ST_REJECTED, EvictStrategy, HKVTable, HostDynamicTable, InitializerArgs, InitMode, OptimizerType,
                  opt_state_dim)


class Storage(abc.ABC):
    """Tier below the cache: addressed by key, holds full rows ``[embedding | optimizer state]``."""

    @abc.abstractmethod
    def find(self, keys: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """-> (rows [n, row_dim] fp32 on the keys' device, found mask)."""

    @abc.abstractmethod
    def insert(self, keys: torch.Tensor, rows: torch.Tensor, scores: Optional[torch.Tensor] = None) -> None: ...

    @abc.abstractmethod
    def export_all(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """-> (keys, rows, scores) on the host."""

    def erase(self, keys: torch.Tensor) -> None:  # optional
        return None

    def size(self) -> int:
        return int(self.export_all()[0].numel())


class Cache(abc.ABC):
    """Contract of a device-side cache in front of a ``Storage`` (``dynamic_emb/distributed/types.py:152-227`` of the
    reference): lookups report the keys they missed, inserts report what they evicted."""

    @abc.abstractmethod
    def find(self, unique_keys: torch.Tensor, unique_vals: torch.Tensor, founds: Optional[torch.Tensor] = None
             ) -> Tuple[int, torch.Tensor, torch.Tensor]:
        """Fill ``unique_vals`` rows of the resident keys -> (number missing, missing keys, their positions)."""

    @abc.abstractmethod
    def insert_and_evict(self, keys: torch.Tensor, values: torch.Tensor) -> Tuple[int, torch.Tensor, torch.Tensor, torch.Tensor]:
        """-> (number evicted, evicted keys, evicted rows, evicted scores)."""

    @abc.abstractmethod
    def flush(self, storage: Optional[Storage] = None) -> None: ...

    @abc.abstractmethod
    def reset(self) -> None: ...


class TableStorage(Storage):
    """Storage backed by another table object (host-resident ``HKVTable`` or ``HostDynamicTable``)."""

    def __init__(self, table) -> None:
        self.table = table

    def find(self, keys):
        slots, found = self.table.find(keys)
        return self.table.gather(slots, 0, self.table.row_dim), found

    def insert(self, keys, rows, scores=None) -> None:
        self.table.insert_and_evict(keys, rows, scores)

    def export_all(self):
        k, s, v, _ = self.table.export_batch()
        return k.cpu(), v.cpu(), s.cpu()

    def erase(self, keys) -> None:
        self.table.erase(keys)

    def size(self) -> int:
        return self.table.size()


class DiskStorage(Storage):
    """External storage on the log-structured disk tier (``csrc/host/disk_tier.h``)."""

    def __init__(self, name: str, paths: List[str], row_dim: int, max_bytes_per_path: int = 0, engine=None) -> None:
        from ..host import host

        self.name, self.row_dim = name, row_dim
        self.engine = engine or host().DiskEngine()
        if not self.engine.has_table(name):
            self.engine.create_table(name, paths, row_dim, max_bytes_per_path)
        self._scores: Dict[int, int] = {}

    def find(self, keys):
        from ..host import host

        rc, rows, found = self.engine.fetch(self.name, keys.cpu().numpy().astype(np.int64), self.row_dim)
        if rc != host().DISK_OK:
            raise RuntimeError("disk tier fetch failed (code %d)" % rc)
        return torch.from_numpy(rows).to(keys.device), torch.from_numpy(found.astype(np.bool_)).to(keys.device)

    def insert(self, keys, rows, scores=None) -> None:
        from ..host import host

        rc = self.engine.insert(self.name, keys.cpu().numpy().astype(np.int64), rows.float().cpu().numpy())
        if rc == host().DISK_SPACE_NOT_ENOUGH:
            raise RuntimeError("disk tier: no space left on any configured path")
        if rc != host().DISK_OK:
            raise RuntimeError("disk tier insert failed (code %d)" % rc)
        if scores is not None:
            for k, s in zip(keys.tolist(), scores.tolist()):
                self._scores[k] = s

    def export_all(self):
        keys = torch.from_numpy(self.engine.export_keys(self.name).astype(np.int64))
        rows, _ = self.find(keys)
        scores = torch.tensor([self._scores.get(k, 0) for k in keys.tolist()], dtype=torch.int64)
        return keys, rows.cpu(), scores

    def erase(self, keys) -> None:
        self.engine.erase(self.name, keys.cpu().numpy().astype(np.int64))

    def size(self) -> int:
        return int(self.engine.size(self.name))


def file_names(save_dir: str, table: str, rank: int, world: int) -> Dict[str, str]:
    sfx = ".rank_%d.world_size_%d" % (rank, world)
    return {k: os.path.join(save_dir, "%s_emb_%s%s" % (table, k, sfx)) for k in ("keys", "values", "scores", "opt_values")}


class KeyValueTable(Cache):
    def __init__(self, name: str, options: DynamicEmbTableOptions, device: torch.device, lr: float = 0.01,
                 eps: float = 1e-8, betas=(0.9, 0.999), weight_decay: float = 0.0, seed: int = 0,
                 initial_accumulator_value: float = 0.0) -> None:
        o = options
        self.name, self.options, self.device = name, o, torch.device(device)
        self.dim = o.dim
        self.optimizer = OptimizerType(o.optimizer_type)
        self.state_dim = opt_state_dim(self.optimizer, self.dim)
        self.row_dim = self.dim + self.state_dim
        self.lr, self.eps, self.betas, self.weight_decay = lr, eps, betas, weight_decay
        self._step = 0                 # optimizer iterations ("iters" in the opt-args file)
        self.score_value = 1           # STEP / CUSTOMIZED score for the current step
        init = o.initializer_args.to_native(o.max_capacity or 0, seed)
        init.state_init = initial_accumulator_value if self.optimizer in (OptimizerType.ADAGRAD, OptimizerType.ROWWISE_ADAGRAD) else 0.0
        self._init = init
        cap = o.init_capacity or o.max_capacity or 1024
        max_cap = o.max_capacity or cap
        cuda = self.device.type == "cuda"
        hbm_rows = None
        if cuda and o.local_hbm_for_values > 0:
            hbm_rows = max(128, int(o.local_hbm_for_values // (4 * self.row_dim)))
        kw = dict(optimizer=self.optimizer, evict_strategy=o.evict_strategy, init=init)
        if cuda:
            self.table = HKVTable(self.dim, cap, self.device, max_capacity=max_cap, max_load_factor=o.max_load_factor,
                                  hbm_rows=hbm_rows, **kw)
        else:
            self.table = HostDynamicTable(self.dim, max_cap, **kw)
        self.storage: Optional[Storage] = None
        if o.caching:
            if o.external_storage is not None:
                self.storage = o.external_storage
            elif cuda:
                self.storage = TableStorage(HKVTable(self.dim, max(max_cap * 8, 1024), self.device, hbm_rows=0, **kw))
            else:
                self.storage = TableStorage(HostDynamicTable(self.dim, max_cap * 8, **kw))
        self.probation = None
        if o.admit_threshold and o.admit_threshold > 1:
            pkw = dict(optimizer=OptimizerType.SGD, evict_strategy=EvictStrategy.LFU, init=InitializerArgs(mode=InitMode.CONSTANT))
            self.probation = HKVTable(0, max_cap, self.device, **pkw) if cuda else HostDynamicTable(0, max_cap, **pkw)
        # lookups, hits, storage hits, inserts, evictions (cf. KeyValueTable._cache_metrics)
        self.metrics = {"lookups": 0, "cache_hits": 0, "storage_hits": 0, "inserts": 0, "evictions": 0}
        self.record_metrics = False
        self._touched: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ scores
    def _scores_for(self, n: int) -> Optional[torch.Tensor]:
        st = self.options.score_strategy
        if st == DynamicEmbScoreStrategy.TIMESTAMP:
            return None
        v = 1 if st == DynamicEmbScoreStrategy.LFU else self.score_value
        return torch.full((n,), int(v), dtype=torch.int64, device=self.device)

    # ------------------------------------------------------------------ lookup
    def lookup(self, unique_keys: torch.Tensor, training: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
        """-> (slots, rows [U, dim] fp32).  ``slots == -1`` marks keys that are not resident (eval miss or not
        admitted); their rows hold the default value."""
        t = self.table
        n = unique_keys.numel()
        default = self.options.eval_initializer_args.value
        if not training:
            slots, found = t.find(unique_keys)
            rows = t.gather(slots, 0, self.dim, missing_value=default)
            if self.storage is not None and n:
                miss = ~found
                if bool(miss.any()):
                    srows, sfound = self.storage.find(unique_keys[miss])
                    fill = torch.where(sfound[:, None], srows[:, : self.dim], torch.full_like(srows[:, : self.dim], default))
                    rows[miss] = fill
            return slots, rows
        keys = unique_keys
        admitted_mask = None
        if self.probation is not None and n and self.storage is None:
            return self._lookup_with_admission(unique_keys, default)
        if self.probation is not None and n:
            _, resident = t.find(keys)
            cand = keys[~resident]
            if cand.numel():
                pslots, _, _ = self.probation.find_or_insert(cand)
                if isinstance(self.probation, HKVTable):
                    counts = self.probation.scores[pslots.clamp(min=0)]
                else:
                    counts = torch.tensor([self.probation.score.get(k, 0) for k in cand.tolist()], dtype=torch.int64)
                ok = counts >= self.options.admit_threshold
                self.probation.erase(cand[ok])
                admitted_mask = resident.clone()
                admitted_mask[~resident] = ok.to(admitted_mask.device)
            else:
                admitted_mask = resident
            keys = torch.where(admitted_mask, keys, torch.full_like(keys, -1))   # -1 = empty key: skipped
        if self.storage is None:
            slots, status, _ = t.find_or_insert(keys, self._scores_for(n))
        else:
            slots = self._caching_lookup(keys)
        rows = t.gather(slots, 0, self.dim, missing_value=default)
        if self.record_metrics:
            self.metrics["lookups"] += n
        if self.options.training:
            self._touched = unique_keys if self._touched is None else torch.cat([self._touched, unique_keys])
        return slots, rows

    def _admit(self, keys: torch.Tensor, resident: torch.Tensor) -> torch.Tensor:
        """Keys that are not resident are counted on probation; -> mask of the ones that reach ``admit_threshold`` now
        (they leave the probation table).  Masks only: no boolean indexing, no host synchronisation."""
        empty = torch.full_like(keys, -1)
        cand = torch.where(resident, empty, keys)
        pslots, _, _ = self.probation.find_or_insert(cand)
        if isinstance(self.probation, HKVTable):
            counts = self.probation.scores[pslots.clamp(min=0)]
        else:
            counts = torch.tensor([self.probation.score.get(k, 0) for k in cand.tolist()], dtype=torch.int64)
        ok = (counts >= self.options.admit_threshold) & (pslots >= 0)
        self.probation.erase(torch.where(ok, cand, empty))
        return ok

    def _find_then_insert(self, keys: torch.Tensor) -> torch.Tensor:
        """Slots of ``keys`` with admission: ONE lock-free pass finds the resident keys, refreshes their scores and stamps
        their slots; only the keys admitted now go through the locked insert (same launch stamp, so it cannot evict what
        the first pass found)."""
        t, n = self.table, keys.numel()
        scores = self._scores_for(n)
        slots, resident = t.find(keys, update_score=True, scores=scores, stamp=True)
        ok = self._admit(keys, resident)
        new_slots, _status, _ = t.find_or_insert(torch.where(ok, keys, torch.full_like(keys, -1)), scores, keep_epoch=True)
        return torch.where(resident, slots, new_slots)

    def _lookup_with_admission(self, unique_keys: torch.Tensor, default: float) -> Tuple[torch.Tensor, torch.Tensor]:
        slots = self._find_then_insert(unique_keys)
        rows = self.table.gather(slots, 0, self.dim, missing_value=default)
        if self.record_metrics:
            self.metrics["lookups"] += unique_keys.numel()
        if self.options.training:
            self._touched = unique_keys if self._touched is None else torch.cat([self._touched, unique_keys])
        return slots, rows

    def lookup_slots_padded(self, keys: torch.Tensor, training: bool = True) -> torch.Tensor:
        """Slots of a fixed-size key list whose unused entries hold the empty key (-1): no boolean indexing, no host
        synchronisation (the table must not be able to grow any more: ``init_capacity == max_capacity``).  Admission on the
        ``admit_threshold``-th sighting works on masks: keys on probation are replaced by the empty key, which every table
        kernel skips.  Not available for tables with a storage tier below them."""
        if self.storage is not None:
            raise NotImplementedError("padded lookups do not serve tables with a storage tier")
        t = self.table
        if not training:
            return t.find(keys)[0]
        n = keys.numel()
        if self.probation is not None and n:
            slots = self._find_then_insert(keys)
        else:
            slots, _status, _ = t.find_or_insert(keys, self._scores_for(n))
        if self.options.training:
            self._touched = keys if self._touched is None else torch.cat([self._touched, keys])
        return slots

    def _caching_lookup(self, keys: torch.Tensor) -> torch.Tensor:
        """cache.find -> storage.find for the misses -> insert_and_evict into the cache -> evicted rows back
        to storage (``KeyValueTableCachingFunction.lookup``, ``key_value_table.py:803-864``)."""
        t = self.table
        slots, found = t.find(keys, update_score=True, scores=self._scores_for(keys.numel()))
        miss = (~found) & (keys != -1)
        if bool(miss.any()):
            mk = keys[miss]
            srows, sfound = self.storage.find(mk)
            mslots, status, ev = t.find_or_insert(mk, self._scores_for(mk.numel()), evict_cap=mk.numel())
            hit = sfound & (mslots >= 0)
            if bool(hit.any()):
                t.scatter(mslots[hit], srows[hit], 0, self.row_dim)          # full row incl. optimizer state
            slots = slots.clone()
            slots[miss] = mslots
            n_ev = int(ev[3].item()) if ev is not None else 0
            if n_ev:
                self.storage.insert(ev[0][:n_ev], ev[2][:n_ev], ev[1][:n_ev])
            if self.record_metrics:
                self.metrics["storage_hits"] += int(sfound.sum().item())
                self.metrics["inserts"] += int(mk.numel())
                self.metrics["evictions"] += n_ev
        if self.record_metrics:
            self.metrics["cache_hits"] += int(found.sum().item())
        return slots

    # ------------------------------------------------------------------ update
    def update(self, slots: torch.Tensor, grads: torch.Tensor) -> None:
        self._step += 1
        self.table.update(slots, grads, self.lr, self.eps, self.betas[0], self.betas[1], self.weight_decay, self._step)

    def flush(self, storage: Optional[Storage] = None) -> None:
        """Write every cached row back to ``storage`` (default: this table's own storage tier; before a dump)."""
        storage = storage if storage is not None else self.storage
        if storage is None:
            return
        k, s, v, _ = self.table.export_batch()
        if k.numel():
            storage.insert(k, v, s)

    def size(self) -> int:
        return self.table.size() + (self.storage.size() if self.storage is not None else 0)

    # ------------------------------------------------------------------ export / dump / load
    def export_keys_values(self, min_score: Optional[int] = None):
        """-> host (keys, rows [n,row_dim], scores); cache entries override storage entries."""
        k, s, v, _ = self.table.export_batch(min_score=min_score)
        k, s, v = k.cpu(), s.cpu(), v.cpu()
        if self.storage is not None:
            sk, sv, ss = self.storage.export_all()
            if min_score is not None and sk.numel():
                keep = ss >= min_score
                sk, sv, ss = sk[keep], sv[keep], ss[keep]
            if sk.numel():
                cached = set(k.tolist())
                keep = torch.tensor([x not in cached for x in sk.tolist()], dtype=torch.bool)
                k, v, s = torch.cat([k, sk[keep]]), torch.cat([v, sv[keep]]), torch.cat([s, ss[keep]])
        return k, v, s

    def dump(self, save_dir: str, rank: int, world: int, optim: bool = True) -> None:
        os.makedirs(save_dir, exist_ok=True)
        self.flush()
        k, v, s = self.export_keys_values()
        if self.options.evict_strategy == EvictStrategy.LRU and k.numel():
            now = self.table.device_timestamp() if isinstance(self.table, HKVTable) else getattr(self.table, "_clock", 0)
            s = now - s                                   # stored as an age, restored relative to load time
        f = file_names(save_dir, self.name, rank, world)
        k.numpy().astype("<i8").tofile(f["keys"])
        v[:, : self.dim].contiguous().numpy().astype("<f4").tofile(f["values"])
        s.numpy().astype("<i8").tofile(f["scores"])
        if optim:
            v[:, self.dim:].contiguous().numpy().astype("<f4").tofile(f["opt_values"])
        if rank == 0:
            args = {"optimizer": self.optimizer.name, "lr": self.lr, "eps": self.eps, "beta1": self.betas[0],
                    "beta2": self.betas[1], "weight_decay": self.weight_decay, "iters": self._step,
                    "evict_strategy": EvictStrategy(self.options.evict_strategy).name, "dim": self.dim,
                    "opt_state_dim": self.state_dim}
            with open(os.path.join(save_dir, "%s_opt_args.json" % self.name), "w") as fh:
                json.dump(args, fh)

    def load(self, save_dir: str, rank: int, world: int, optim: bool = True) -> int:
        """Reads this rank's file when the world size matches, else every file, keeping ``key % world == rank``.
        Optimizer mismatch -> optimizer state is skipped; evict-strategy mismatch -> error."""
        meta_path = os.path.join(save_dir, "%s_opt_args.json" % self.name)
        meta = json.load(open(meta_path)) if os.path.exists(meta_path) else {}
        if meta and meta.get("evict_strategy") != EvictStrategy(self.options.evict_strategy).name:
            raise ValueError("evict strategy of the checkpoint (%s) differs from the table's (%s)"
                             % (meta.get("evict_strategy"), EvictStrategy(self.options.evict_strategy).name))
        use_opt = optim and meta.get("optimizer") == self.optimizer.name and meta.get("opt_state_dim") == self.state_dim
        if use_opt:
            self._step = int(meta.get("iters", 0))
        files = []
        for fn in sorted(os.listdir(save_dir)):
            if fn.startswith(self.name + "_emb_keys.rank_"):
                r, w = fn.split(".rank_")[1].split(".world_size_")
                files.append((int(r), int(w)))
        same = [(r, w) for r, w in files if w == world and r == rank]
        todo = same if (same and all(w == world for _r, w in files)) else files
        total = 0
        for r, w in todo:
            f = file_names(save_dir, self.name, r, w)
            k = torch.from_numpy(np.fromfile(f["keys"], dtype="<i8").astype(np.int64))
            if k.numel() == 0:
                continue
            v = torch.from_numpy(np.fromfile(f["values"], dtype="<f4")).view(-1, self.dim)
            s = torch.from_numpy(np.fromfile(f["scores"], dtype="<i8").astype(np.int64))
            rows = torch.zeros(k.numel(), self.row_dim)
            rows[:, : self.dim] = v
            if use_opt and os.path.exists(f["opt_values"]) and self.state_dim:
                rows[:, self.dim:] = torch.from_numpy(np.fromfile(f["opt_values"], dtype="<f4")).view(-1, self.state_dim)
            keep = (k % world) == rank if not (w == world and r == rank and todo is same) else torch.ones_like(k, dtype=torch.bool)
            k, rows, s = k[keep], rows[keep], s[keep]
            if self.options.evict_strategy == EvictStrategy.LRU:
                now = self.table.device_timestamp() if isinstance(self.table, HKVTable) else 0
                s = torch.clamp(now - s, min=0)
            for i in range(0, k.numel(), 65536):
                kk = k[i:i + 65536].to(self.device)
                target = self.storage if self.storage is not None else None
                if target is not None:
                    target.insert(kk, rows[i:i + 65536].to(self.device), s[i:i + 65536].to(self.device))
                else:
                    self.table.maybe_grow(kk.numel())
                    self.table.insert_and_evict(kk, rows[i:i + 65536].to(self.device), s[i:i + 65536].to(self.device))
            total += int(k.numel())
        return total

    # ------------------------------------------------------------------ key-addressed calls under the reference's names
    # (``dynamic_emb/distributed/key_value_table.py:228-690``: find / insert / insert_and_evict / scores / shape queries)
    def find(self, unique_keys: torch.Tensor, unique_vals: torch.Tensor, founds: Optional[torch.Tensor] = None
             ) -> Tuple[int, torch.Tensor, torch.Tensor]:
        """Rows ``[embedding | state]`` (as many columns as ``unique_vals`` has) of the resident keys are written into
        ``unique_vals``; rows of absent keys are left as they are.  ``founds`` (bool, optional) receives the hit mask.
        -> (number missing, missing keys, their positions in ``unique_keys``).  Nothing is inserted."""
        slots, found = self.table.find(unique_keys, update_score=True, scores=self._scores_for(unique_keys.numel()))
        cols = unique_vals.shape[1]
        if cols:
            rows = self.table.gather(slots, 0, cols)
            unique_vals.copy_(torch.where(found[:, None], rows.to(unique_vals.dtype), unique_vals))
        if founds is not None:
            founds.copy_(found)
        missing = ~found
        idx = torch.nonzero(missing, as_tuple=True)[0]
        return int(idx.numel()), unique_keys[missing], idx

    def find_embeddings(self, unique_keys: torch.Tensor, unique_embs: torch.Tensor, founds: Optional[torch.Tensor] = None):
        return self.find(unique_keys, unique_embs, founds)

    def find_missed_keys(self, unique_keys: torch.Tensor, founds: Optional[torch.Tensor] = None):
        return self.find(unique_keys, torch.empty(unique_keys.numel(), 0, device=unique_keys.device), founds)

    def insert(self, keys: torch.Tensor, values: torch.Tensor, scores: Optional[torch.Tensor] = None) -> None:
        """Insert or overwrite full rows (``values`` ``[n, <= row_dim]``); scores default to the table's current score."""
        if scores is None:
            scores = self._scores_for(keys.numel())
        self.table.insert_and_evict(keys, values.float(), scores)

    def insert_and_evict(self, keys: torch.Tensor, values: torch.Tensor) -> Tuple[int, torch.Tensor, torch.Tensor, torch.Tensor]:
        _slots, _status, ev = self.table.insert_and_evict(keys, values.float(), self._scores_for(keys.numel()))
        n = int(ev[3].item()) if ev is not None else 0
        if self.record_metrics:
            self.metrics["inserts"] += int(keys.numel())
            self.metrics["evictions"] += n
        if n == 0:
            return 0, keys[:0], values[:0], torch.zeros(0, dtype=torch.int64, device=keys.device)
        return n, ev[0][:n], ev[2][:n], ev[1][:n]

    def update_by_keys(self, keys: torch.Tensor, grads: torch.Tensor, return_missing: bool = True):
        """The reference's ``update(keys, grads)``: fused optimizer on the rows of the resident keys
        -> (number missing, missing keys, their positions) or three Nones.  (``update`` here takes slots.)"""
        slots, found = self.table.find(keys)
        self.update(slots, grads)
        if not return_missing:
            return None, None, None
        idx = torch.nonzero(~found, as_tuple=True)[0]
        return int(idx.numel()), keys[~found], idx

    def enable_update(self) -> bool:
        return True

    def set_score(self, score: int) -> None:
        self.score_value = int(score)

    score_update = False              # True while a lookup may refresh scores only (kept for API parity; unused here)

    def update_timestamp(self) -> None:
        self._timestamp = self.table.device_timestamp() if isinstance(self.table, HKVTable) else getattr(self.table, "_clock", 0)

    def embedding_dtype(self) -> torch.dtype:
        return self.options.embedding_dtype

    def embedding_dim(self) -> int:
        return self.dim

    def value_dim(self) -> int:
        return self.row_dim

    def optim_state_dim(self) -> int:
        return self.state_dim

    def init_optimizer_state(self) -> float:
        return float(self._init.state_init)

    def key_type(self) -> torch.dtype:
        return self.options.index_type

    def value_type(self) -> torch.dtype:
        return torch.float32

    def capacity(self) -> int:
        return int(self.options.max_capacity or getattr(self.table, "capacity", 0))

    def evict_strategy(self) -> EvictStrategy:
        return EvictStrategy(self.options.evict_strategy)

    def reset(self) -> None:
        """Drop every resident row (the storage tier, if any, is left alone)."""
        self.table.clear()
        if self.probation is not None:
            self.probation.clear()

    def cache_metrics(self) -> Optional[torch.Tensor]:
        """[lookups, cache hits, inserts, evictions, storage hits] when recording is on, else None."""
        if not self.record_metrics:
            return None
        m = self.metrics
        return torch.tensor([m["lookups"], m["cache_hits"], m["inserts"], m["evictions"], m["storage_hits"]], dtype=torch.long)

    def set_record_cache_metrics(self, record: bool) -> None:
        self.record_metrics = bool(record)

    def count_matched(self, threshold: int, num_matched: Optional[torch.Tensor] = None) -> int:
        """Resident entries whose score is at least ``threshold`` (also written into ``num_matched[0]`` when given)."""
        n = int(self.table.count_matched(int(threshold)))
        if num_matched is not None:
            num_matched.reshape(-1)[0] = n
        return n

    def export_batch_matched(self, threshold: int, batch_size: Optional[int] = None, search_offset: int = 0, d_count=None, d_keys=None,
                             d_vals=None):
        """Entries with score >= ``threshold`` among the slots ``[search_offset, search_offset + batch_size)``; written into
        the given buffers when there are any -> (keys, scores, rows, slots)."""
        k, sc, rows, slots = self.table.export_batch_matched(int(threshold), int(search_offset), batch_size)
        n = int(k.numel())
        if d_count is not None:
            d_count.reshape(-1)[0] = n
        if d_keys is not None and n:
            d_keys[:n] = k.to(d_keys.device)
        if d_vals is not None and n:
            d_vals[:n, : rows.shape[1]] = rows.to(d_vals.device, d_vals.dtype)
        return k, sc, rows, slots

    def take_touched(self) -> Optional[torch.Tensor]:
        t, self._touched = self._touched, None
        return t if t is None else t[t != -1]


# ----------------------------------------------------------------------------------------------------------------------
# Stateless forms (``key_value_table.py:691-947`` of the reference): the lookup / update protocol of a storage alone and of
# a cache in front of a storage, written over the two contracts above.
# ----------------------------------------------------------------------------------------------------------------------
def _storage_find(storage, keys: torch.Tensor, value_dim: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(rows, found) from either kind of lower tier: a ``Storage`` (``find(keys)``) or another key-value table (``find(keys, vals, founds)``)."""
    if isinstance(storage, Cache):
        vals = torch.zeros(keys.numel(), value_dim, device=keys.device)
        found = torch.zeros(keys.numel(), dtype=torch.bool, device=keys.device)
        storage.find(keys, vals, found)
        return vals, found
    return storage.find(keys)


def update_cache(cache: Cache, storage: Storage, missing_keys: torch.Tensor, missing_values: torch.Tensor) -> None:
    """Rows fetched from (or created in) the storage become resident; what the cache evicts for them goes back down."""
    if missing_keys.numel() == 0:
        return
    n, ek, ev, es = cache.insert_and_evict(missing_keys, missing_values)
    if n:
        storage.insert(ek, ev, es)


class KeyValueTableFunction:
    """One table without a cache tier."""

    @staticmethod
    def lookup(storage: "KeyValueTable", unique_keys: torch.Tensor, unique_embs: torch.Tensor, training: bool = True,
               initializer=None) -> None:
        """Embeddings of ``unique_keys`` into ``unique_embs``; while training absent keys are created (drawn by the table's
        own initialiser, or by ``initializer(buffer, indices, keys)`` when one is given), in evaluation they read as the
        evaluation default."""
        slots, rows = storage.lookup(unique_keys, training=training)
        unique_embs.copy_(rows.to(unique_embs.dtype))
        if training and initializer is not None:
            n, _keys, idx = storage.find_missed_keys(unique_keys)
            if n:
                initializer(unique_embs, idx, unique_keys[idx])

    @staticmethod
    def update(storage: "KeyValueTable", unique_keys: torch.Tensor, unique_grads: torch.Tensor) -> None:
        storage.update_by_keys(unique_keys, unique_grads, return_missing=False)


class KeyValueTableCachingFunction:
    """A cache table in front of a storage: hits are served by the cache, misses come up from the storage (or are created
    there), evictions are written back."""

    @staticmethod
    def lookup(cache: "KeyValueTable", storage: Storage, unique_keys: torch.Tensor, unique_embs: torch.Tensor, training: bool = True
               ) -> None:
        dim = unique_embs.shape[1]
        vals = torch.zeros(unique_keys.numel(), cache.value_dim(), device=unique_keys.device)
        n, mk, idx = cache.find(unique_keys, vals)
        if n:
            rows, found = _storage_find(storage, mk, cache.value_dim())
            rows = rows.to(vals.device).float()
            if training and not bool(found.all()):
                # new keys: the cache table draws them, then they are read back like any other row
                slots, _st, _ev = cache.table.find_or_insert(mk[~found], cache._scores_for(int((~found).sum())))
                rows[~found] = cache.table.gather(slots, 0, cache.value_dim())
            vals[idx] = rows[:, : vals.shape[1]]
            if training:
                update_cache(cache, storage, mk, rows)
        unique_embs.copy_(vals[:, :dim].to(unique_embs.dtype))

    @staticmethod
    def update(cache: "KeyValueTable", storage: Storage, unique_keys: torch.Tensor, unique_grads: torch.Tensor) -> None:
        n, mk, idx = cache.update_by_keys(unique_keys, unique_grads)
        if n and hasattr(storage, "update_by_keys"):
            storage.update_by_keys(mk, unique_grads[idx], return_missing=False)

    @staticmethod
    def prefetch(cache: "KeyValueTable", storage: Storage, unique_keys: torch.Tensor) -> int:
        """Bring the rows of ``unique_keys`` that the storage holds into the cache -> number of rows moved."""
        n, mk, _idx = cache.find_missed_keys(unique_keys)
        if not n:
            return 0
        rows, found = _storage_find(storage, mk, cache.value_dim())
        if not bool(found.any()):
            return 0
        update_cache(cache, storage, mk[found], rows[found].to(mk.device).float())
        return int(found.sum())


def encode_meta_json_file_path(root_path: str, table_name: str) -> str:
    return os.path.join(root_path, "%s_opt_args.json" % table_name)


def encode_checkpoint_file_path(root_path: str, table_name: str, rank, world_size, item: str) -> str:
    if item not in ("keys", "values", "scores", "opt_values"):
        raise ValueError("Invalid item '%s'. Must be one of: keys, values, scores, opt_values" % item)
    return os.path.join(root_path, "%s_emb_%s.rank_%s.world_size_%s" % (table_name, item, rank, world_size))


def find_files(root_path: str, table_name: str, suffix: str) -> Tuple[List[str], int]:
    """Checkpoint files of one kind (``emb_keys`` / ``emb_values`` / ``emb_scores`` / ``opt_values``) of a table, sorted by
    rank -> (paths, world size they were written with)."""
    import glob
    import re

    item = {"emb_keys": "keys", "emb_values": "values", "emb_scores": "scores", "opt_values": "opt_values"}.get(suffix)
    if item is None:
        raise RuntimeError("Invalid suffix: %s" % suffix)
    rx = re.compile(r"\.rank_(\d+)\.world_size_(\d+)$")
    hits = []
    for f in glob.glob(encode_checkpoint_file_path(root_path, table_name, "*", "*", item)):
        m = rx.search(f)
        if m:
            hits.append((int(m.group(1)), int(m.group(2)), f))
    hits.sort()
    worlds = {w for _r, w, _f in hits}
    if len(worlds) > 1:
        raise RuntimeError("files of table %s were written with different world sizes: %s" % (table_name, sorted(worlds)))
    return [f for _r, _w, f in hits], (worlds.pop() if worlds else 0)

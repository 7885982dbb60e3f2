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


class KeyValueTable:
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

    def flush(self) -> None:
        """Write every cached row back to storage (before a dump)."""
        if self.storage is None:
            return
        k, s, v, _ = self.table.export_batch()
        if k.numel():
            self.storage.insert(k, v, s)

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

    def take_touched(self) -> Optional[torch.Tensor]:
        t, self._touched = self._touched, None
        return t if t is None else t[t != -1]

"""GPU dynamic hash table (``csrc/cuda/hkv.cu``) and a host reference with the same interface.

``HKVTable`` is the type-erased table handle of the reference (``DynamicEmbTable`` /
``HKVVariable``, ``dynamic_emb/csrc/dynamic_variable_base.h:32-83``, ``hkv_variable.cpp:353-717``):
``find``, ``find_or_insert``, ``insert_and_evict``, ``assign``, ``accum_or_assign``, ``erase``, ``clear``,
``reserve``, ``export_batch[_if]``, ``size``, ``capacity``, plus slot-addressed ``gather`` (load from
pointer) and ``update`` (fused optimizer on pointers).  Value rows are ``[embedding | optimizer state]``;
rows beyond ``hbm_rows`` live in pinned host memory that the kernels address directly (the
host-DRAM tier).  Nothing here synchronises with the host except ``size()`` and ``export``.
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..ops import _lib

BUCKET = 128
EMPTY_KEY = -1          # 0xFFFF_FFFF_FFFF_FFFF as int64

ST_FOUND, ST_INSERTED, ST_EVICTED_OTHER, ST_REJECTED, ST_MISSING, ST_LOCK_TIMEOUT = range(6)


class EvictStrategy(enum.IntEnum):
    LRU = 0
    LFU = 1
    EPOCH_LRU = 2
    EPOCH_LFU = 3
    CUSTOMIZED = 4


class InitMode(enum.IntEnum):
    UNIFORM = 0
    NORMAL = 1
    TRUNCATED_NORMAL = 2
    CONSTANT = 3
    DEBUG = 4


class OptimizerType(enum.IntEnum):
    SGD = 0
    ROWWISE_ADAGRAD = 1
    ADAGRAD = 2
    ADAM = 3


def opt_state_dim(opt: OptimizerType, dim: int) -> int:
    """Optimizer-state floats stored behind the embedding in every row (row-wise Adagrad keeps one
    accumulator padded to 16 bytes, like the reference: ``hkv_variable.h:100-244``)."""
    return {OptimizerType.SGD: 0, OptimizerType.ROWWISE_ADAGRAD: 4, OptimizerType.ADAGRAD: dim,
            OptimizerType.ADAM: 2 * dim}[OptimizerType(opt)]


@dataclasses.dataclass
class InitializerArgs:
    mode: InitMode = InitMode.UNIFORM
    lower: float = -0.01
    upper: float = 0.01
    mean: float = 0.0
    std_dev: float = 1.0
    value: float = 0.0
    seed: int = 0
    state_init: float = 0.0


def _pow2_ceil(x: int) -> int:
    p = 1
    while p < x:
        p <<= 1
    return p


class _VariableInterface:
    """The remaining calls of the reference's table handle, stated over ``find`` / ``gather`` / ``export_batch``
    (dynamic_emb ``csrc/dynamic_variable_base.h:99-251`` of the reference: ``find_and_initialize``, ``export_batch_matched``,
    ``count_matched``)."""

    def find_and_initialize(self, keys: torch.Tensor, value: float = 0.0, dtype: torch.dtype = torch.float32):
        """Evaluation lookup: rows of resident keys, ``value`` for the others; nothing is inserted.  -> (rows, found)."""
        slots, found = self.find(keys)
        return self.gather(slots, dtype=dtype, missing_value=value), found

    def export_batch_matched(self, threshold: int, slot0: int = 0, count: Optional[int] = None, with_values: bool = True):
        """Entries whose score is at least ``threshold`` (the incremental-dump filter)."""
        return self.export_batch(slot0, count, min_score=int(threshold), with_values=with_values)

    def count_matched(self, threshold: int) -> int:
        return int(self.export_batch(0, None, min_score=int(threshold), with_values=False)[0].numel())


class HKVTable(_VariableInterface):
    def __init__(self, dim: int, capacity: int, device: torch.device, optimizer: OptimizerType = OptimizerType.SGD,
                 evict_strategy: EvictStrategy = EvictStrategy.LRU, max_capacity: Optional[int] = None,
                 max_load_factor: float = 0.5, hbm_rows: Optional[int] = None,
                 init: Optional[InitializerArgs] = None) -> None:
        self.device = torch.device(device)
        self.dim = int(dim)
        self.optimizer = OptimizerType(optimizer)
        self.state_dim = opt_state_dim(self.optimizer, dim)
        self.row_dim = self.dim + self.state_dim
        self.evict_strategy = EvictStrategy(evict_strategy)
        self.max_load_factor = float(max_load_factor)
        self.init = init or InitializerArgs()
        cap = max(BUCKET, _pow2_ceil(int(capacity)))
        self.max_capacity = max(cap, _pow2_ceil(int(max_capacity))) if max_capacity else cap
        self._hbm_rows_limit = None if hbm_rows is None else int(hbm_rows)
        self._alloc(cap)
        self.clear()

    # ------------------------------------------------------------------ storage
    def _alloc(self, cap: int) -> None:
        dev = self.device
        self.capacity = cap
        self.num_buckets = cap // BUCKET
        self.keys = torch.empty(cap, dtype=torch.int64, device=dev)
        self.scores = torch.empty(cap, dtype=torch.int64, device=dev)
        self.digests = torch.empty(cap, dtype=torch.uint8, device=dev)
        self.locks = torch.zeros(self.num_buckets, dtype=torch.int32, device=dev)
        hbm = cap if self._hbm_rows_limit is None else min(cap, self._hbm_rows_limit)
        self.hbm_rows = hbm
        self.values_hbm = torch.empty(max(hbm, 1) * self.row_dim, dtype=torch.float32, device=dev)
        host_rows = cap - hbm
        # host tier: pinned memory, addressed by the kernels through its device mapping
        self.values_host = torch.empty(max(host_rows, 1) * self.row_dim, dtype=torch.float32, pin_memory=True) \
            if host_rows > 0 else None
        self._size = torch.zeros(1, dtype=torch.int64, device=dev)
        # launch stamps: a slot handed out by a find_or_insert launch is not evicted by a later warp of the same launch
        self.touch = torch.zeros(cap, dtype=torch.int32, device=dev)
        self._epoch = 0
        if not hasattr(self, "_counters"):             # life-time counters survive growth
            self._counters = torch.zeros(4, dtype=torch.int64, device=dev)
        host_ptr = self.values_host.data_ptr() if self.values_host is not None else 0
        self._desc = np.asarray([self.keys.data_ptr(), self.scores.data_ptr(), self.digests.data_ptr(),
                                 self.locks.data_ptr(), self.values_hbm.data_ptr(), host_ptr, hbm, cap, self.num_buckets,
                                 self.row_dim, self.dim, int(self.evict_strategy), self._size.data_ptr(),
                                 self.touch.data_ptr(), 0, self._counters.data_ptr()], dtype=np.int64)

    def _d(self) -> int:
        return self._desc.ctypes.data

    def _st(self) -> int:
        return _lib.stream_ptr(self.device)

    def _sms(self) -> int:
        return _lib.num_sms(self.device)

    # ------------------------------------------------------------------ basic ops
    def clear(self) -> None:
        _lib.check(_lib.lib().rb_hkv_clear(self._d(), self._sms(), self._st()), "rb_hkv_clear")

    def size(self) -> int:
        return int(self._size.item())

    def load_factor(self) -> float:
        return self.size() / self.capacity

    def _probe(self, keys: torch.Tensor, insert: bool, update_score: bool, scores: Optional[torch.Tensor],
               evict_cap: int = 0, stamp: bool = False, keep_epoch: bool = False):
        keys = keys.contiguous()
        assert keys.dtype == torch.int64 and keys.device == self.device
        n = keys.numel()
        slots = torch.empty(n, dtype=torch.int64, device=self.device)
        status = torch.empty(n, dtype=torch.uint8, device=self.device)
        ev = None
        if evict_cap > 0:
            ev = (torch.empty(evict_cap, dtype=torch.int64, device=self.device),
                  torch.empty(evict_cap, dtype=torch.int64, device=self.device),
                  torch.empty(evict_cap, self.row_dim, dtype=torch.float32, device=self.device),
                  torch.zeros(1, dtype=torch.int32, device=self.device))
        if scores is not None:
            scores = scores.contiguous()
            assert scores.dtype == torch.int64 and scores.numel() == n
        i = self.init
        if (insert and not keep_epoch) or stamp:
            self._epoch = self._epoch % 0x7FFFFFFF + 1       # never 0: freshly allocated stamps are 0
            self._desc[14] = self._epoch
        rc = _lib.lib().rb_hkv_find_or_insert(
            self._d(), keys.data_ptr(), n, int(insert), int(bool(update_score)) | (2 if stamp else 0), _lib.ptr(scores),
            slots.data_ptr(),
            status.data_ptr(), int(i.mode), i.lower, i.upper, i.mean, i.std_dev, i.value, int(i.seed), i.state_init,
            ev[0].data_ptr() if ev else None, ev[1].data_ptr() if ev else None, ev[2].data_ptr() if ev else None,
            ev[3].data_ptr() if ev else None, evict_cap, self._sms(), _lib.status_tensor(self.device).data_ptr(),
            self._st())
        _lib.check(rc, "rb_hkv_find_or_insert")
        return slots, status, ev

    def find(self, keys: torch.Tensor, update_score: bool = False, scores: Optional[torch.Tensor] = None,
             stamp: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        """-> (slots [-1 when missing], found mask).  Takes no bucket locks (a find changes no key or slot; keep the launches
        on one table in one stream).  ``stamp`` opens a new launch stamp and marks the found slots with it: a following
        ``find_or_insert(..., keep_epoch=True)`` will not evict them - together the two calls are one find-or-insert in
        which only the (few) missing keys pay for locks."""
        slots, _status, _ = self._probe(keys, False, update_score, scores, stamp=stamp)
        return slots, slots >= 0

    def find_or_insert(self, keys: torch.Tensor, scores: Optional[torch.Tensor] = None, evict_cap: int = 0,
                       keep_epoch: bool = False):
        """-> (slots, status, evicted) where evicted = (keys, scores, rows, count) or None.  Keys must be
        distinct within one call.  Grows the table first when the load factor would exceed the limit.  ``keep_epoch``
        continues the launch stamp of the preceding ``find(..., stamp=True)``."""
        self.maybe_grow(keys.numel())
        return self._probe(keys, True, True, scores, evict_cap, keep_epoch=keep_epoch)

    def insert_and_evict(self, keys: torch.Tensor, values: torch.Tensor, scores: Optional[torch.Tensor] = None):
        """Insert (or overwrite) full rows; returns what had to be evicted to make room."""
        slots, status, ev = self._probe(keys, True, True, scores, evict_cap=max(keys.numel(), 1))
        self.scatter(slots, values, 0, values.shape[1])
        return slots, status, ev

    def assign(self, keys: torch.Tensor, values: torch.Tensor, col0: int = 0) -> torch.Tensor:
        """Overwrite columns of rows that already exist; returns the found mask."""
        slots, found = self.find(keys)
        self.scatter(slots, values, col0, values.shape[1])
        return found

    def accum_or_assign(self, keys: torch.Tensor, values: torch.Tensor, accum_or_assigns: torch.Tensor,
                        scores: Optional[torch.Tensor] = None) -> None:
        """Rows flagged ``True`` are accumulated into when present; rows flagged ``False`` are inserted /
        overwritten."""
        acc = accum_or_assigns.bool()
        if acc.any():
            slots, _ = self.find(keys[acc])
            self.scatter(slots, values[acc], 0, values.shape[1], accumulate=True)
        if (~acc).any():
            self.insert_and_evict(keys[~acc], values[~acc], None if scores is None else scores[~acc])

    # ------------------------------------------------------------------ pointers, pins, counters
    def _pointers(self, slots: torch.Tensor) -> torch.Tensor:
        """Device address of the value row of every slot (0 for slot -1); rows beyond ``hbm_rows`` live in mapped host memory."""
        rb = self.row_dim * 4
        hbm = self.values_hbm.data_ptr() + slots * rb
        if self.values_host is not None:
            host = self.values_host.data_ptr() + (slots - self.hbm_rows) * rb
            hbm = torch.where(slots < self.hbm_rows, hbm, host)
        return torch.where(slots >= 0, hbm, torch.zeros_like(hbm))

    def find_pointers(self, keys: torch.Tensor, update_score: bool = False, scores: Optional[torch.Tensor] = None):
        """-> (row addresses [n] int64, found mask): what the fused optimizer-on-pointer kernels of the reference consume
        (``csrc/hkv_variable.h:193-205``)."""
        slots, found = self.find(keys, update_score, scores)
        return self._pointers(slots), found

    def find_or_insert_pointers(self, keys: torch.Tensor, scores: Optional[torch.Tensor] = None):
        slots, status, _ = self.find_or_insert(keys, scores)
        return self._pointers(slots), status

    def _pin(self, keys: torch.Tensor, pin: bool):
        keys = keys.contiguous()
        n = keys.numel()
        slots = torch.empty(n, dtype=torch.int64, device=self.device)
        flags = torch.empty(n, dtype=torch.uint8, device=self.device)
        rc = _lib.lib().rb_hkv_pin(self._d(), keys.data_ptr(), n, int(pin), slots.data_ptr(), flags.data_ptr(), self._sms(),
                                   _lib.status_tensor(self.device).data_ptr(), self._st())
        _lib.check(rc, "rb_hkv_pin")
        return slots, flags.bool()

    def lock(self, keys: torch.Tensor):
        """Pin resident keys: until ``unlock`` they are never chosen as eviction victims, so row pointers handed out for
        them stay valid.  -> (slots, found mask)."""
        return self._pin(keys, True)

    def unlock(self, keys: torch.Tensor):
        return self._pin(keys, False)

    def counters(self) -> Dict[str, int]:
        """Life-time counts of the probe kernel's outcomes (a cheap health signal: a growing ``rejected`` or
        ``lock_timeouts`` count means the table is too small or contended)."""
        c = self._counters.tolist()
        return {"inserted": c[0], "evicted_other": c[1], "rejected": c[2], "lock_timeouts": c[3]}

    def erase(self, keys: torch.Tensor) -> None:
        keys = keys.contiguous()
        _lib.check(_lib.lib().rb_hkv_erase(self._d(), keys.data_ptr(), keys.numel(), self._sms(),
                                           _lib.status_tensor(self.device).data_ptr(), self._st()), "rb_hkv_erase")

    # ------------------------------------------------------------------ rows by slot
    def gather(self, slots: torch.Tensor, col0: int = 0, cols: Optional[int] = None,
               out: Optional[torch.Tensor] = None, dtype: torch.dtype = torch.float32, missing_value: float = 0.0):
        cols = self.dim if cols is None else cols
        n = slots.numel()
        if out is None:
            out = torch.empty(n, cols, dtype=dtype, device=self.device)
        rc = _lib.lib().rb_hkv_gather(self._d(), slots.data_ptr(), n, col0, cols, out.data_ptr(),
                                      _lib.dtype_code(out.dtype), out.stride(0), float(missing_value), self._sms(),
                                      self._st())
        _lib.check(rc, "rb_hkv_gather")
        return out

    def scatter(self, slots: torch.Tensor, values: torch.Tensor, col0: int, cols: int, accumulate: bool = False) -> None:
        values = values.float().contiguous()
        rc = _lib.lib().rb_hkv_scatter(self._d(), slots.data_ptr(), slots.numel(), col0, cols, values.data_ptr(),
                                       values.stride(0), int(accumulate), self._sms(), self._st())
        _lib.check(rc, "rb_hkv_scatter")

    def update(self, slots: torch.Tensor, grads: torch.Tensor, lr: float, eps: float = 1e-8, beta1: float = 0.9,
               beta2: float = 0.999, weight_decay: float = 0.0, step: int = 1) -> None:
        """Fused optimizer on row pointers (one warp per row); ``grads[i]`` is the summed gradient of row
        ``slots[i]`` (slots must be distinct)."""
        assert grads.stride(1) == 1
        bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
        rc = _lib.lib().rb_hkv_update(self._d(), slots.data_ptr(), slots.numel(), grads.data_ptr(),
                                      _lib.dtype_code(grads.dtype), grads.stride(0), int(self.optimizer), lr, eps, beta1,
                                      beta2, weight_decay, bc1, bc2, self._sms(), self._st())
        _lib.check(rc, "rb_hkv_update")

    # ------------------------------------------------------------------ export / growth
    def export_batch(self, slot0: int = 0, count: Optional[int] = None, min_score: Optional[int] = None,
                     with_values: bool = True):
        """Live entries among slots ``[slot0, slot0+count)`` (``export_batch_if`` when ``min_score`` is set):
        -> (keys, scores, rows or None, slots), each of length = number of matches."""
        count = self.capacity - slot0 if count is None else min(count, self.capacity - slot0)
        cap = max(count, 1)
        dev = self.device
        ok = torch.empty(cap, dtype=torch.int64, device=dev)
        osc = torch.empty(cap, dtype=torch.int64, device=dev)
        osl = torch.empty(cap, dtype=torch.int64, device=dev)
        ov = torch.empty(cap, self.row_dim, dtype=torch.float32, device=dev) if with_values else None
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        rc = _lib.lib().rb_hkv_export(self._d(), slot0, count, 0 if min_score is None else int(min_score), ok.data_ptr(),
                                      osc.data_ptr(), _lib.ptr(ov), osl.data_ptr(), counter.data_ptr(), cap, self._sms(),
                                      self._st())
        _lib.check(rc, "rb_hkv_export")
        m = int(counter.item())
        return ok[:m], osc[:m], (ov[:m] if ov is not None else None), osl[:m]

    def reserve(self, new_capacity: int) -> None:
        """Rehash into a table of at least ``new_capacity`` slots (bounded by ``max_capacity``)."""
        new_cap = min(self.max_capacity, max(self.capacity, _pow2_ceil(int(new_capacity))))
        if new_cap <= self.capacity:
            return
        old = dict(keys=self.keys, scores=self.scores, digests=self.digests, locks=self.locks, vh=self.values_hbm,
                   vhost=self.values_host, size=self._size, desc=self._desc)
        self._alloc(new_cap)
        self.clear()
        rc = _lib.lib().rb_hkv_rehash(old["desc"].ctypes.data, self._d(), self._sms(),
                                      _lib.status_tensor(self.device).data_ptr(), self._st())
        _lib.check(rc, "rb_hkv_rehash")
        torch.cuda.current_stream(self.device).synchronize()   # the old arrays may be freed now

    def maybe_grow(self, incoming: int) -> None:
        """Double the capacity while (size + incoming) would exceed ``max_load_factor`` (host-synchronising;
        called from ``find_or_insert`` only while the table can still grow)."""
        if self.capacity >= self.max_capacity:
            return
        need = self.size() + incoming
        cap = self.capacity
        while cap < self.max_capacity and need > self.max_load_factor * cap:
            cap *= 2
        if cap > self.capacity:
            self.reserve(cap)

    def device_timestamp(self) -> int:
        t = torch.zeros(1, dtype=torch.int64, device=self.device)
        _lib.check(_lib.lib().rb_device_timestamp(t.data_ptr(), self._st()), "rb_device_timestamp")
        return int(t.item())


class HostDynamicTable(_VariableInterface):
    """Dictionary-backed table with the ``HKVTable`` interface (CPU execution and test oracle)."""

    def __init__(self, dim: int, capacity: int, optimizer: OptimizerType = OptimizerType.SGD,
                 evict_strategy: EvictStrategy = EvictStrategy.LRU, init: Optional[InitializerArgs] = None, **_kw) -> None:
        self.dim, self.capacity = dim, capacity
        self.optimizer = OptimizerType(optimizer)
        self.state_dim = opt_state_dim(self.optimizer, dim)
        self.row_dim = dim + self.state_dim
        self.evict_strategy = EvictStrategy(evict_strategy)
        self.init = init or InitializerArgs()
        self.rows: Dict[int, np.ndarray] = {}
        self.score: Dict[int, int] = {}
        self._clock = 0
        self.device = torch.device("cpu")

    def size(self) -> int:
        return len(self.rows)

    def clear(self) -> None:
        self.rows.clear()
        self.score.clear()

    def _new_row(self, key: int) -> np.ndarray:
        i = self.init
        r = np.full(self.row_dim, i.state_init, dtype=np.float32)
        rng = np.random.default_rng((int(i.seed) * 1000003 + (key & 0xFFFFFFFFFFFF)) & 0x7FFFFFFFFFFFFFFF)
        if i.mode == InitMode.UNIFORM:
            r[: self.dim] = rng.uniform(i.lower, i.upper, self.dim)
        elif i.mode == InitMode.NORMAL:
            r[: self.dim] = rng.normal(i.mean, i.std_dev, self.dim)
        elif i.mode == InitMode.TRUNCATED_NORMAL:
            r[: self.dim] = i.mean + i.std_dev * np.clip(rng.normal(0, 1, self.dim), -2, 2)
        elif i.mode == InitMode.CONSTANT:
            r[: self.dim] = i.value
        else:
            r[: self.dim] = float(key % 100000)
        return r

    def _touch(self, key: int, given: Optional[int], new: bool) -> None:
        self._clock += 1
        if self.evict_strategy == EvictStrategy.LRU:
            self.score[key] = self._clock
        elif self.evict_strategy == EvictStrategy.LFU:
            self.score[key] = (0 if new else self.score.get(key, 0)) + (1 if given is None else given)
        else:
            self.score[key] = given if given is not None else (1 if new else self.score.get(key, 1))

    def find_or_insert(self, keys: torch.Tensor, scores: Optional[torch.Tensor] = None, evict_cap: int = 0,
                       keep_epoch: bool = False):
        ks = keys.tolist()
        sc = scores.tolist() if scores is not None else [None] * len(ks)
        status = []
        evk, evs, evr = [], [], []
        stamped = set(getattr(self, "_stamped", ())) if keep_epoch else set()
        for k, s in zip(ks, sc):
            if k == EMPTY_KEY:
                status.append(ST_MISSING)
                continue
            if k in self.rows:
                status.append(ST_FOUND)
                self._touch(k, s, False)
                stamped.add(k)
                continue
            if len(self.rows) >= self.capacity:
                # keys handed out by this call are never evicted by it (their slots are in use by the caller)
                free = [q for q in self.score if q not in stamped]
                if not free:
                    status.append(ST_REJECTED)
                    continue
                victim = min(free, key=self.score.get)
                evk.append(victim); evs.append(self.score.pop(victim)); evr.append(self.rows.pop(victim))
                status.append(ST_EVICTED_OTHER)
            else:
                status.append(ST_INSERTED)
            self.rows[k] = self._new_row(k)
            self._touch(k, s, True)
            stamped.add(k)
        ev = None
        if evict_cap > 0:
            ev = (torch.tensor(evk, dtype=torch.int64), torch.tensor(evs, dtype=torch.int64),
                  torch.from_numpy(np.stack(evr)) if evr else torch.zeros(0, self.row_dim),
                  torch.tensor([len(evk)], dtype=torch.int32))
        st = torch.tensor(status, dtype=torch.uint8)
        return torch.where((st == ST_MISSING) | (st == ST_REJECTED), torch.full_like(keys, -1), keys), st, ev

    def find(self, keys: torch.Tensor, update_score: bool = False, scores=None, stamp: bool = False):
        ks = keys.tolist()
        found = torch.tensor([k in self.rows for k in ks], dtype=torch.bool)
        if update_score:
            sc = scores.tolist() if scores is not None else [None] * len(ks)
            for k, s in zip(ks, sc):
                if k in self.rows:
                    self._touch(k, s, False)
        if stamp:
            self._stamped = {k for k in ks if k in self.rows}
        slots = torch.where(found, keys, torch.full_like(keys, -1))
        return slots, found

    def gather(self, slots: torch.Tensor, col0: int = 0, cols: Optional[int] = None, out=None,
               dtype: torch.dtype = torch.float32, missing_value: float = 0.0):
        cols = self.dim if cols is None else cols
        res = torch.full((slots.numel(), cols), missing_value, dtype=torch.float32)
        for i, k in enumerate(slots.tolist()):
            if k in self.rows:
                res[i] = torch.from_numpy(self.rows[k][col0:col0 + cols])
        res = res.to(dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def scatter(self, slots, values, col0, cols, accumulate=False) -> None:
        v = values.float().numpy()
        for i, k in enumerate(slots.tolist()):
            if k in self.rows:
                if accumulate:
                    self.rows[k][col0:col0 + cols] += v[i]
                else:
                    self.rows[k][col0:col0 + cols] = v[i]

    def insert_and_evict(self, keys, values, scores=None):
        slots, status, ev = self.find_or_insert(keys, scores, evict_cap=max(keys.numel(), 1))
        self.scatter(slots, values, 0, values.shape[1])
        return slots, status, ev

    def erase(self, keys) -> None:
        for k in keys.tolist():
            self.rows.pop(k, None)
            self.score.pop(k, None)

    def update(self, slots, grads, lr, eps=1e-8, beta1=0.9, beta2=0.999, weight_decay=0.0, step=1) -> None:
        D = self.dim
        g_all = grads.float().numpy()
        for i, k in enumerate(slots.tolist()):
            if k not in self.rows:
                continue
            row, g = self.rows[k], g_all[i]
            if self.optimizer == OptimizerType.SGD:
                row[:D] -= lr * (g + weight_decay * row[:D])
            elif self.optimizer == OptimizerType.ROWWISE_ADAGRAD:
                row[D] += float((g * g).mean())
                row[:D] -= lr * g / (np.sqrt(row[D]) + eps)
            elif self.optimizer == OptimizerType.ADAGRAD:
                row[D:2 * D] += g * g
                row[:D] -= lr * g / (np.sqrt(row[D:2 * D]) + eps)
            else:
                # decoupled decay (dynamic_emb csrc/dynamic_emb_op.cpp:1602 of the reference)
                row[D:2 * D] = beta1 * row[D:2 * D] + (1 - beta1) * g
                row[2 * D:3 * D] = beta2 * row[2 * D:3 * D] + (1 - beta2) * g * g
                bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
                row[:D] = row[:D] * (1 - lr * weight_decay) - (lr / bc1) * row[D:2 * D] / (np.sqrt(row[2 * D:3 * D] / bc2) + eps)

    def export_batch(self, slot0: int = 0, count=None, min_score=None, with_values: bool = True):
        ks = [k for k in self.rows if min_score is None or self.score[k] >= min_score]
        keys = torch.tensor(ks, dtype=torch.int64)
        sc = torch.tensor([self.score[k] for k in ks], dtype=torch.int64)
        rows = torch.from_numpy(np.stack([self.rows[k] for k in ks])) if (ks and with_values) else (
            torch.zeros(0, self.row_dim) if with_values else None)
        return keys, sc, rows, keys.clone()

    def reserve(self, new_capacity: int) -> None:
        self.capacity = max(self.capacity, new_capacity)

    def maybe_grow(self, incoming: int) -> None:
        return None

    def load_factor(self) -> float:
        return len(self.rows) / max(self.capacity, 1)

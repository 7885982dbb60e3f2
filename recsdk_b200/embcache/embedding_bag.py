"""Multi-tier embedding collections: the full table lives in host DRAM (native ``EmbcacheManager``), a cache of
hot rows (weights and optimizer state) lives in device memory, and every step swaps the rows the batch needs in
and the least recently needed ones out.

``EmbCacheEmbeddingBagCollection`` / ``EmbCacheEmbeddingCollection`` are the unsharded declarations (they size the
device cache); ``EmbCacheShardedEmbeddingBagCollection`` does the work: row-wise (``id % world``) input
distribution, per-table swap planning on the native thread pool, gather of victims / scatter of incoming rows on
the device, pooled lookup over the cache with the sparse update applied in backward, and pooled output
distribution.  Keys that the admission filter rejects read slot 0, which holds ``not_admitted_default_value`` and
is never trained.  Reference: ``torchrec_embcache/distributed/embedding_bag.py:171-337`` (cache sizing
``:308-337``), ``:340-850``; ``embedding.py:587-625`` (not-admitted ids); swap stages
``train_pipeline.py:424-537``.
"""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch
from torch import nn
from torch.autograd.profiler import record_function

from ..host import host
from ..modules.embedding_configs import PoolingType
from ..ops import embedding_ops as E
from ..parallel.collective_embeddingbag import CollectiveShardedEmbeddingBagCollection
from ..parallel.comm import ShardingEnv
from ..parallel.embeddingbag import ParameterSharding
from ..sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor
from .configs import POLICY_SHOW_CLICK, EmbCacheEmbeddingBagConfig, InitializerType

DEFAULT_CACHE_BYTES = 16 << 30
MAX_CACHE_BYTES = 64 << 30

_OPTIM_NUM = {E.OPT_SGD: 0, E.OPT_ADAGRAD: 1, E.OPT_ADAM: 2}


def _cache_budget_bytes() -> int:
    try:
        v = int(os.environ.get("EMBCACHE_SIZE_ON_DEVICE_MEM", DEFAULT_CACHE_BYTES))
    except ValueError:
        v = DEFAULT_CACHE_BYTES
    return max(1, min(v, MAX_CACHE_BYTES))


def calculate_caches(tables: Sequence, world_size: int, batch_size: int, multi_hot_sizes: Sequence[int], optim_num: int
                     ) -> List[int]:
    """Device-cache rows per table.  The floor is what two in-flight batches can touch
    (``hot * 2 * batch * world`` rows); the device budget (``EMBCACHE_SIZE_ON_DEVICE_MEM``, default 16 GiB, at most
    64 GiB) scales every table by the same factor above that floor, never beyond the table itself."""
    floor_rows = [max(1, int(h)) * 2 * batch_size * world_size for h in multi_hot_sizes]
    min_bytes = sum(r * t.embedding_dim * 4 * (optim_num + 1) for r, t in zip(floor_rows, tables))
    scale = max(1.0, _cache_budget_bytes() / max(min_bytes, 1))
    return [int(min(t.num_embeddings + 1, max(r, int(r * scale)))) for r, t in zip(floor_rows, tables)]


class EmbCacheEmbeddingBagCollection(nn.Module):
    """Unsharded declaration: validates the tables and computes the device-cache sizes.  ``forward`` exists for
    single-process use (it builds a world-size-1 sharded module on first call)."""

    def __init__(self, tables: List[EmbCacheEmbeddingBagConfig], world_size: int, batch_size: int, multi_hot_sizes: List[int],
                 is_weighted: bool = False, need_accumulate_offset: bool = True, device=None,
                 embedding_optimizer_cls=torch.optim.Adagrad) -> None:
        super().__init__()
        if is_weighted:
            raise ValueError("weighted embcache tables are not supported")
        if len(multi_hot_sizes) != len(tables):
            raise ValueError("multi_hot_sizes needs one entry per table")
        names = [t.name for t in tables]
        if len(set(names)) != len(names):
            raise ValueError("duplicate table names")
        for t in tables:
            if t.embedding_dim % 8 or not (8 <= t.embedding_dim <= 4096):
                raise ValueError("embedding_dim must be a multiple of 8 in [8, 4096]")
        self.tables, self.world_size, self.batch_size = list(tables), world_size, batch_size
        self.multi_hot_sizes = list(multi_hot_sizes)
        self.need_accumulate_offset = need_accumulate_offset
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.embedding_optimizer_cls = embedding_optimizer_cls
        self._sharded: Optional[EmbCacheShardedEmbeddingBagCollection] = None

    def embedding_bag_configs(self):
        return self.tables

    def is_weighted(self) -> bool:
        return False

    def optimizer_spec(self, **kw) -> E.OptimizerSpec:
        kind = {torch.optim.SGD: E.OPT_SGD, torch.optim.Adagrad: E.OPT_ADAGRAD, torch.optim.Adam: E.OPT_ADAM}.get(
            self.embedding_optimizer_cls)
        if kind is None:
            raise ValueError("embcache tables train with SGD, Adagrad or Adam")
        return E.OptimizerSpec(kind=kind, **kw)

    def cache_rows(self, optim_num: int) -> List[int]:
        return calculate_caches(self.tables, self.world_size, self.batch_size, self.multi_hot_sizes, optim_num)

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        if self._sharded is None:
            self._sharded = EmbCacheShardedEmbeddingBagCollection(self, ShardingEnv(1, 0, None), self.device, self.optimizer_spec())
        return self._sharded(features)


class EmbCacheShardedEmbeddingBagCollection(CollectiveShardedEmbeddingBagCollection):
    def __init__(self, module: EmbCacheEmbeddingBagCollection, env: ShardingEnv, device, optimizer_spec: Optional[E.OptimizerSpec] = None,
                 cache_rows: Optional[List[int]] = None, threads: int = 4) -> None:
        spec = optimizer_spec or module.optimizer_spec()
        if spec.kind not in _OPTIM_NUM:
            raise ValueError("embcache tables train with SGD, Adagrad or Adam")
        self.optim_num = _OPTIM_NUM[spec.kind]
        rows = cache_rows or module.cache_rows(self.optim_num)
        # the parent allocates one weight tensor per table with `local_rows` rows: make that the cache size
        import copy

        cache_tables = []
        for t, r in zip(module.tables, rows):
            c = copy.copy(t)
            c.num_embeddings = int(r) * env.world_size                 # row-wise split -> r rows on this rank
            cache_tables.append(c)
        plan = {t.name: ParameterSharding("row_wise", row_partition="mod") for t in module.tables}
        super().__init__(cache_tables, plan, env, torch.device(device), spec, hashed=True, init_weights=False)
        self.mappers = None
        self.full_tables = list(module.tables)
        self.cache_rows_per_table = [int(r) for r in rows]
        cfgs = []
        for t, r in zip(module.tables, rows):
            c = host().EmbConfig()
            c.table_name, c.emb_dim, c.optim_num, c.cache_size = t.name, t.embedding_dim, self.optim_num, int(r)
            ic = host().InitializerConfig()
            it = getattr(t, "initializer_type", InitializerType.LINEAR)
            ic.type = {InitializerType.LINEAR: host().InitializerType.LINEAR,
                       InitializerType.TRUNCATED_NORMAL: host().InitializerType.TRUNCATED_NORMAL,
                       InitializerType.UNIFORM: host().InitializerType.UNIFORM}[it]
            ic.min, ic.max = t.get_weight_init_min(), t.get_weight_init_max()
            ic.mean, ic.stddev = getattr(t, "weight_init_mean", 0.0), getattr(t, "weight_init_stddev", 0.05)
            ic.seed = 1234 + env.rank
            c.init = ic
            ae = getattr(t, "admit_and_evict_config", None)
            if ae is not None:
                a = host().AdmitEvictConfig()
                a.admit_threshold, a.evict_threshold = ae.admit_threshold, ae.evict_threshold
                a.policy = 1 if ae.policy_type == POLICY_SHOW_CLICK else 0
                p = ae.show_click_params
                a.alpha, a.beta, a.sc_admit_threshold = p.alpha, p.beta, p.admit_threshold
                a.evict_percentage, a.score_decay = p.evict_percentage, p.score_decay
                c.admit_evict = a
            c.is_incremental = bool(getattr(t, "is_incremental", False))
            cfgs.append(c)
        self.manager = host().EmbcacheManager(cfgs, threads)
        self.admit = [bool(getattr(t, "admit_and_evict_config", None) and t.admit_and_evict_config.is_admit_enabled())
                      for t in module.tables]
        self.evict = [bool(getattr(t, "admit_and_evict_config", None) and t.admit_and_evict_config.is_evict_enabled())
                      for t in module.tables]
        self.default_value = [getattr(getattr(t, "admit_and_evict_config", None), "not_admitted_default_value", 0.0)
                              for t in module.tables]
        self.swap_step = 0
        self.stats = {"swap_in": 0, "swap_out": 0}
        # asynchronous swap state (CUDA): memcpy stream, pinned staging ring, host worker for lookups / updates
        from concurrent.futures import ThreadPoolExecutor

        self._memcpy_stream = torch.cuda.Stream(torch.device(device)) if torch.device(device).type == "cuda" else None
        self._host_pool = ThreadPoolExecutor(max_workers=2)
        self._pinned: Dict[tuple, torch.Tensor] = {}
        self._out_busy: Dict[tuple, object] = {}
        self._in_busy: Dict[tuple, object] = {}
        self._upd_fut: List[Optional[object]] = [None] * len(module.tables)
        self._step_done = self._step_done_prev = None
        self._swap_ready = None
        self.record_timing = False               # tests: keep (batch, begin, end) CUDA events of every swap
        self.swap_events: List[tuple] = []
        with torch.no_grad():
            for ti, t in enumerate(self.tables):
                self.embedding_bags[t.name].weight.zero_()

    # -- state rows <-> host rows ------------------------------------------------------------------------
    def _gather_cache_rows(self, ti: int, offs: torch.Tensor) -> torch.Tensor:
        w = self.embedding_bags[self.tables[ti].name].weight.data
        parts = [E.gather_rows(w, offs)]
        st = self.state[ti]
        for k in ("state1", "state2")[: self.optim_num]:
            parts.append(E.gather_rows(st[k], offs))
        return torch.cat(parts, dim=1) if len(parts) > 1 else parts[0]

    def _scatter_cache_rows(self, ti: int, offs: torch.Tensor, rows: torch.Tensor) -> None:
        D = self.tables[ti].embedding_dim
        w = self.embedding_bags[self.tables[ti].name].weight.data
        E.scatter_rows(rows[:, :D].contiguous(), offs, w)
        st = self.state[ti]
        for j, k in enumerate(("state1", "state2")[: self.optim_num]):
            E.scatter_rows(rows[:, (j + 1) * D:(j + 2) * D].contiguous(), offs, st[k])

    # -- the swap ----------------------------------------------------------------------------------------
    def compute_swap_info_async(self, ti: int, keys: np.ndarray):
        return self.manager.compute_swap_info_async(ti, keys, self.swap_step)

    def apply_swap(self, ti: int, info: Dict[str, np.ndarray]) -> None:
        """Victims device -> host, incoming rows host -> device."""
        dev = self.device
        so_k, so_o = info["swapout_keys"], info["swapout_offs"]
        if so_k.size:
            rows = self._gather_cache_rows(ti, torch.from_numpy(so_o).to(dev))
            self.manager.embedding_update(ti, so_k, rows.float().cpu().numpy())
            self.stats["swap_out"] += int(so_k.size)
        si_k, si_o = info["swapin_keys"], info["swapin_offs"]
        if si_k.size:
            rows = torch.from_numpy(self.manager.embedding_lookup(ti, si_k))
            if dev.type == "cuda":
                rows = rows.pin_memory().to(dev, non_blocking=True)
            self._scatter_cache_rows(ti, torch.from_numpy(si_o).to(dev), rows)
            self.stats["swap_in"] += int(si_k.size)
        if self.admit[ti]:
            w = self.embedding_bags[self.tables[ti].name].weight.data
            w[0].fill_(self.default_value[ti])

    # -- asynchronous swap (CUDA): pinned staging, copies and row kernels on a memcpy stream ---------------------
    RING = 3                                     # staging sets in rotation: a set is reused three batches later

    def _async_ready(self) -> bool:
        return self.device.type == "cuda" and (self.world == 1 or self.input_pg is not None)

    def _staging(self, kind: str, ti: int, slot: int, rows: int) -> torch.Tensor:
        """Pinned host buffer ``[>= rows, row_floats]`` of table ``ti`` (grown geometrically, never per step)."""
        key = (kind, ti, slot)
        buf = self._pinned.get(key)
        if buf is None or buf.shape[0] < rows:
            rf = self.tables[ti].embedding_dim * (1 + self.optim_num)
            cap = max(1024, int(rows * 1.5))
            buf = torch.empty(cap, rf, dtype=torch.float32).pin_memory()
            self._pinned[key] = buf
        return buf

    def record_batch_keys_async(self, lengths: torch.Tensor, ids_np: np.ndarray):
        """Start the per-table batch planning on the native pool (distinct keys + counts for the admission filter,
        last-seen timestamps, swap plan).  -> (futures, positions of each table's ids in ``ids_np``)."""
        self.swap_step += 1
        W, F, B = lengths.shape
        seg = lengths.sum(dim=2).reshape(-1).cpu().numpy()
        seg_off = np.concatenate([[0], np.cumsum(seg)])
        tab_pos: List[List[np.ndarray]] = [[] for _ in self.tables]
        for s_ in range(W):
            for f in range(F):
                tab_pos[self.feature_table[f]].append(np.arange(seg_off[s_ * F + f], seg_off[s_ * F + f + 1]))
        pos = [np.concatenate(p) if p else np.zeros(0, dtype=np.int64) for p in tab_pos]
        now = int(time.time())
        with record_function("## _compute_swap_info_async ##"):
            futs = [self.manager.plan_batch_async(ti, ids_np[p], self.swap_step, self.admit[ti], self.evict[ti], now)
                    for ti, p in enumerate(pos)]
        return futs, pos

    def host_embedding_update_async(self, ti: int, keys: np.ndarray, staged: torch.Tensor, copied: "torch.cuda.Event"):
        """Host InsertOrAssign of swapped-out rows once their device-to-host copy has landed in the pinned buffer."""
        prev = self._upd_fut[ti]

        def run():
            if prev is not None:
                prev.result()
            copied.synchronize()
            with record_function("## _host_embedding_update ##"):
                self.manager.embedding_update_from(ti, keys, staged.data_ptr())

        fut = self._host_pool.submit(run)
        self._upd_fut[ti] = fut
        return fut

    def host_embedding_lookup_async(self, ti: int, keys: np.ndarray, staged: torch.Tensor):
        """Host FindOrInsert of the rows a batch swaps in, written into the pinned buffer; ordered after every earlier
        update of the table (a key evicted by the previous batch may come straight back)."""
        prev = self._upd_fut[ti]

        def run():
            if prev is not None:
                prev.result()
            with record_function("## host_embedding_lookup_async ##"):
                self.manager.embedding_lookup_into(ti, keys, staged.data_ptr(), staged.shape[0])

        return self._host_pool.submit(run)

    def apply_swap_async(self, ti: int, info: Dict[str, np.ndarray], slot: int) -> None:
        """Enqueue the swap traffic of one table on the memcpy stream (the caller has made it current): victims
        gather -> pinned (D2H) -> host update on the pool; host lookup -> pinned -> H2D -> scatter."""
        dev = self.device
        so_k, so_o = info["swapout_keys"], info["swapout_offs"]
        if so_k.size:
            rows = self._gather_cache_rows(ti, torch.from_numpy(so_o).to(dev, non_blocking=True))
            st = self._staging("out", ti, slot, so_k.size)
            busy = self._out_busy.get((ti, slot))
            if busy is not None:
                busy.result()                                   # the update that last read this staging set is done
            st[: so_k.size].copy_(rows, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._out_busy[(ti, slot)] = self.host_embedding_update_async(ti, so_k, st, ev)
            self.stats["swap_out"] += int(so_k.size)
        si_k, si_o = info["swapin_keys"], info["swapin_offs"]
        if si_k.size:
            st = self._staging("in", ti, slot, si_k.size)
            busy = self._in_busy.get((ti, slot))
            if busy is not None:
                busy.synchronize()                              # the H2D copy that last read this staging set is done
            self.host_embedding_lookup_async(ti, si_k, st).result()
            rows = st[: si_k.size].to(dev, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._in_busy[(ti, slot)] = ev
            self._scatter_cache_rows(ti, torch.from_numpy(si_o).to(dev, non_blocking=True), rows)
            self.stats["swap_in"] += int(si_k.size)
        if self.admit[ti]:
            w = self.embedding_bags[self.tables[ti].name].weight.data
            w[0].fill_(self.default_value[ti])

    def post_input_dist_async(self, lengths: torch.Tensor, ids_host: torch.Tensor):
        """Ids on the host -> device-cache slots, with the swap traffic on the memcpy stream.  The stream first waits for
        the step that last trained the victims (``mark_step_done``), so it can run beside the current step's compute."""
        ids_np = ids_host.numpy().astype(np.int64, copy=False)
        lengths = lengths.cpu()
        futs, pos = self.record_batch_keys_async(lengths, ids_np)
        slot = self.swap_step % self.RING
        out = np.empty_like(ids_np)
        with torch.cuda.stream(self._memcpy_stream):
            # Victims were last used by batch (this - 2) or earlier: wait for THAT step's backward, not for the step that
            # is running now, whose rows the slot allocator protects.
            if self._step_done_prev is not None:
                self._memcpy_stream.wait_event(self._step_done_prev)
            if self.record_timing:
                t_begin = torch.cuda.Event(enable_timing=True)
                t_begin.record()
            for ti, p in enumerate(pos):
                with record_function("## wait_and_get_swap_info ##"):
                    info = futs[ti].get()
                with record_function("## swap_out / swapin_embs_optims_to_gpu ##"):
                    self.apply_swap_async(ti, info, slot)
                out[p] = info["batch_offs"]
            slots = torch.from_numpy(out).pin_memory().to(self.device, non_blocking=True)
            lengths_dev = lengths.pin_memory().to(self.device, non_blocking=True)
            ready = torch.cuda.Event(enable_timing=self.record_timing)
            ready.record()
            if self.record_timing:
                self.swap_events.append((self.swap_step, t_begin, ready))     # device-side span of this batch's swap traffic
        self._swap_ready = ready
        return slots, lengths_dev

    def mark_step_done(self) -> None:
        """Called by the pipeline after a step's backward is enqueued.  The swap that is planned next (for the batch after
        the one now running) waits for the step BEFORE this one: that is the last step that can have trained its victims."""
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._step_done_prev, self._step_done = self._step_done, ev

    def wait_swap(self) -> None:
        """The compute stream waits for the scatter of the batch it is about to look up."""
        if self._swap_ready is not None:
            with record_function("## wait_and_swapin ##"):
                torch.cuda.current_stream(self.device).wait_event(self._swap_ready)
            self._swap_ready = None

    def drain_host_updates(self) -> None:
        """Block until every pending host update has been applied (before a save, an eviction or a flush)."""
        for f in self._upd_fut:
            if f is not None:
                f.result()

    def prefetch_async(self, features_dev: KeyedJaggedTensor, features_host: KeyedJaggedTensor) -> None:
        """Pipelined ``prefetch``: input distribution on the host copy of the batch (native bucketize; gloo exchange with
        more than one rank), swap planning on the native pool, swap traffic on the memcpy stream - nothing here makes the
        host wait for the compute stream."""
        F, B = len(self.feature_names), features_host.stride()
        new_lengths, new_ids, _perm = self._bucketize(features_host)
        if self.world > 1:
            import torch.distributed as dist

            recv_lengths = torch.empty_like(new_lengths)
            dist.all_to_all_single(recv_lengths, new_lengths.contiguous(), group=self.input_pg)
            in_splits = new_lengths.sum(dim=1).tolist()
            out_splits = recv_lengths.view(self.world, -1).sum(dim=1).tolist()
            recv_ids = new_ids.new_empty(int(sum(out_splits)))
            dist.all_to_all_single(recv_ids, new_ids, out_splits, in_splits, group=self.input_pg)
            new_lengths, new_ids = recv_lengths, recv_ids
        lengths = new_lengths.view(self.world, F, B)
        slots, lengths_dev = self.post_input_dist_async(lengths, new_ids)
        orig = features_dev.lengths().view(F, B)
        self._prepared[id(features_dev)] = (lengths_dev, slots, B, orig, self._swap_ready)
        self._swap_ready = None

    def post_input_dist(self, lengths: torch.Tensor, ids: torch.Tensor):
        """Raw ids (this rank's share of the global batch) -> device-cache slots."""
        self.swap_step += 1
        W, F, B = lengths.shape
        seg = lengths.sum(dim=2).reshape(-1).cpu().numpy()
        seg_off = np.concatenate([[0], np.cumsum(seg)])
        ids_np = ids.cpu().numpy().astype(np.int64)
        tab_pos: List[List[np.ndarray]] = [[] for _ in self.tables]
        for s in range(W):
            for f in range(F):
                tab_pos[self.feature_table[f]].append(np.arange(seg_off[s * F + f], seg_off[s * F + f + 1]))
        pos = [np.concatenate(p) if p else np.zeros(0, dtype=np.int64) for p in tab_pos]
        now = int(time.time())
        futs = []
        for ti, p in enumerate(pos):
            keys = ids_np[p]
            if self.admit[ti] or self.evict[ti]:
                uk, cnt = np.unique(keys, return_counts=True)
                if self.admit[ti]:
                    self.manager.statistics_key_count(ti, uk, cnt.astype(np.int64), None)
                if self.evict[ti]:
                    self.manager.record_timestamp(ti, uk, np.full(uk.shape, now, dtype=np.int64))
            futs.append(self.compute_swap_info_async(ti, keys))
        out = np.empty_like(ids_np)
        for ti, p in enumerate(pos):
            info = futs[ti].get()
            self.apply_swap(ti, info)
            out[p] = info["batch_offs"]
        return torch.from_numpy(out).to(ids.device)

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        ctx = self._prepared.get(id(features))
        if ctx is not None and self.device.type == "cuda":
            cur = torch.cuda.current_stream(self.device)
            for t in ctx[:2]:                      # produced on a side stream, consumed here
                if isinstance(t, torch.Tensor) and t.is_cuda:
                    t.record_stream(cur)
        return super().forward(features)

    def _apply_update(self, ti: int, rows: torch.Tensor, grads: torch.Tensor) -> None:
        if self.admit[ti]:                                   # slot 0 = "not admitted": never trained
            keep = rows != 0
            rows, grads = rows[keep], grads[keep]
        super()._apply_update(ti, rows, grads)

    # -- names of the reference's sharded module ----------------------------------------------------------
    @property
    def embcache_mgr(self):
        """The native host-side manager (reference ``distributed/embedding_bag.py:593-595``)."""
        return self.manager

    @property
    def config_list(self):
        """The unsharded table configs (reference ``distributed/embedding_bag.py:597-599``)."""
        return self.full_tables

    def get_batched_embedding_kernels(self) -> List[List["CacheKernelView"]]:
        """One group with one view over this rank's device cache: ``[0][0].weights_dev`` is the flat cache weight and
        ``get_momentum()`` the optimizer-state tensors, which is what a saver reads before it writes rows back to the
        host (reference ``distributed/embedding_bag.py:790-799`` returns its codegen modules for the same purpose)."""
        return [[CacheKernelView(self)]]

    def record_host_emb_update_times(self) -> None:
        """Kept for pipelines written against the reference, which calls it once per host update: there, rows of evicted
        features leave the host table only after a fixed number of further updates, so that swaps already planned do not
        meet a missing row (``embcache_manager.cpp:1245-1252``).  Here ``host_embedding_evict`` first drains the pending
        host updates and then removes the rows at once, so there is nothing to count."""

    # -- eviction / checkpoint helpers -------------------------------------------------------------------
    def host_embedding_evict(self) -> Dict[str, int]:
        self.drain_host_updates()
        out = {}
        with record_function("## feature_evict ##"):
            for ti, t in enumerate(self.full_tables):
                if self.evict[ti]:
                    out[t.name] = int(self.manager.evict_features(ti).size)
        return out

    @torch.no_grad()
    def embedding_to_host(self) -> None:
        """Write every device-resident row back to the host table (before a save)."""
        self.drain_host_updates()
        if self._memcpy_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._memcpy_stream)
        for ti in range(len(self.tables)):
            keys, offs = self.manager.resident(ti)
            if keys.size:
                rows = self._gather_cache_rows(ti, torch.from_numpy(offs).to(self.device))
                self.manager.embedding_update(ti, keys, rows.float().cpu().numpy())

    def invalidate_device_cache(self) -> None:
        for ti in range(len(self.tables)):
            self.manager.invalidate_cache(ti)

    def host_rows(self, name: str, keys: Sequence[int]) -> torch.Tensor:
        """Current value ``[len(keys), dim * (1 + optim_num)]`` of rows wherever they live (device cache first)."""
        ti = [t.name for t in self.full_tables].index(name)
        self.embedding_to_host()
        return torch.from_numpy(self.manager.embedding_lookup(ti, np.asarray(keys, dtype=np.int64)))


class CacheKernelView:
    """Read-only view of a sharded cache module in the shape of a batched embedding kernel: the per-table device
    weights, flat (``weights_dev``) or split (``split_embedding_weights``), and the optimizer state (``get_momentum``)."""

    def __init__(self, module: "EmbCacheShardedEmbeddingBagCollection") -> None:
        self._m = module

    def split_embedding_weights(self) -> List[torch.Tensor]:
        return [self._m.embedding_bags[t.name].weight.data for t in self._m.tables]

    @property
    def weights_dev(self) -> torch.Tensor:
        ws = self.split_embedding_weights()
        return torch.cat([w.reshape(-1) for w in ws]) if ws else torch.empty(0)

    def get_momentum(self) -> List[torch.Tensor]:
        """``optim_num`` flat tensors, each the concatenation over tables of that state slot."""
        out = []
        for k in ("state1", "state2")[: self._m.optim_num]:
            out.append(torch.cat([self._m.state[ti][k].reshape(-1) for ti in range(len(self._m.tables))]))
        return out


class EmbCacheHashTable(nn.Module):
    """One table whose ids are arbitrary 64-bit keys: an ``IdsMapper`` hands out rows in order of first sight and a plain
    ``nn.EmbeddingBag`` holds them (reference ``distributed/embedding_bag.py:142-168``; the unsharded, single-process
    form of a cached table, used to check the sharded one)."""

    def __init__(self, config, device=None) -> None:
        super().__init__()
        from ..modules.ids_process import IdsMapper

        self.config = config
        self.ids2slot_dict = IdsMapper(config.num_embeddings, only_device_memory=False)
        mode = getattr(getattr(config, "pooling", None), "name", "SUM").lower()
        self.vector_table = nn.EmbeddingBag(config.num_embeddings, config.embedding_dim, mode=mode, device=device,
                                            include_last_offset=True)
        self.index = 0
        self.register_parameter("weight", self.vector_table.weight)

    def forward(self, input_feat: torch.Tensor, offsets: Optional[torch.Tensor] = None, per_sample_weights=None) -> torch.Tensor:
        idx, _, _ = self.ids2slot_dict(input_feat.cpu())
        return self.vector_table(idx.to(input_feat.device), offsets, per_sample_weights)


class EmbCacheEmbeddingBagCollectionSharder:
    """``shard(module, env, device)`` -> sharded module; row-wise is the only sharding
    (reference ``sharding/embedding_sharder.py:70-132``)."""

    def __init__(self, cpu_device=None, cpu_env: Optional[ShardingEnv] = None, npu_device=None, npu_env: Optional[ShardingEnv] = None,
                 fused_params: Optional[dict] = None, qcomm_codecs_registry=None) -> None:
        self.cpu_device, self.cpu_env, self.device, self.env = cpu_device, cpu_env, npu_device, npu_env
        self.fused_params = dict(fused_params or {})

    def sharding_types(self, compute_device_type: str = "cuda") -> List[str]:
        return ["row_wise"]

    @property
    def module_type(self):
        return EmbCacheEmbeddingBagCollection

    def shard(self, module: EmbCacheEmbeddingBagCollection, params=None, env: Optional[ShardingEnv] = None, device=None):
        spec = module.optimizer_spec(**{k: v for k, v in self.fused_params.items() if k in ("lr", "eps", "beta1", "beta2", "weight_decay")})
        return EmbCacheShardedEmbeddingBagCollection(module, env or self.env or ShardingEnv(1, 0, None),
                                                     device or self.device or module.device, spec)

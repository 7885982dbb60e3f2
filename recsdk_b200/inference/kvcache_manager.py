"""Paged KV-cache manager for HSTU-style generative-recommender inference.

Per request batch: ``lookup_kvcache`` (what is cached where) -> ``allocate_kvcache`` (pages for the whole
history, packed metadata on the device) -> ``onboard_launch`` (host-resident prefixes travel host -> device on a
side stream, layer by layer) -> per layer: ``handle.stream_wait_layer(l)``, ``append_kvcache`` of the new tokens,
paged attention -> ``offload_launch`` (full chunks that only live on the device are copied to pinned host
memory) -> ``offload_try_wait``.  Failures of the host tier degrade to recomputation (``fail_open``) or raise
(``fail_close``); page locks are released on every path.

API surface and behaviour follow the reference (``inference/kvcache_manager/recsys_kvcache_manager/*.py``,
``src/npu_kvcache_manager_impl.cpp``, ``src/native_host_kvcache_manager_impl.cpp``, ``docs/codeview.md``).
The page allocator and the host chunk index are native (``csrc/host/kvcache.h``); the device kernels are in
``csrc/cuda/hstu_misc.cu`` (append, positions) and ``csrc/cuda/embedding.cu`` (``rb_copy_rows``).  Unlike the
reference's staging-buffer pipeline (H2D copy, then a scatter kernel), the host pool is stored page-major in
pinned memory and ONE kernel per layer moves pages directly between it and the paged cache through the unified
address space, so a transfer costs one launch per layer whatever the batch.
"""
from __future__ import annotations

import abc
import dataclasses
import enum
import time
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

from ..host import host
from ..ops import _lib
from ..ops import embedding_ops as E


class KVCacheOffloadMode(str, enum.Enum):
    LAZY = "lazy"
    EAGER = "eager"


class HostKVStorageBackend(str, enum.Enum):
    NATIVE_HOST = "native_host"


class HostKVStorageFailPolicy(str, enum.Enum):
    FAIL_OPEN = "fail_open"
    FAIL_CLOSE = "fail_close"


@dataclasses.dataclass
class KVCacheConfig:
    num_layers: int
    num_heads: int
    head_dim: int
    page_size: int
    offload_chunksize: int
    num_primary_cache_pages: int
    num_buffer_pages: int
    host_capacity_per_layer: int          # bytes of pinned host memory per layer
    max_batch_size: int
    max_seq_len: int
    dtype: torch.dtype
    device: Any
    host_kvstorage_backend: str = HostKVStorageBackend.NATIVE_HOST.value
    onload_timeout_ms: float = 0.0
    offload_timeout_ms: float = 1000.0
    offload_mode: str = KVCacheOffloadMode.LAZY.value
    host_kvstorage_fail_policy: str = HostKVStorageFailPolicy.FAIL_OPEN.value
    extra_configs: Dict[str, Any] = dataclasses.field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.offload_chunksize % self.page_size:
            raise ValueError("offload_chunksize must be a multiple of page_size")
        if self.head_dim not in (64, 128, 256, 512):
            raise ValueError("head_dim must be one of 64, 128, 256, 512")
        if self.host_kvstorage_backend != HostKVStorageBackend.NATIVE_HOST.value:
            raise ValueError("unknown host_kvstorage_backend %r" % (self.host_kvstorage_backend,))

    def torch_device(self) -> torch.device:
        if isinstance(self.device, torch.device):
            return self.device
        if isinstance(self.device, int):
            return torch.device("cuda", self.device) if torch.cuda.is_available() else torch.device("cpu")
        return torch.device(self.device)


def get_kvcache_config(num_layers, num_heads, head_dim, page_size, offload_chunksize, num_primary_cache_pages,
                       num_buffer_pages, host_capacity_per_layer, max_batch_size, max_seq_len, dtype, device,
                       host_kvstorage_backend=HostKVStorageBackend.NATIVE_HOST.value, onload_timeout_ms=0.0,
                       offload_timeout_ms=0.0, offload_mode=KVCacheOffloadMode.LAZY.value,
                       host_kvstorage_fail_policy=HostKVStorageFailPolicy.FAIL_OPEN.value, extra_configs=None) -> KVCacheConfig:
    return KVCacheConfig(num_layers, num_heads, head_dim, page_size, offload_chunksize, num_primary_cache_pages,
                         num_buffer_pages, host_capacity_per_layer, max_batch_size, max_seq_len, dtype, device,
                         host_kvstorage_backend, onload_timeout_ms, offload_timeout_ms, offload_mode,
                         host_kvstorage_fail_policy, dict(extra_configs or {}))


@dataclasses.dataclass
class KVIndexMeta:
    user_ids: torch.Tensor            # int64 [B] (host)
    sequence_lengths: torch.Tensor    # int32 [B] total history length per user (host)


@dataclasses.dataclass
class KVLookupResult:
    user_ids: torch.Tensor
    cached_start_indices: torch.Tensor      # merged view over both tiers
    cached_lengths: torch.Tensor
    npu_cached_start_indices: Optional[torch.Tensor] = None
    npu_cached_lengths: Optional[torch.Tensor] = None
    host_cached_start_indices: Optional[torch.Tensor] = None
    host_cached_lengths: Optional[torch.Tensor] = None
    token_ids: Optional[torch.Tensor] = None
    token_mask: Optional[torch.Tensor] = None
    extra: Dict[str, Any] = dataclasses.field(default_factory=dict)

    @staticmethod
    def merge(user_ids, dev_start, dev_len, host_start, host_len) -> "KVLookupResult":
        """Usable cached prefix = [0, max(device end, host end)): the host tier always starts at token 0 and the
        device only drops a prefix after it reached the host, so the two ranges never leave a gap."""
        end = torch.maximum(dev_start + dev_len, host_start + host_len)
        return KVLookupResult(user_ids, torch.zeros_like(end), end, dev_start, dev_len, host_start, host_len)


@dataclasses.dataclass
class KVCacheMetadata:
    page_ids_npu_buffer: torch.Tensor
    metadata_npu_buffer: torch.Tensor
    kv_indices: torch.Tensor
    kv_indptr: torch.Tensor
    kv_last_page_len: torch.Tensor
    total_history_lengths: torch.Tensor
    total_history_offsets: torch.Tensor
    new_history_offsets: torch.Tensor
    batch_indices: torch.Tensor
    position: torch.Tensor
    new_history_nnz: int
    new_history_nnz_npu: torch.Tensor
    kv_seqlens: Optional[torch.Tensor] = None
    kv_seqlen_offsets: Optional[torch.Tensor] = None
    kv_cache_table: Optional[torch.Tensor] = None
    kv_onload_handle: Any = None
    max_seqlen: int = 0
    onboard_slot_mappings: Any = None
    onboard_task_ids: Any = None
    host_page_indptr: Optional[List[int]] = None      # host copies, for planning transfers without a D2H read
    host_page_ids: Optional[np.ndarray] = None


def get_kvcache_metadata_buffer(batch_size: int, num_new_tokens: int, num_pages: int, page_ids_npu_buffer: Optional[torch.Tensor] = None,
                                metadata_npu_buffer: Optional[torch.Tensor] = None, device=None) -> KVCacheMetadata:
    """A metadata record over preallocated (or given) buffers, sized for ``batch_size`` requests, ``num_new_tokens`` new
    tokens and ``num_pages`` pages: the static buffers a captured graph reads while ``copy_kvcache_metadata`` refreshes them
    (``kvcache_metadata.py:64-123`` of the reference; layout of the int32 buffer: page indptr ``[B+1]``, last-page lengths
    ``[B]``, total lengths ``[B]``, total offsets ``[B+1]``, new-token count ``[1]``, new offsets ``[B+1]``, batch index
    and position of every new token)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    elif isinstance(device, int):
        device = torch.device("cuda", device) if torch.cuda.is_available() else torch.device("cpu")
    device = torch.device(device)
    B, n = int(batch_size), int(num_new_tokens)
    pages = page_ids_npu_buffer if page_ids_npu_buffer is not None else torch.empty(int(num_pages), dtype=torch.int32, device=device)
    buf = metadata_npu_buffer if metadata_npu_buffer is not None else torch.empty(5 * B + 4 + 2 * n, dtype=torch.int32, device=device)
    if buf.numel() < 5 * B + 4 + 2 * n:
        raise ValueError("metadata buffer holds %d ints, %d are needed" % (buf.numel(), 5 * B + 4 + 2 * n))
    tot_len, tot_off = buf.narrow(0, 2 * B + 1, B), buf.narrow(0, 3 * B + 1, B + 1)
    return KVCacheMetadata(
        page_ids_npu_buffer=pages, metadata_npu_buffer=buf, kv_indices=pages, kv_indptr=buf.narrow(0, 0, B + 1),
        kv_last_page_len=buf.narrow(0, B + 1, B), total_history_lengths=tot_len, total_history_offsets=tot_off,
        new_history_offsets=buf.narrow(0, 4 * B + 3, B + 1), batch_indices=buf.narrow(0, 5 * B + 4, n),
        position=buf.narrow(0, 5 * B + 4 + n, n), new_history_nnz=n, new_history_nnz_npu=buf.narrow(0, 4 * B + 2, 1),
        kv_seqlens=torch.empty_like(tot_len), kv_seqlen_offsets=torch.empty_like(tot_off), kv_onload_handle=None)


def copy_kvcache_metadata(dst_metadata: KVCacheMetadata, src_metadata: KVCacheMetadata) -> None:
    """Refresh preallocated metadata from a step's metadata: value lists are copied and zero-padded, offset lists are copied
    and padded with their last entry (so the padding describes empty requests) (``kvcache_metadata.py:126-150``)."""
    def copy_tensor(dst, src):
        k = src.shape[0]
        if k > dst.shape[0]:
            raise ValueError("destination buffer holds %d entries, the source %d" % (dst.shape[0], k))
        dst[:k].copy_(src, non_blocking=True)
        dst[k:] = 0

    def copy_offsets(dst, src):
        k = src.shape[0]
        if k > dst.shape[0]:
            raise ValueError("destination buffer holds %d entries, the source %d" % (dst.shape[0], k))
        dst[:k].copy_(src, non_blocking=True)
        if k:
            dst[k:] = src[-1]

    d, s = dst_metadata, src_metadata
    copy_tensor(d.kv_indices, s.kv_indices)
    copy_offsets(d.kv_indptr, s.kv_indptr)
    copy_tensor(d.kv_last_page_len, s.kv_last_page_len)
    copy_tensor(d.batch_indices, s.batch_indices)
    copy_tensor(d.position, s.position)
    copy_tensor(d.new_history_nnz_npu, s.new_history_nnz_npu)
    copy_offsets(d.total_history_offsets, s.total_history_offsets)
    copy_offsets(d.new_history_offsets, s.new_history_offsets)
    copy_tensor(d.kv_seqlens, s.kv_seqlens)
    copy_offsets(d.kv_seqlen_offsets, s.kv_seqlen_offsets)
    d.new_history_nnz = s.new_history_nnz
    d.kv_onload_handle = s.kv_onload_handle


class HostKVTaskStatus(enum.Enum):
    UNINITIALIZED = "uninitialized"
    SKIPPED = "skipped"
    LAUNCHED = "launched"
    READY = "ready"
    EVENT_READY = "event_ready"
    TIMEOUT = "timeout"
    FAILED = "failed"
    CANCELLED = "cancelled"


class HostKVStorageErrorCode(str, enum.Enum):
    SDK_IMPORT_FAILED = "sdk_import_failed"
    SDK_INIT_FAILED = "sdk_init_failed"
    LOOKUP_FAILED = "lookup_failed"
    LOOKUP_MISSING_TOKENS = "lookup_missing_tokens"
    ONBOARD_TASK_NOT_FOUND = "onboard_task_not_found"
    ONBOARD_WAIT_FAILED = "onboard_wait_failed"
    ONBOARD_TIMEOUT = "onboard_timeout"
    OFFLOAD_TASK_NOT_FOUND = "offload_task_not_found"
    OFFLOAD_WAIT_FAILED = "offload_wait_failed"
    OFFLOAD_TIMEOUT = "offload_timeout"
    OFFLOAD_NO_SPACE = "offload_no_space"
    CANCEL_FAILED = "cancel_failed"


@dataclasses.dataclass
class HostKVTaskHandle:
    backend: str = "native"
    user_ids: Optional[torch.Tensor] = None
    handle: Any = None
    status: HostKVTaskStatus = HostKVTaskStatus.UNINITIALIZED
    metadata: Optional[Dict[str, Any]] = None
    time_launched: Optional[float] = None
    is_layerwise: bool = False
    layer_events: Optional[List[Any]] = None

    def stream_wait_layer(self, layer_idx: int) -> None:
        """Make the current stream wait until layer ``layer_idx`` of an onboard task has landed in its pages."""
        if self.layer_events and self.layer_events[layer_idx] is not None:
            ev = self.layer_events[layer_idx]
            if hasattr(ev, "storage"):                     # a layer of a native storage task
                ev.wait(torch.cuda.current_stream())
            else:
                torch.cuda.current_stream().wait_event(ev)


@dataclasses.dataclass
class HostKVWaitResult:
    status: HostKVTaskStatus
    ready: Optional[bool] = None          # None: derived from the status (ready / event-ready / skipped count as ready)
    message: str = ""
    failed_mask: Optional[torch.Tensor] = None
    failed_user_ids: Optional[List[int]] = None
    error_code: Optional[HostKVStorageErrorCode] = None

    def __post_init__(self) -> None:
        if self.ready is None:
            self.ready = self.status in (HostKVTaskStatus.READY, HostKVTaskStatus.EVENT_READY, HostKVTaskStatus.SKIPPED)


class HostKVStorageManagerBase(abc.ABC):
    """Contract of a host KV tier (reference ``host_kvstorage_manager.py``)."""

    @abc.abstractmethod
    def register_npu_cache_tables(self, cache_table_list: List[torch.Tensor]) -> None: ...

    @abc.abstractmethod
    def build_index_meta(self, user_ids: torch.Tensor, sequence_lengths: torch.Tensor) -> KVIndexMeta: ...

    @abc.abstractmethod
    def lookup_kvcache(self, index_meta: KVIndexMeta) -> Tuple[torch.Tensor, torch.Tensor]: ...

    @abc.abstractmethod
    def onboard_kvcache_launch(self, index_meta, lookup_result, kvcache_metadata) -> HostKVTaskHandle: ...

    @abc.abstractmethod
    def onboard_kvcache_wait(self, task_handle: HostKVTaskHandle) -> HostKVWaitResult: ...

    @abc.abstractmethod
    def offload_kvcache_launch(self, user_ids, start_indices, page_lists, index_meta=None, kvcache_metadata=None) -> HostKVTaskHandle: ...

    @abc.abstractmethod
    def offload_kvcache_wait(self, task_handle: HostKVTaskHandle) -> HostKVWaitResult: ...

    @abc.abstractmethod
    def finish_task(self, task_handle: HostKVTaskHandle) -> List[int]: ...

    @abc.abstractmethod
    def cancel_task(self, task_handle: HostKVTaskHandle) -> bool: ...

    @abc.abstractmethod
    def evict(self, user_ids: torch.Tensor) -> None: ...

    @abc.abstractmethod
    def evict_all(self) -> None: ...

    @staticmethod
    def get_offload_handle_metadata(task_handle: HostKVTaskHandle) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """-> (user ids, start token of each user's offloaded range, tokens offloaded) of an offload task."""
        md = task_handle.metadata or {}
        uids = task_handle.user_ids if task_handle.user_ids is not None else torch.zeros(0, dtype=torch.int64)
        n = uids.numel()
        return (uids, torch.tensor(list(md.get("starts", [0] * n)), dtype=torch.int32),
                torch.tensor(list(md.get("lengths", [0] * n)), dtype=torch.int32))


def _np64(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().numpy().astype(np.int64))


def _np32(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().numpy().astype(np.int32))


# =============================================================================== device tier
class GPUKVCacheManager:
    """Owns the cache tensor ``[layers, pages, 2, page_size, heads, head_dim]`` and the native page allocator."""

    def __init__(self, cfg: KVCacheConfig) -> None:
        self.cfg = cfg
        self.device = cfg.torch_device()
        self.impl = host().KVPageAllocator(cfg.page_size, cfg.offload_chunksize, cfg.num_primary_cache_pages,
                                           cfg.num_buffer_pages, cfg.max_batch_size, cfg.max_seq_len)
        self.cache = torch.zeros(cfg.num_layers, cfg.num_primary_cache_pages, 2, cfg.page_size, cfg.num_heads, cfg.head_dim,
                                 dtype=cfg.dtype, device=self.device)
        self.max_offload_pages = int(cfg.extra_configs.get("max_offload_pages", cfg.num_primary_cache_pages))

    def get_cache_table(self, layer: int) -> torch.Tensor:
        return self.cache[layer]

    def get_cache_tables(self, layer_idx: int = -1):
        """All per-layer cache tables (``layer_idx = -1``) or one of them."""
        return [self.cache[l] for l in range(self.cfg.num_layers)] if layer_idx == -1 else self.cache[layer_idx]

    def get(self, page_ids, last_page_lens, layer_idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """K and V ``[tokens, heads, head_dim]`` of one sequence: its pages in order, the last one cut at ``last_page_lens``."""
        table = self.cache[layer_idx]
        pages = torch.as_tensor(page_ids, device=table.device).long()
        n = pages.numel() * self.cfg.page_size - (self.cfg.page_size - int(last_page_lens)) if pages.numel() else 0
        k = table[pages, 0].reshape(-1, self.cfg.num_heads, self.cfg.head_dim)[:n].clone()
        v = table[pages, 1].reshape(-1, self.cfg.num_heads, self.cfg.head_dim)[:n].clone()
        return k, v

    def lookup(self, user_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        s, l = self.impl.lookup(_np64(user_ids))
        return torch.from_numpy(s.astype(np.int32)), torch.from_numpy(l.astype(np.int32))

    def allocate(self, user_ids: torch.Tensor, total_lens: torch.Tensor, host_cached_lens: torch.Tensor) -> KVCacheMetadata:
        B = user_ids.numel()
        pages, meta, nnz = self.impl.allocate(_np64(user_ids), _np32(total_lens), _np32(host_cached_lens))
        nnz = int(nnz)
        dev = self.device
        cuda = dev.type == "cuda"
        pages_t, meta_t = torch.from_numpy(pages.astype(np.int32)), torch.from_numpy(meta.astype(np.int32))
        if cuda:
            pages_t, meta_t = pages_t.pin_memory(), meta_t.pin_memory()
        page_buf = pages_t.to(dev, non_blocking=True)
        buf = torch.empty(5 * B + 4 + 2 * nnz, dtype=torch.int32, device=dev)
        buf[: 5 * B + 4].copy_(meta_t, non_blocking=True)
        indptr = buf[0:B + 1]
        last = buf[B + 1:2 * B + 1]
        tot_len = buf[2 * B + 1:3 * B + 1]
        tot_off = buf[3 * B + 1:4 * B + 2]
        new_off = buf[4 * B + 3:5 * B + 4]
        bidx = buf[5 * B + 4:5 * B + 4 + nnz]
        pos = buf[5 * B + 4 + nnz:5 * B + 4 + 2 * nnz]
        if nnz:
            if cuda:
                rc = _lib.lib().rb_kv_positions(new_off.data_ptr(), tot_len.data_ptr(), B, bidx.data_ptr(), pos.data_ptr(),
                                                _lib.stream_ptr(dev))
                _lib.check(rc, "rb_kv_positions")
            else:
                no, tl = new_off.tolist(), tot_len.tolist()
                for b in range(B):
                    n = no[b + 1] - no[b]
                    bidx[no[b]:no[b + 1]] = b
                    pos[no[b]:no[b + 1]] = torch.arange(tl[b] - n, tl[b], dtype=torch.int32)
        return KVCacheMetadata(page_buf, buf, page_buf, indptr, last, tot_len, tot_off, new_off, bidx, pos, nnz,
                               buf[4 * B + 2:4 * B + 3], kv_seqlens=tot_len, kv_seqlen_offsets=tot_off,
                               max_seqlen=int(total_lens.max().item()) if B else 0,
                               host_page_indptr=meta[: B + 1].tolist(), host_page_ids=np.asarray(pages, dtype=np.int64))

    def append_kvcache(self, layer: int, k: torch.Tensor, v: torch.Tensor, md: KVCacheMetadata) -> None:
        """Write the new tokens' K/V ``[nnz, heads, head_dim]`` of one layer into their pages."""
        nnz = md.new_history_nnz
        if nnz == 0:
            return
        cache = self.cache[layer]
        row_bytes = self.cfg.num_heads * self.cfg.head_dim * cache.element_size()
        if cache.is_cuda:
            k, v = k.contiguous(), v.contiguous()
            rc = _lib.lib().rb_kv_append_paged(k.data_ptr(), v.data_ptr(), md.batch_indices.data_ptr(), md.position.data_ptr(),
                                               md.kv_indices.data_ptr(), md.kv_indptr.data_ptr(), nnz, self.cfg.page_size,
                                               row_bytes, cache.data_ptr(), _lib.num_sms(cache.device), _lib.stream_ptr(cache.device))
            _lib.check(rc, "rb_kv_append_paged")
            return
        ps = self.cfg.page_size
        b, p = md.batch_indices.long(), md.position.long()
        page = md.kv_indices.long()[md.kv_indptr.long()[b] + p // ps]
        cache[page, 0, p % ps] = k.to(cache.dtype)
        cache[page, 1, p % ps] = v.to(cache.dtype)

    put = append_kvcache

    # ---- offload bookkeeping (thin wrappers over the native allocator)
    def check_for_offload(self, user_ids: torch.Tensor) -> torch.Tensor:
        return torch.from_numpy(np.asarray(self.impl.check_for_offload(_np64(user_ids), self.max_offload_pages), dtype=np.int64))

    def acquire_offload_pages(self, user_ids: torch.Tensor, offloaded_lengths: Optional[torch.Tensor] = None, always_offload=False):
        u, s, pages = self.impl.acquire_offload_pages(_np64(user_ids), None if offloaded_lengths is None else _np32(offloaded_lengths),
                                                      always_offload)
        return (torch.from_numpy(np.asarray(u, dtype=np.int64)), torch.from_numpy(np.asarray(s, dtype=np.int32)),
                [np.asarray(p, dtype=np.int64) for p in pages])

    def release_offload_pages(self, user_ids, start, lengths, done: List[int]) -> None:
        self.impl.release_offload_pages(_np64(user_ids), _np32(start), _np32(lengths), np.asarray(done, dtype=np.uint8))

    def revoke_onboard_pages(self, user_ids, start, lengths) -> None:
        self.impl.revoke_onboard_pages(_np64(user_ids), _np32(start), _np32(lengths))

    def evict(self, user_ids: torch.Tensor) -> None:
        for u in user_ids.tolist():
            self.impl.evict(int(u))

    def truncate(self, user_ids: torch.Tensor, lengths: torch.Tensor) -> None:
        """Drop every token at or beyond ``lengths[i]`` of user i (request-scoped tokens such as ranking candidates)."""
        for u, n in zip(user_ids.tolist(), lengths.tolist()):
            self.impl.truncate(int(u), int(n))

    def evict_all(self) -> None:
        self.impl.evict_all()


NPUKVCacheManager = GPUKVCacheManager   # the name the reference API uses for the device tier


# =============================================================================== host tier
class _NativeLayerEvent:
    """One layer of a transfer task of the native storage: ``query()`` like a CUDA event, ``wait(stream)`` for a stream."""

    def __init__(self, storage: "NativeKVStorage", task: int, layer: int) -> None:
        self.storage, self.task, self.layer = storage, task, layer
        self.done = False                 # seen complete: the task slot may have been given back since

    def query(self) -> bool:
        if self.done:
            return True
        rc = self.storage.query(self.task, self.layer)
        if rc < 0:
            raise RuntimeError("KV storage task %d layer %d: error %d" % (self.task, self.layer, rc))
        self.done = rc == 0
        return self.done

    def wait(self, stream=None) -> None:
        if not self.done:
            self.storage.stream_wait(self.task, self.layer, stream)


class NativeKVStorage:
    """The native host tier (``csrc/cuda/kv_storage.cu``): pinned chunk pool ``[chunk][layer][rows_per_chunk_layer][row]``,
    four streams (H2D, scatter, gather, D2H), two staging slots per direction and one event per layer of every task.
    ``pool`` is a tensor view of the pinned memory (for inspection, export and tests)."""

    def __init__(self, device: torch.device, num_layers: int, num_chunks: int, rows_per_chunk_layer: int, row_elems: int,
                 dtype: torch.dtype, stage_rows: int) -> None:
        import ctypes

        self.device, self.num_layers = device, num_layers
        self._lib = _lib.lib()
        item = torch.empty(0, dtype=dtype).element_size()
        h = ctypes.c_void_p()
        _lib.check(self._lib.rb_kvs_create(device.index or 0, num_layers, num_chunks, rows_per_chunk_layer, row_elems * item,
                                           int(stage_rows), ctypes.byref(h)), "rb_kvs_create")
        self._h = h
        nbytes = int(self._lib.rb_kvs_pool_bytes(self._h))
        buf = (ctypes.c_uint8 * nbytes).from_address(int(self._lib.rb_kvs_pool(self._h)))
        self._buf = buf
        self.pool = torch.frombuffer(buf, dtype=torch.uint8).view(dtype).view(num_chunks, num_layers, rows_per_chunk_layer, row_elems)
        self.pool.zero_()

    def register_cache(self, layer: int, rows: torch.Tensor) -> None:
        _lib.check(self._lib.rb_kvs_register_cache(self._h, layer, rows.data_ptr()), "rb_kvs_register_cache")

    def _transfer(self, fn, chunks: np.ndarray, rows: np.ndarray) -> Tuple[int, int]:
        import ctypes

        chunks = np.ascontiguousarray(chunks, dtype=np.int64)
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        task = ctypes.c_int(-1)
        rc = fn(self._h, chunks.ctypes.data, len(chunks), rows.ctypes.data, _lib.stream_ptr(self.device), ctypes.byref(task))
        if rc < 0:
            _lib.check(rc, "rb_kvs transfer")
        return int(task.value), int(rc)

    def onload(self, chunks: np.ndarray, dst_rows: np.ndarray) -> Tuple[int, int]:
        """-> (task id, 0 or the error of the call that failed while launching)."""
        return self._transfer(self._lib.rb_kvs_onload, chunks, dst_rows)

    def offload(self, chunks: np.ndarray, src_rows: np.ndarray) -> Tuple[int, int]:
        return self._transfer(self._lib.rb_kvs_offload, chunks, src_rows)

    def query(self, task: int, layer: int = -1) -> int:
        return int(self._lib.rb_kvs_task_query(self._h, task, layer))

    def stream_wait(self, task: int, layer: int, stream=None) -> None:
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        _lib.check(self._lib.rb_kvs_task_stream_wait(self._h, task, layer, st), "rb_kvs_task_stream_wait")

    def release(self, task: int, drain: bool = False) -> bool:
        """-> True when the slot was given back (a running task is only released with ``drain``)."""
        rc = int(self._lib.rb_kvs_task_release(self._h, task, 1 if drain else 0))
        if rc > 1 or rc < 0:
            _lib.check(rc, "rb_kvs_task_release")
        return rc == 0

    def inject_failure(self, countdown: int) -> None:
        self._lib.rb_kvs_inject_failure(self._h, int(countdown))

    def stats(self) -> Dict[str, int]:
        import ctypes

        out = (ctypes.c_longlong * 4)()
        self._lib.rb_kvs_stats(self._h, out)
        return {"h2d_bytes": out[0], "d2h_bytes": out[1], "copy_calls": out[2], "kernels": out[3]}

    def close(self) -> None:
        if self._h is not None:
            self.pool = None
            self._buf = None
            self._lib.rb_kvs_destroy(self._h)
            self._h = None

    def __del__(self) -> None:  # noqa: D401
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


class NativeHostKVCacheManager(HostKVStorageManagerBase):
    """Pinned host chunk store, page-major: ``pool[chunk, layer, page_in_chunk, 2, page_size * heads * head_dim]``.
    A row of the flattened pool is one K or V page, the same unit as a row of the flattened device cache, so
    moving a layer is one ``copy_rows`` launch on a side stream followed by one event."""

    def __init__(self, cfg: KVCacheConfig) -> None:
        self.cfg = cfg
        self.device = cfg.torch_device()
        self.cuda = self.device.type == "cuda"
        hd = cfg.num_heads * cfg.head_dim
        item = torch.empty(0, dtype=cfg.dtype).element_size()
        self.row_elems = cfg.page_size * hd
        self.ppc = cfg.offload_chunksize // cfg.page_size
        chunk_bytes_per_layer = 2 * cfg.offload_chunksize * hd * item
        self.num_chunks = max(1, int(cfg.host_capacity_per_layer // chunk_bytes_per_layer))
        self.index = host().HostChunkIndex(self.num_chunks, cfg.offload_chunksize)
        # transfer engine: "staged" (CUDA default) = native storage with DMA copies through device staging buffers on four
        # streams; "zero_copy" = one kernel per layer that reads / writes the pinned pool through the unified address space
        self.transfer = str(cfg.extra_configs.get("host_transfer", "staged" if self.cuda else "zero_copy"))
        if self.transfer not in ("staged", "zero_copy") or (self.transfer == "staged" and not self.cuda):
            raise ValueError("host_transfer must be 'staged' (CUDA only) or 'zero_copy'")
        self.native: Optional[NativeKVStorage] = None
        if self.transfer == "staged":
            stage_rows = int(cfg.extra_configs.get("staging_rows", max(2 * self.ppc, 2 * min(cfg.max_seq_len, 8192) // cfg.page_size)))
            self.native = NativeKVStorage(self.device, cfg.num_layers, self.num_chunks, self.ppc * 2, self.row_elems, cfg.dtype,
                                          stage_rows)
            self.pool = self.native.pool.view(self.num_chunks, cfg.num_layers, self.ppc, 2, self.row_elems)
        else:
            self.pool = torch.zeros(self.num_chunks, cfg.num_layers, self.ppc, 2, self.row_elems, dtype=cfg.dtype,
                                    pin_memory=self.cuda)
        self.pool_rows = self.pool.view(-1, self.row_elems)
        self.cache_rows: List[torch.Tensor] = []
        if self.cuda:
            self.onboard_stream, self.offload_stream = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        self.fail_next_offload = False        # test hook: the next offload reports a failed copy (host-side injection)
        self.fail_next_onboard = False

    def register_npu_cache_tables(self, cache_table_list: List[torch.Tensor]) -> None:
        self.cache_rows = [t.view(-1, self.row_elems) for t in cache_table_list]        # rows: (page, kv)
        if self.native is not None:
            for layer, rows in enumerate(self.cache_rows):
                self.native.register_cache(layer, rows)

    def build_index_meta(self, user_ids, sequence_lengths) -> KVIndexMeta:
        return KVIndexMeta(user_ids.cpu().long(), sequence_lengths.cpu().int())

    def lookup_kvcache(self, index_meta: KVIndexMeta):
        s, l = self.index.lookup(_np64(index_meta.user_ids))
        return torch.from_numpy(s.astype(np.int32)), torch.from_numpy(l.astype(np.int32))

    def _pool_rows_of(self, chunks: np.ndarray, layer: int) -> np.ndarray:
        """Row numbers, in token order, of all (page, kv) rows of ``chunks`` for ``layer``."""
        per = self.ppc * 2
        base = (chunks.astype(np.int64) * self.cfg.num_layers + layer) * per
        return (base[:, None] + np.arange(per, dtype=np.int64)[None, :]).reshape(-1)

    @staticmethod
    def _cache_rows_of(pages: np.ndarray) -> np.ndarray:
        p = pages.astype(np.int64)
        return np.stack([p * 2, p * 2 + 1], axis=1).reshape(-1)

    def _idx(self, a: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(a)
        return t.pin_memory().to(self.device, non_blocking=True) if self.cuda else t

    def onboard_kvcache_launch(self, index_meta, lookup_result, kvcache_metadata) -> HostKVTaskHandle:
        """Copy every host-resident prefix that the device does not hold into the pages just allocated for it."""
        cfg = self.cfg
        uids = index_meta.user_ids.tolist()
        dev_start = lookup_result.npu_cached_start_indices.tolist()
        dev_len = lookup_result.npu_cached_lengths.tolist()
        host_len = lookup_result.host_cached_lengths.tolist()
        indptr, page_ids = kvcache_metadata.host_page_indptr, kvcache_metadata.host_page_ids
        jobs = []                                   # (uid, tokens, chunk ids, destination pages)
        for b, u in enumerate(uids):
            need = host_len[b] if dev_len[b] == 0 else min(dev_start[b], host_len[b])
            need = (need // cfg.offload_chunksize) * cfg.offload_chunksize
            if need <= 0:
                continue
            chunks = np.asarray(self.index.chunks_of(int(u), 0, need), dtype=np.int64)
            if len(chunks) * cfg.offload_chunksize < need:
                raise RuntimeError("host index lost chunks of user %d between lookup and onboard" % u)
            jobs.append((int(u), need, chunks, page_ids[indptr[b]: indptr[b] + need // cfg.page_size]))
        h = HostKVTaskHandle(user_ids=index_meta.user_ids, status=HostKVTaskStatus.SKIPPED, time_launched=time.time(), is_layerwise=True,
                             metadata={"jobs": [(u, n) for u, n, _c, _p in jobs]})
        if not jobs:
            return h
        if self.fail_next_onboard:
            self.fail_next_onboard = False
            raise RuntimeError("injected onboard failure")
        if self.native is not None:
            task, err = self.native.onload(np.concatenate([c for _u, _n, c, _p in jobs]),
                                           np.concatenate([self._cache_rows_of(p) for _u, _n, _c, p in jobs]))
            h.handle = task
            if err:
                self.native.release(task, drain=True)
                raise RuntimeError("onboard copy failed while launching (CUDA error %d)" % err)
            h.layer_events = [_NativeLayerEvent(self.native, task, layer) for layer in range(cfg.num_layers)]
            h.status = HostKVTaskStatus.LAUNCHED
            return h
        dst = self._idx(np.concatenate([self._cache_rows_of(p) for _u, _n, _c, p in jobs]))
        src_all = self._idx(np.stack([np.concatenate([self._pool_rows_of(c, layer) for _u, _n, c, _p in jobs])
                                      for layer in range(cfg.num_layers)]))
        events: List[Any] = [None] * cfg.num_layers
        if self.cuda:
            self.onboard_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.onboard_stream):
                for layer in range(cfg.num_layers):
                    E.copy_rows(self.pool_rows, src_all[layer], self.cache_rows[layer], dst, self.device)
                    events[layer] = torch.cuda.Event()
                    events[layer].record(self.onboard_stream)
            dst.record_stream(self.onboard_stream)
            src_all.record_stream(self.onboard_stream)
        else:
            for layer in range(cfg.num_layers):
                E.copy_rows(self.pool_rows, src_all[layer], self.cache_rows[layer], dst)
        h.layer_events, h.status = events, HostKVTaskStatus.LAUNCHED
        return h

    def _poll(self, events, limit_ms: float) -> bool:
        t0 = time.time()
        for ev in events or []:
            if ev is None:
                continue
            while not ev.query():
                if limit_ms > 0 and (time.time() - t0) * 1e3 > limit_ms:
                    return False
                time.sleep(0.0001)
        return True

    def onboard_kvcache_wait(self, task_handle: HostKVTaskHandle) -> HostKVWaitResult:
        if task_handle.status == HostKVTaskStatus.SKIPPED:
            return HostKVWaitResult(HostKVTaskStatus.SKIPPED)
        if not self._poll(task_handle.layer_events, self.cfg.onload_timeout_ms):
            task_handle.status = HostKVTaskStatus.TIMEOUT
            return HostKVWaitResult(HostKVTaskStatus.TIMEOUT, error_code=HostKVStorageErrorCode.ONBOARD_TIMEOUT, message="onboard timed out")
        if self.native is not None and task_handle.handle is not None:
            self.native.release(task_handle.handle)
            task_handle.handle = None
        task_handle.status = HostKVTaskStatus.READY
        return HostKVWaitResult(HostKVTaskStatus.READY)

    def onboard_kvcache_wait_by_layer(self, task_handle: HostKVTaskHandle, layer_idx: int) -> HostKVWaitResult:
        """Make the current stream wait for one layer of an onboard task (no host wait): the attention of layer ``layer_idx``
        may then be enqueued while later layers are still in flight."""
        if task_handle.status == HostKVTaskStatus.SKIPPED or not task_handle.layer_events:
            return HostKVWaitResult(HostKVTaskStatus.SKIPPED)
        if self.cuda:
            task_handle.stream_wait_layer(layer_idx)
        return HostKVWaitResult(HostKVTaskStatus.EVENT_READY)

    def offload_kvcache_launch(self, user_ids, start_indices, page_lists, index_meta=None, kvcache_metadata=None) -> HostKVTaskHandle:
        """Copy whole chunks (``start`` is chunk-aligned by construction) from device pages into new host chunks."""
        cfg = self.cfg
        uids, starts = user_ids.tolist(), start_indices.tolist()
        pinned = [int(u) for u in uids]
        plan, lengths, no_space = [], [], []
        for u, s, pages in zip(uids, starts, page_lists):
            n_chunks = len(pages) // self.ppc
            n_tok = n_chunks * cfg.offload_chunksize
            chunks = np.asarray(self.index.append(int(u), int(s), n_tok, pinned), dtype=np.int64) if n_tok > 0 else np.zeros(0, np.int64)
            if n_tok > 0 and len(chunks) == 0:
                no_space.append(int(u))
                lengths.append(0)
                continue
            if n_tok > 0:
                plan.append((int(u), chunks, np.asarray(pages[: n_chunks * self.ppc], dtype=np.int64)))
            lengths.append(n_tok)
        h = HostKVTaskHandle(user_ids=user_ids, status=HostKVTaskStatus.LAUNCHED, time_launched=time.time(),
                             metadata={"plan": plan, "lengths": lengths, "starts": starts, "no_space": no_space})
        if not plan:
            h.status = HostKVTaskStatus.SKIPPED
            return h
        if self.native is not None:
            task, err = self.native.offload(np.concatenate([c for _u, c, _p in plan]),
                                            np.concatenate([self._cache_rows_of(p) for _u, _c, p in plan]))
            h.handle = task
            h.metadata["launch_error"] = err
            h.layer_events = [_NativeLayerEvent(self.native, task, cfg.num_layers - 1)] if not err else []
            return h
        src = self._idx(np.concatenate([self._cache_rows_of(p) for _u, _c, p in plan]))
        dst_all = self._idx(np.stack([np.concatenate([self._pool_rows_of(c, layer) for _u, c, _p in plan])
                                      for layer in range(cfg.num_layers)]))
        if self.cuda:
            self.offload_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.offload_stream):
                for layer in range(cfg.num_layers):
                    E.copy_rows(self.cache_rows[layer], src, self.pool_rows, dst_all[layer], self.device)
                ev = torch.cuda.Event()
                ev.record(self.offload_stream)
            src.record_stream(self.offload_stream)
            dst_all.record_stream(self.offload_stream)
            h.layer_events = [ev]
        else:
            for layer in range(cfg.num_layers):
                E.copy_rows(self.cache_rows[layer], src, self.pool_rows, dst_all[layer])
        return h

    def offload_kvcache_wait(self, task_handle: HostKVTaskHandle) -> HostKVWaitResult:
        no_space = (task_handle.metadata or {}).get("no_space") or None
        code = HostKVStorageErrorCode.OFFLOAD_NO_SPACE if no_space else None
        if task_handle.status == HostKVTaskStatus.SKIPPED:
            return HostKVWaitResult(HostKVTaskStatus.SKIPPED, error_code=code, failed_user_ids=no_space)
        if self.fail_next_offload:
            self.fail_next_offload = False
            if self.cuda:
                self.offload_stream.synchronize()
            task_handle.status = HostKVTaskStatus.FAILED
            return HostKVWaitResult(HostKVTaskStatus.FAILED, error_code=HostKVStorageErrorCode.OFFLOAD_WAIT_FAILED, message="injected copy failure")
        if (task_handle.metadata or {}).get("launch_error"):
            task_handle.status = HostKVTaskStatus.FAILED
            return HostKVWaitResult(HostKVTaskStatus.FAILED, error_code=HostKVStorageErrorCode.OFFLOAD_WAIT_FAILED,
                                    message="offload copy failed while launching (CUDA error %d)" % task_handle.metadata["launch_error"])
        if not self._poll(task_handle.layer_events, self.cfg.offload_timeout_ms):
            task_handle.status = HostKVTaskStatus.TIMEOUT
            return HostKVWaitResult(HostKVTaskStatus.TIMEOUT, error_code=HostKVStorageErrorCode.OFFLOAD_TIMEOUT, message="offload timed out")
        task_handle.status = HostKVTaskStatus.READY
        return HostKVWaitResult(HostKVTaskStatus.READY, error_code=code, failed_user_ids=no_space)

    def finish_task(self, task_handle: HostKVTaskHandle) -> List[int]:
        """-> per user 1 (offloaded) / 0 (not).  A failed, timed-out or cancelled task gives its chunks back; a
        timed-out copy may still be writing, so the stream is drained before the chunks can be reused."""
        plan = task_handle.metadata.get("plan", []) if task_handle.metadata else []
        ok = task_handle.status == HostKVTaskStatus.READY
        if self.native is not None and task_handle.handle is not None:
            self.native.release(task_handle.handle, drain=not ok)
            task_handle.handle = None
        if not ok and plan:
            if self.cuda and self.native is None:
                self.offload_stream.synchronize()
            for u, chunks, _p in plan:
                self.index.rollback(u, len(chunks))
        done_users = {u for u, _c, _p in plan} if ok else set()
        return [1 if int(u) in done_users else 0 for u in task_handle.user_ids.tolist()]

    def cancel_task(self, task_handle: HostKVTaskHandle) -> bool:
        task_handle.status = HostKVTaskStatus.CANCELLED
        self.finish_task(task_handle)
        return True

    def evict(self, user_ids: torch.Tensor) -> None:
        for u in user_ids.tolist():
            self.index.evict(int(u))

    def evict_all(self) -> None:
        self.index.evict_all()


# =============================================================================== orchestration
class KVCacheManager:
    def __init__(self, npu_kvcache_manager: GPUKVCacheManager, host_kvstorage_manager: Optional[HostKVStorageManagerBase],
                 offload_mode: str = KVCacheOffloadMode.LAZY.value,
                 host_kvstorage_fail_policy: str = HostKVStorageFailPolicy.FAIL_OPEN.value) -> None:
        self.gpu, self.host = npu_kvcache_manager, host_kvstorage_manager
        self.offload_mode, self.fail_policy = offload_mode, host_kvstorage_fail_policy
        if self.host is not None:
            self.host.register_npu_cache_tables([self.gpu.get_cache_table(l) for l in range(self.gpu.cfg.num_layers)])
        self._pending_offload: Optional[Tuple[HostKVTaskHandle, torch.Tensor, torch.Tensor, torch.Tensor]] = None
        self.stats = {"onboard_failures": 0, "offload_failures": 0, "offload_timeouts": 0, "offloaded_tokens": 0,
                      "onboarded_tokens": 0}

    @classmethod
    def from_config(cls, cfg: KVCacheConfig) -> "KVCacheManager":
        hostm = NativeHostKVCacheManager(cfg) if cfg.host_capacity_per_layer > 0 else None
        return cls(GPUKVCacheManager(cfg), hostm, cfg.offload_mode, cfg.host_kvstorage_fail_policy)

    def _fail(self, what: str, res: HostKVWaitResult) -> None:
        if self.fail_policy == HostKVStorageFailPolicy.FAIL_CLOSE.value:
            raise RuntimeError("%s failed: %s %s" % (what, res.error_code, res.message))

    def lookup_kvcache(self, user_ids: torch.Tensor, sequence_lengths: torch.Tensor) -> Tuple[KVIndexMeta, KVLookupResult]:
        meta = KVIndexMeta(user_ids.cpu().long(), sequence_lengths.cpu().int())
        ds, dl = self.gpu.lookup(meta.user_ids)
        if self.host is not None:
            got = self.host.lookup_kvcache(meta)
            if isinstance(got, KVLookupResult):                       # a backend written against the reference's contract
                hs = got.host_cached_start_indices if got.host_cached_start_indices is not None else got.cached_start_indices
                hl = got.host_cached_lengths if got.host_cached_lengths is not None else got.cached_lengths
            else:
                hs, hl = got
        else:
            hs, hl = torch.zeros_like(ds), torch.zeros_like(dl)
        return meta, KVLookupResult.merge(meta.user_ids, ds, dl, hs, hl)

    def allocate_kvcache(self, index_meta: KVIndexMeta, lookup_results: KVLookupResult,
                         output_kvcache_metadata: Optional[KVCacheMetadata] = None) -> KVCacheMetadata:
        md = self.gpu.allocate(index_meta.user_ids, index_meta.sequence_lengths,
                               torch.minimum(lookup_results.host_cached_lengths, index_meta.sequence_lengths))
        md.kv_cache_table = self.gpu.cache
        return md

    def _onboard_need(self, lookup_result: KVLookupResult) -> torch.Tensor:
        c = self.gpu.cfg.offload_chunksize
        need = torch.where(lookup_result.npu_cached_lengths == 0, lookup_result.host_cached_lengths,
                           torch.minimum(lookup_result.npu_cached_start_indices, lookup_result.host_cached_lengths))
        return (need // c) * c

    def onboard_launch(self, index_meta, lookup_result, kvcache_metadata) -> HostKVTaskHandle:
        if self.host is None:
            return HostKVTaskHandle(user_ids=index_meta.user_ids, status=HostKVTaskStatus.SKIPPED)
        try:
            h = self.host.onboard_kvcache_launch(index_meta, lookup_result, kvcache_metadata)
        except Exception as e:  # noqa: BLE001 - the host tier is best effort under fail_open
            self.stats["onboard_failures"] += 1
            self._fail("onboard", HostKVWaitResult(HostKVTaskStatus.FAILED, error_code=HostKVStorageErrorCode.ONBOARD_WAIT_FAILED, message=str(e)))
            return HostKVTaskHandle(user_ids=index_meta.user_ids, status=HostKVTaskStatus.FAILED,
                                    metadata={"need": self._onboard_need(lookup_result)})
        kvcache_metadata.kv_onload_handle = h
        self.stats["onboarded_tokens"] += sum(n for _u, n in h.metadata["jobs"])
        return h

    def onboard_try_wait(self, handle: HostKVTaskHandle) -> HostKVWaitResult:
        if self.host is None or handle.status in (HostKVTaskStatus.SKIPPED, HostKVTaskStatus.FAILED):
            return HostKVWaitResult(handle.status)
        res = self.host.onboard_kvcache_wait(handle)
        if res.status not in (HostKVTaskStatus.READY, HostKVTaskStatus.SKIPPED):
            self.stats["onboard_failures"] += 1
            self._fail("onboard", res)
        return res

    onboard_wait = onboard_try_wait

    def revoke_failed_onboard(self, index_meta: KVIndexMeta, lookup_result: KVLookupResult) -> None:
        """After a failed onboard the request is recomputed from token 0: drop the pages that were reserved for the
        host prefix so the device range no longer claims tokens that never arrived."""
        need = self._onboard_need(lookup_result)
        self.gpu.revoke_onboard_pages(index_meta.user_ids, torch.zeros_like(need), need)

    def offload_launch(self, index_meta: KVIndexMeta, kvcache_metadata: Optional[KVCacheMetadata] = None) -> Optional[HostKVTaskHandle]:
        if self.host is None:
            return None
        if self._pending_offload is not None:
            self.offload_try_wait()
        cands = index_meta.user_ids
        if self.offload_mode != KVCacheOffloadMode.EAGER.value:
            cands = self.gpu.check_for_offload(index_meta.user_ids)
        if cands.numel() == 0:
            return None
        _hs, hl = self.host.lookup_kvcache(KVIndexMeta(cands, torch.zeros(cands.numel(), dtype=torch.int32)))
        uids, starts, pages = self.gpu.acquire_offload_pages(cands, hl.int(), False)
        if uids.numel() == 0:
            return None
        h = self.host.offload_kvcache_launch(uids, starts, pages, index_meta, kvcache_metadata)
        lengths = torch.tensor(h.metadata["lengths"], dtype=torch.int32)
        self._pending_offload = (h, uids, starts, lengths)
        return h

    def offload_try_wait(self) -> Optional[HostKVWaitResult]:
        if self._pending_offload is None:
            return None
        h, uids, starts, lengths = self._pending_offload
        self._pending_offload = None
        res = self.host.offload_kvcache_wait(h)
        done = self.host.finish_task(h)
        self.gpu.release_offload_pages(uids, starts, lengths, done)       # locks are released on every path
        if res.status == HostKVTaskStatus.READY:
            self.stats["offloaded_tokens"] += int(sum(l for l, d in zip(lengths.tolist(), done) if d))
        elif res.status == HostKVTaskStatus.TIMEOUT:
            self.stats["offload_timeouts"] += 1
            self._fail("offload", res)
        elif res.status == HostKVTaskStatus.FAILED:
            self.stats["offload_failures"] += 1
            self._fail("offload", res)
        return res

    def evict(self, user_ids: torch.Tensor, for_npu: bool = True, for_host: bool = True) -> None:
        if for_npu:
            self.gpu.evict(user_ids)
        if for_host and self.host is not None:
            self.host.evict(user_ids)

    def evict_all(self, for_npu: bool = True, for_host: bool = True) -> None:
        if for_npu:
            self.gpu.evict_all()
        if for_host and self.host is not None:
            self.host.evict_all()

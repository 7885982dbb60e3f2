"""Operator-level calls of the dynamic-embedding stack under the names and argument lists of the reference's native
module (``dynamic_emb_extensions``, bound in ``dynamic_emb/csrc/dynamic_emb_op.cpp:2739-3036``).

The reference's Python layers, its operator unit tests and user code that drives a table by hand all go through that
module: a type-erased ``DynamicEmbTable`` plus free functions that take the table, an element count ``n`` and
caller-allocated output tensors.  Here the same calls sit on ``HKVTable`` (the CUDA hash table of ``csrc/cuda/hkv.cu``)
or, without a GPU, on ``HostDynamicTable``; the batched modules of this package call the tables directly and do not
pass through this file.

Conventions kept from the reference: outputs are written in place into the caller's tensors; ``n`` limits a call to the
first ``n`` keys; ``score`` of the insert-type calls is one integer for the whole call and is required for LFU and
customised eviction; ``values`` rows are ``[embedding | optimizer state]`` and a narrower ``values`` tensor receives
the leading columns; ``export_batch_matched`` / ``count_matched`` keep entries whose score is >= the threshold
(``csrc/hkv_variable.cpp:131-152``).
"""
from __future__ import annotations

import enum
from typing import Optional, Tuple

import numpy as np
import torch

from ..ops import by_address as BA
from ..ops import sparse_ops as S
from .dynamicemb_config import DynamicEmbCheckMode as SafeCheckMode
from .dynamicemb_config import DynamicEmbDataType
from .hkv import EvictStrategy as _Evict
from .hkv import HKVTable, HostDynamicTable, InitMode
from .hkv import InitializerArgs as _NativeInit
from .hkv import OptimizerType as _Opt
from .hkv import opt_state_dim
from .optimizers import OptimizerArgs, _apply

__all__ = ["InitializerArgs", "DynamicEmbTable", "DynamicEmbDataType", "EvictStrategy", "SafeCheckMode", "OptimizerType",
           "CurandStateContext", "find", "find_or_insert", "find_pointers", "find_pointers_with_scores",
           "find_or_insert_pointers", "find_and_initialize", "insert_and_evict", "assign", "accum_or_assign", "erase",
           "clear", "reserve", "dyn_emb_rows", "dyn_emb_cols", "dyn_emb_is_pure_hbm_mode", "export_batch_matched",
           "count_matched", "device_timestamp", "load_from_pointer", "load_from_pointer_hybrid", "gather_embedding",
           "reduce_grads", "unique_op", "segmented_unique_op", "select", "select_index", "get_table_range_op",
           "get_new_length_and_offsets_op", "dedup_input_indices_op", "lookup_forward", "lookup_forward_hybrid",
           "lookup_backward", "normal_init", "uniform_init", "truncated_normal_init", "const_init", "debug_init"]


class EvictStrategy(enum.IntEnum):
    kLru = int(_Evict.LRU)
    kLfu = int(_Evict.LFU)
    kEpochLru = int(_Evict.EPOCH_LRU)
    kEpochLfu = int(_Evict.EPOCH_LFU)
    kCustomized = int(_Evict.CUSTOMIZED)


class OptimizerType(enum.IntEnum):
    Null = 0
    SGD = 1
    Adam = 2
    AdamW = 3
    AdaGrad = 4
    RowWiseAdaGrad = 5


_TO_NATIVE_OPT = {OptimizerType.Null: _Opt.SGD, OptimizerType.SGD: _Opt.SGD, OptimizerType.Adam: _Opt.ADAM, OptimizerType.AdamW: _Opt.ADAM,
                  OptimizerType.AdaGrad: _Opt.ADAGRAD, OptimizerType.RowWiseAdaGrad: _Opt.ROWWISE_ADAGRAD}
_MODES = {"uniform": InitMode.UNIFORM, "normal": InitMode.NORMAL, "truncated_normal": InitMode.TRUNCATED_NORMAL,
          "constant": InitMode.CONSTANT, "debug": InitMode.DEBUG}


class InitializerArgs:
    """``InitializerArgs(mode, mean, std_dev, lower, upper, value)`` with ``mode`` a string; compares by value and pickles."""

    def __init__(self, mode: str = "uniform", mean: float = 0.0, std_dev: float = 1.0, lower: float = 0.0, upper: float = 1.0,
                 value: float = 0.0) -> None:
        m = str(mode).lower()
        if m not in _MODES:
            raise ValueError("unknown initializer mode %r (one of %s)" % (mode, sorted(_MODES)))
        self.mode, self.mean, self.std_dev, self.lower, self.upper, self.value = m, float(mean), float(std_dev), float(lower), float(upper), float(value)

    def _tuple(self):
        return (self.mode, self.mean, self.std_dev, self.lower, self.upper, self.value)

    def __eq__(self, other) -> bool:
        return isinstance(other, InitializerArgs) and self._tuple() == other._tuple()

    def __hash__(self) -> int:
        return hash(self._tuple())

    def __reduce__(self):
        return (InitializerArgs, self._tuple())

    def to_native(self, seed: int = 0, state_init: float = 0.0) -> _NativeInit:
        return _NativeInit(mode=_MODES[self.mode], lower=self.lower, upper=self.upper, mean=self.mean, std_dev=self.std_dev,
                           value=self.value, seed=seed, state_init=state_init)


class CurandStateContext:
    """Random state handed to the initializer calls (a seeded ``torch.Generator`` per device, created on first use)."""

    def __init__(self, seed: int = 0) -> None:
        self.seed = int(seed)
        self._gens = {}

    def generator(self, device: torch.device) -> torch.Generator:
        g = self._gens.get(device)
        if g is None:
            g = torch.Generator(device=device)
            g.manual_seed(self.seed)
            self._gens[device] = g
        return g


def _next_pow2(x: int) -> int:
    p = 1
    while p < x:
        p <<= 1
    return p


class DynamicEmbTable:
    """The type-erased table handle.  Keys are 64-bit, values fp32 rows of ``dim`` embedding columns followed by the
    optimizer's state columns; ``device_id < 0`` means the current CUDA device, or the host table without CUDA.  Capacities
    are rounded up to powers of two, as the reference's constructor does (``dynamic_emb_op.cpp:2766-2782``);
    ``max_hbm_for_vectors`` bytes of rows stay in device memory and the rest in mapped host memory (0: all on the device).
    Arguments that tune the reference's kernels (block sizes, constant memory, bucket allocation) are accepted and unused."""

    def __init__(self, key_type: DynamicEmbDataType, value_type: DynamicEmbDataType, evict_type: EvictStrategy, dim: int = 128,
                 init_capaity: int = 1024, max_capaity: int = 2048, max_hbm_for_vectors: int = 0, max_bucket_size: int = 128,
                 max_load_factor: float = 0.5, block_size: int = 128, io_block_size: int = 1024, device_id: int = -1,
                 io_by_cpu: bool = False, use_constant_memory: bool = False, reserved_key_start_bit: int = 0,
                 num_of_buckets_per_alloc: int = 1, initializer_args: Optional[InitializerArgs] = None,
                 safe_check_mode: int = int(SafeCheckMode.IGNORE), optimizer_type: int = int(OptimizerType.Null)) -> None:
        if key_type not in (DynamicEmbDataType.Int64, DynamicEmbDataType.UInt64):
            raise ValueError("keys are 64-bit integers (Int64 / UInt64), got %s" % key_type)
        if value_type != DynamicEmbDataType.Float32:
            raise ValueError("table rows are stored as Float32 (outputs may be narrower), got %s" % value_type)
        if max_bucket_size != 128:
            raise ValueError("buckets hold 128 slots")
        self._key_type, self._value_type = key_type, value_type
        self._evict = EvictStrategy(int(evict_type))
        self._opt = OptimizerType(int(optimizer_type))
        self._init_args = initializer_args or InitializerArgs()
        self._safe_check_mode = SafeCheckMode(int(safe_check_mode))
        self._initial_optstate = 0.0
        cap, max_cap = _next_pow2(int(init_capaity)), _next_pow2(int(max_capaity))
        native = dict(optimizer=_TO_NATIVE_OPT[self._opt], evict_strategy=_Evict(int(self._evict)), init=self._init_args.to_native())
        if torch.cuda.is_available():
            dev = torch.device("cuda", device_id if device_id >= 0 else torch.cuda.current_device())
            row_bytes = 4 * (dim + opt_state_dim(native["optimizer"], dim))
            hbm_rows = max(128, int(max_hbm_for_vectors) // row_bytes) if max_hbm_for_vectors else None
            self.table = HKVTable(dim, cap, dev, max_capacity=max(cap, max_cap), max_load_factor=max_load_factor, hbm_rows=hbm_rows, **native)
        else:
            self.table = HostDynamicTable(dim, max(cap, max_cap), **native)

    # -- queries of the reference's handle ---------------------------------------------------------------------------
    def get_key_type(self) -> DynamicEmbDataType:
        return self._key_type

    def get_value_type(self) -> DynamicEmbDataType:
        return self._value_type

    def get_evict_strategy(self) -> EvictStrategy:
        return self._evict

    evict_strategy = get_evict_strategy

    def get_max_capacity(self) -> int:
        return int(getattr(self.table, "max_capacity", self.table.capacity))

    def get_initializer_args(self) -> InitializerArgs:
        return self._init_args

    def optstate_dim(self) -> int:
        return int(self.table.state_dim)

    def get_emb_cols(self) -> int:
        return int(self.table.dim)

    def set_initial_optstate(self, value: float) -> None:
        self._initial_optstate = float(value)
        self.table.init.state_init = float(value)

    def get_initial_optstate(self) -> float:
        return self._initial_optstate

    # -- whole-row IO (checkpoint load / export) ---------------------------------------------------------------------
    def load(self, n: int, keys: torch.Tensor, values: torch.Tensor, score: Optional[torch.Tensor] = None, unique_key: bool = True,
             ignore_evict_strategy: bool = False) -> None:
        """Insert or overwrite ``n`` full rows (per-key ``score`` tensor optional)."""
        if n:
            self.table.insert_and_evict(keys[:n].contiguous(), values[:n].float(), None if score is None else score[:n].contiguous())

    update = load

    def export_batch(self, n: int, offset: int, d_counter: torch.Tensor, keys: torch.Tensor, values: torch.Tensor,
                     score: Optional[torch.Tensor] = None) -> None:
        k, s, rows, _ = self.table.export_batch(int(offset), int(n))
        m = int(k.numel())
        d_counter.reshape(-1)[0] = m
        keys[:m] = k.to(keys.dtype)
        values.view(-1, self.table.row_dim)[:m] = rows.to(values.dtype)
        if score is not None:
            score[:m] = s.to(score.dtype)


def _t(table):
    return getattr(table, "table", table)


def _score_tensor(t, n: int, score) -> Optional[torch.Tensor]:
    if score is None:
        return None
    if isinstance(score, torch.Tensor):
        return score[:n].to(device=t.device, dtype=torch.int64).contiguous()
    return torch.full((n,), int(score), dtype=torch.int64, device=t.device)


def _need_score(t, score, what: str) -> None:
    if score is None and t.evict_strategy in (_Evict.CUSTOMIZED, _Evict.LFU):
        raise ValueError("Must specify the score when evict strategy is customized or LFU. (%s)" % what)


def _write_rows(t, slots: torch.Tensor, ok: torch.Tensor, values: torch.Tensor, n: int) -> None:
    cols = min(int(values.shape[1]), t.row_dim)
    rows = t.gather(slots, 0, cols)
    dst = values[:n]
    dst[:, :cols] = torch.where(ok[:, None], rows.to(dst.dtype), dst[:, :cols])


def _pointers(t, slots: torch.Tensor) -> torch.Tensor:
    """Addresses of the value rows: device (or mapped host) addresses for the CUDA table, the addresses of the host rows of
    the dictionary-backed table (they stay valid while the key is resident)."""
    if isinstance(t, HKVTable):
        return t._pointers(slots)
    return torch.tensor([t.rows[k].ctypes.data if k in t.rows else 0 for k in slots.tolist()], dtype=torch.int64)


# ----------------------------------------------------------------------------------------------------------------------
# table calls
# ----------------------------------------------------------------------------------------------------------------------
def find(table, n: int, keys: torch.Tensor, values: torch.Tensor, founds: torch.Tensor, score: Optional[torch.Tensor] = None) -> None:
    """Rows of the resident keys go to ``values`` (rows of missing keys are left as they are), ``founds`` gets the mask."""
    if not n:
        return
    t = _t(table)
    sc = _score_tensor(t, n, score)
    slots, ok = t.find(keys[:n].contiguous(), update_score=sc is not None, scores=sc)
    founds[:n] = ok
    _write_rows(t, slots, ok, values, n)


def _unique_keys(keys: torch.Tensor, unique_key: bool) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    if unique_key:
        return keys.contiguous(), None
    u, inv = torch.unique(keys, return_inverse=True)
    return u.contiguous(), inv


def find_or_insert(table, n: int, keys: torch.Tensor, values: torch.Tensor, score: Optional[int] = None, unique_key: bool = True,
                   ignore_evict_strategy: bool = False) -> None:
    """Missing keys are inserted with the table's initializer; every key's row goes to ``values`` (a key that found no
    room reads as zeros)."""
    if not n:
        return
    t = _t(table)
    _need_score(t, score, "find_or_insert")
    k, inv = _unique_keys(keys[:n], unique_key)
    slots, _status, _ = t.find_or_insert(k, _score_tensor(t, k.numel(), score))
    if inv is not None:
        slots = slots[inv]
    _write_rows(t, slots, torch.ones(n, dtype=torch.bool, device=slots.device), values, n)


def find_pointers(table, n: int, keys: torch.Tensor, values: torch.Tensor, founds: torch.Tensor, score: Optional[int] = None) -> None:
    """``values`` (int64) receives the address of every resident key's row, 0 for the others."""
    if not n:
        return
    t = _t(table)
    sc = _score_tensor(t, n, score)
    slots, ok = t.find(keys[:n].contiguous(), update_score=sc is not None, scores=sc)
    founds[:n] = ok
    values[:n] = _pointers(t, slots).to(values.dtype)


find_pointers_with_scores = find_pointers          # the scores variant differs in taking one score per key (a tensor)


def find_or_insert_pointers(table, n: int, keys: torch.Tensor, values: torch.Tensor, founds: torch.Tensor, score: Optional[int] = None,
                            unique_key: bool = True, ignore_evict_strategy: bool = False) -> None:
    """Like ``find_or_insert``, handing out row addresses; ``founds`` tells which keys were resident before the call."""
    if not n:
        return
    t = _t(table)
    _need_score(t, score, "find_or_insert_pointers")
    k, inv = _unique_keys(keys[:n], unique_key)
    _s, before = t.find(k)
    slots, _status, _ = t.find_or_insert(k, _score_tensor(t, k.numel(), score))
    if inv is not None:
        slots, before = slots[inv], before[inv]
    founds[:n] = before
    values[:n] = _pointers(t, slots).to(values.dtype)


def _fresh_rows(args: InitializerArgs, keys: torch.Tensor, cols: int, dtype, device) -> torch.Tensor:
    n = keys.numel()
    if args.mode == "constant":
        return torch.full((n, cols), args.value, dtype=dtype, device=device)
    if args.mode == "debug":
        return (keys % 100000).to(dtype)[:, None].expand(n, cols).contiguous()
    g = torch.Generator(device=device)
    g.manual_seed(0)
    if args.mode == "uniform":
        return (torch.rand(n, cols, generator=g, device=device) * (args.upper - args.lower) + args.lower).to(dtype)
    z = torch.randn(n, cols, generator=g, device=device)
    if args.mode == "truncated_normal":
        z = z.clamp(-2.0, 2.0)
    return (z * args.std_dev + args.mean).to(dtype)


def find_and_initialize(table, n: int, keys: torch.Tensor, value_ptrs: torch.Tensor, values: torch.Tensor, founds: torch.Tensor,
                        initializer_args: Optional[InitializerArgs] = None) -> None:
    """Evaluation lookup: resident rows are copied, missing keys read as freshly initialised rows (the table's own
    initializer unless one is given) and nothing is inserted."""
    if not n:
        return
    t = _t(table)
    k = keys[:n].contiguous()
    slots, ok = t.find(k)
    founds[:n] = ok
    value_ptrs[:n] = _pointers(t, slots).to(value_ptrs.dtype)
    args = initializer_args or getattr(table, "_init_args", None) or InitializerArgs("constant", value=0.0)
    cols = min(int(values.shape[1]), t.dim)
    values[:n, :cols] = _fresh_rows(args, k, cols, values.dtype, values.device)
    _write_rows(t, slots, ok, values, n)


def insert_and_evict(table, n: int, keys: torch.Tensor, values: torch.Tensor, score: Optional[int], evicted_keys: torch.Tensor,
                     evicted_values: torch.Tensor, evicted_score: torch.Tensor, d_evicted_counter: torch.Tensor, unique_key: bool = True,
                     ignore_evict_strategy: bool = False) -> None:
    """Insert or overwrite full rows; entries that had to leave are written to the ``evicted_*`` tensors and counted."""
    d_evicted_counter.reshape(-1)[0] = 0
    if not n:
        return
    t = _t(table)
    _need_score(t, score, "insert_and_evict")
    _slots, _status, ev = t.insert_and_evict(keys[:n].contiguous(), values[:n].float(), _score_tensor(t, n, score))
    m = int(ev[3].reshape(-1)[0]) if ev is not None else 0
    d_evicted_counter.reshape(-1)[0] = m
    if m:
        evicted_keys[:m] = ev[0][:m].to(evicted_keys.dtype)
        evicted_score[:m] = ev[1][:m].to(evicted_score.dtype)
        evicted_values.view(-1, t.row_dim)[:m] = ev[2][:m].to(evicted_values.dtype)


def assign(table, n: int, keys: torch.Tensor, values: torch.Tensor, score: Optional[torch.Tensor] = None, unique_key: bool = True) -> None:
    """Overwrite the leading columns of rows that are resident; other keys are ignored."""
    if not n:
        return
    t = _t(table)
    sc = _score_tensor(t, n, score)
    slots, _ok = t.find(keys[:n].contiguous(), update_score=sc is not None, scores=sc)
    t.scatter(slots, values[:n], 0, int(values.shape[1]))


def accum_or_assign(table, n: int, keys: torch.Tensor, value_or_deltas: torch.Tensor, accum_or_assigns: torch.Tensor,
                    score: Optional[torch.Tensor] = None, ignore_evict_strategy: bool = False) -> None:
    """Rows flagged true are added to when resident; rows flagged false are inserted or overwritten."""
    if not n:
        return
    t = _t(table)
    k, v, acc = keys[:n], value_or_deltas[:n], accum_or_assigns[:n].bool()
    sc = _score_tensor(t, n, score)
    if bool(acc.any()):
        slots, _ = t.find(k[acc].contiguous())
        t.scatter(slots, v[acc], 0, int(v.shape[1]), accumulate=True)
    if bool((~acc).any()):
        t.insert_and_evict(k[~acc].contiguous(), v[~acc].float(), None if sc is None else sc[~acc].contiguous())


def erase(table, n: int, keys: torch.Tensor) -> None:
    if n:
        _t(table).erase(keys[:n].contiguous())


def clear(table) -> None:
    _t(table).clear()


def reserve(table, new_capacity: int) -> None:
    _t(table).reserve(int(new_capacity))


def dyn_emb_rows(table) -> int:
    return int(_t(table).size())


def dyn_emb_cols(table) -> int:
    return int(_t(table).dim)


def dyn_emb_is_pure_hbm_mode(table) -> bool:
    return getattr(_t(table), "values_host", None) is None


def export_batch_matched(table, threshold: int, n: int, offset: int, num_matched: torch.Tensor, keys: torch.Tensor, values: torch.Tensor) -> None:
    t = _t(table)
    k, _s, rows, _ = t.export_batch(int(offset), int(n), min_score=int(threshold))
    m = int(k.numel())
    num_matched.reshape(-1)[0] = m
    keys[:m] = k.to(keys.dtype)
    values.view(-1, t.row_dim)[:m] = rows.to(values.dtype)


def count_matched(table, threshold: int, num_matched: torch.Tensor) -> None:
    num_matched.reshape(-1)[0] = _t(table).count_matched(int(threshold))


def device_timestamp(table=None) -> int:
    """The device's clock (the LRU score source) on CUDA, the host's monotonic nanosecond clock otherwise."""
    if table is not None and isinstance(_t(table), HKVTable):
        return _t(table).device_timestamp()
    if torch.cuda.is_available():
        from ..ops import _lib

        dev = torch.device("cuda", torch.cuda.current_device())
        out = torch.zeros(1, dtype=torch.int64, device=dev)
        _lib.check(_lib.lib().rb_device_timestamp(out.data_ptr(), _lib.stream_ptr(dev)), "rb_device_timestamp")
        return int(out.item())
    import time

    return time.monotonic_ns()


# ----------------------------------------------------------------------------------------------------------------------
# rows by address, gathers, gradient reduction
# ----------------------------------------------------------------------------------------------------------------------
def _resolve_region(region, pointers: torch.Tensor):
    """Row IO by address is bounds-checked in this package, so the caller names the memory the addresses may point into:
    the rows' tensor, its ``(first, one-past-last)`` byte addresses, or the table that handed the addresses out."""
    if region is None:
        raise ValueError("calls on row addresses need region= the rows' tensor, its (lo, hi) addresses or the table (addresses are checked)")
    t = _t(region)
    if isinstance(t, HostDynamicTable):
        known = {r.ctypes.data for r in t.rows.values()}
        stray = [p for p in pointers.tolist() if p and p not in known]
        if stray:
            raise IndexError("address %#x is not a row of the table" % stray[0])
        return (1, 1 << 62)
    if isinstance(t, HKVTable):
        if t.values_host is not None:
            raise ValueError("the table keeps rows in two memories; pass the (lo, hi) addresses of the one the pointers are in")
        return t.values_hbm
    return region


def load_from_pointer(pointers: torch.Tensor, dst: torch.Tensor, region=None) -> torch.Tensor:
    """``dst[i] = row at pointers[i]`` (zeros for address 0); ``region`` as in ``_resolve_region``."""
    rows = BA.embedding_lookup_by_address(pointers, int(dst.shape[1]), _resolve_region(region, pointers))
    dst.copy_(rows.to(dst.dtype))
    return dst


load_from_pointer_hybrid = load_from_pointer


def gather_embedding(inputs: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    from ..ops import embedding_ops as E

    return E.gather_rows(inputs.contiguous(), indices.to(torch.int64).contiguous())


def reduce_grads(grad: torch.Tensor, unique: torch.Tensor, inverse: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``out[inverse[k]] += grad[k]`` over ``len(unique)`` rows (fp32 accumulation) -> (reduced gradients, unique)."""
    out = torch.zeros(unique.shape[0], grad.shape[1], dtype=torch.float32, device=grad.device)
    out.index_add_(0, inverse.to(torch.int64), grad.float())
    return out.to(grad.dtype), unique


# ----------------------------------------------------------------------------------------------------------------------
# id preprocessing
# ----------------------------------------------------------------------------------------------------------------------
def unique_op(key: torch.Tensor):
    """-> (unique keys, inverse, counts)."""
    return S.unique(key, with_counts=True)


def segmented_unique_op(keys: torch.Tensor, segmentRange: torch.Tensor):
    """Per-segment unique -> (unique buffer, inverse, per-segment unique offsets, counts)."""
    return S.segmented_unique(keys, segmentRange, with_counts=True)


def select(flags: torch.Tensor, inputs: torch.Tensor, outputs: torch.Tensor, num_selected: torch.Tensor) -> None:
    buf, cnt = S.select(inputs, flags)
    outputs[: buf.numel()] = buf.to(outputs.dtype)
    num_selected.reshape(-1)[0] = cnt.reshape(-1)[0].to(num_selected.dtype)


def select_index(flags: torch.Tensor, output_indices: torch.Tensor, num_selected: torch.Tensor) -> None:
    buf, cnt = S.select_index(flags)
    output_indices[: buf.numel()] = buf.to(output_indices.dtype)
    num_selected.reshape(-1)[0] = cnt.reshape(-1)[0].to(num_selected.dtype)


def _batch_of(offsets: torch.Tensor, featureOffsets) -> Tuple[list, int]:
    fo = [int(x) for x in (featureOffsets.tolist() if isinstance(featureOffsets, torch.Tensor) else featureOffsets)]
    if fo[-1] <= 0 or (offsets.numel() - 1) % fo[-1]:
        raise ValueError("offsets of %d bags do not split into %d features" % (offsets.numel() - 1, fo[-1]))
    return fo, (offsets.numel() - 1) // fo[-1]


def get_table_range_op(offsets: torch.Tensor, featureOffsets) -> torch.Tensor:
    fo, B = _batch_of(offsets, featureOffsets)
    return S.get_table_range(offsets, fo, B)


def get_new_length_and_offsets_op(d_unique_offsets: torch.Tensor, d_table_offsets_in_feature, new_offsets: torch.Tensor,
                                  new_lengths: torch.Tensor, local_batch_size: int) -> None:
    fo = [int(x) for x in (d_table_offsets_in_feature.tolist() if isinstance(d_table_offsets_in_feature, torch.Tensor) else d_table_offsets_in_feature)]
    lengths, offsets = S.get_new_length_and_offsets(d_unique_offsets, fo, int(local_batch_size))
    new_lengths[: lengths.numel()] = lengths.to(new_lengths.dtype)
    new_offsets[: offsets.numel()] = offsets.to(new_offsets.dtype)


def dedup_input_indices_op(indices: torch.Tensor, offsets: torch.Tensor, d_table_offsets_in_feature, table_num: int, local_batch_size: int,
                           reverse_idx: torch.Tensor, d_unique_nums: torch.Tensor, d_unique_offsets: torch.Tensor, unique_idx: torch.Tensor,
                           new_offsets: torch.Tensor, new_lengths: torch.Tensor) -> None:
    """Per-table de-duplication of a batch's ids into the caller's tensors: distinct ids (``unique_idx``), the map from
    every id to its distinct entry (``reverse_idx``), distinct counts and offsets per table, and the lengths / offsets of
    the de-duplicated batch."""
    fo = [int(x) for x in (d_table_offsets_in_feature.tolist() if isinstance(d_table_offsets_in_feature, torch.Tensor) else d_table_offsets_in_feature)]
    B = int(local_batch_size)
    ranges = S.get_table_range(offsets, fo, B)
    uniq, inv, uoffs, _c = S.segmented_unique(indices, ranges)
    total = int(uoffs[-1])
    unique_idx[:total] = uniq[:total].to(unique_idx.dtype)
    reverse_idx[: inv.numel()] = inv.to(reverse_idx.dtype)
    d_unique_offsets[: uoffs.numel()] = uoffs.to(d_unique_offsets.dtype)
    d_unique_nums[: int(table_num)] = (uoffs[1:] - uoffs[:-1])[: int(table_num)].to(d_unique_nums.dtype)
    lengths, noffs = S.get_new_length_and_offsets(uoffs, fo, B)
    new_lengths[: lengths.numel()] = lengths.to(new_lengths.dtype)
    new_offsets[: noffs.numel()] = noffs.to(new_offsets.dtype)


# ----------------------------------------------------------------------------------------------------------------------
# pooled lookup over distinct rows
# ----------------------------------------------------------------------------------------------------------------------
def lookup_forward(src: torch.Tensor, dst: torch.Tensor, offset: torch.Tensor, inverse: torch.Tensor, combiner: int, total_dims: int,
                   accum_dims: int, ev_size: int, num_vec: int, batch_size: int) -> None:
    """Pool the distinct rows ``src`` back into bags: bag ``b`` of feature ``f`` (``offset`` over ``f * batch_size + b``) is the
    sum (``combiner`` 0) or mean (1) of ``src[inverse[j]]`` and lands in ``dst[b, accum_dims + f * ev_size : ... + ev_size]``
    of a ``[batch_size, total_dims]`` output."""
    bags = offset.numel() - 1
    lens = (offset[1:] - offset[:-1]).to(torch.int64)
    bag_of = torch.repeat_interleave(torch.arange(bags, device=src.device), lens, output_size=int(num_vec))
    pooled = torch.zeros(bags, ev_size, dtype=torch.float32, device=src.device)
    pooled.index_add_(0, bag_of, src[inverse[: int(num_vec)].to(torch.int64), :ev_size].float())
    if int(combiner) == 1:
        pooled = pooled / lens.clamp(min=1)[:, None]
    F = bags // int(batch_size)
    out = dst.view(int(batch_size), int(total_dims))
    out[:, accum_dims:accum_dims + F * ev_size] = pooled.view(F, int(batch_size), ev_size).permute(1, 0, 2).reshape(int(batch_size), F * ev_size).to(dst.dtype)


lookup_forward_hybrid = lookup_forward


def lookup_backward(grad: torch.Tensor, unique_buffer: torch.Tensor, unique_indices: torch.Tensor, inverse_indices: torch.Tensor,
                    biased_offsets: torch.Tensor, dim: int, tables_num: int, batch_size: int, num_feature: int, num_key: int,
                    combiner: int) -> None:
    """Gradient of the pooled lookup per distinct row: ``unique_buffer[inverse[j]] += grad[b, f * dim : (f + 1) * dim]`` for
    every id ``j`` of bag ``(f, b)`` (divided by the bag length for the mean)."""
    bags = int(num_feature) * int(batch_size)
    lens = (biased_offsets[1:bags + 1] - biased_offsets[:bags]).to(torch.int64)
    bag_of = torch.repeat_interleave(torch.arange(bags, device=grad.device), lens, output_size=int(num_key))
    g = grad.view(int(batch_size), int(num_feature), int(dim)).permute(1, 0, 2).reshape(bags, int(dim)).float()
    if int(combiner) == 1:
        g = g / lens.clamp(min=1)[:, None]
    acc = torch.zeros(unique_buffer.shape[0], int(dim), dtype=torch.float32, device=grad.device)
    acc.index_add_(0, inverse_indices[: int(num_key)].to(torch.int64), g[bag_of])
    unique_buffer[:, : int(dim)] = acc.to(unique_buffer.dtype)


# ----------------------------------------------------------------------------------------------------------------------
# optimizers: on gathered rows (fused), through row addresses (with_pointer), through the table (with_table)
# ----------------------------------------------------------------------------------------------------------------------
def _fused(kind: _Opt, grads: torch.Tensor, values: torch.Tensor, step: int = 1, **kw) -> None:
    with torch.no_grad():
        _apply(kind, grads, values, OptimizerArgs(**kw), step)


def dynamic_emb_sgd_fused(grads, values, lr) -> None:
    _fused(_Opt.SGD, grads, values, learning_rate=lr)


def dynamic_emb_adagrad_fused(grads, values, lr, eps) -> None:
    _fused(_Opt.ADAGRAD, grads, values, learning_rate=lr, eps=eps)


def dynamic_emb_rowwise_adagrad_fused(grads, values, lr, eps) -> None:
    _fused(_Opt.ROWWISE_ADAGRAD, grads, values, learning_rate=lr, eps=eps)


def dynamic_emb_adamW_fused(grads, values, lr, beta1, beta2, eps, weight_decay, iter_num) -> None:
    _fused(_Opt.ADAM, grads, values, int(iter_num), learning_rate=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay)


dynamic_emb_sgd_fused_hybrid = dynamic_emb_sgd_fused
dynamic_emb_adagrad_fused_hybrid = dynamic_emb_adagrad_fused
dynamic_emb_rowwise_adagrad_fused_hybrid = dynamic_emb_rowwise_adagrad_fused
dynamic_emb_adamW_fused_hybrid = dynamic_emb_adamW_fused


def _with_table(kind: _Opt, ht, n: int, indices: torch.Tensor, grads: torch.Tensor, step: int = 1, **kw) -> None:
    """Keys -> resident rows -> formula -> rows written back; keys that are not resident are skipped."""
    if not n:
        return
    t = _t(ht)
    if t.optimizer != kind:
        raise ValueError("the table keeps %s state, the call is for %s" % (t.optimizer.name, kind.name))
    slots, ok = t.find(indices[:n].contiguous())
    rows = t.gather(slots, 0, t.row_dim)[ok]
    _fused(kind, grads[:n][ok], rows, step, **kw)
    t.scatter(slots[ok], rows, 0, t.row_dim)


def dynamic_emb_sgd_with_table(ht, n, indices, grads, lr, weight_type=None) -> None:
    _with_table(_Opt.SGD, ht, n, indices, grads, learning_rate=lr)


def dynamic_emb_adagrad_with_table(ht, n, indices, grads, lr, eps, weightType=None) -> None:
    _with_table(_Opt.ADAGRAD, ht, n, indices, grads, learning_rate=lr, eps=eps)


def dynamic_emb_rowwise_adagrad_with_table(ht, n, indices, grads, lr, eps, weightType=None) -> None:
    _with_table(_Opt.ROWWISE_ADAGRAD, ht, n, indices, grads, learning_rate=lr, eps=eps)


def dynamic_emb_adamW_with_table(ht, n, indices, grads, lr, beta1, beta2, eps, weight_decay, iter_num, weight_type=None) -> None:
    _with_table(_Opt.ADAM, ht, n, indices, grads, int(iter_num), learning_rate=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay)


def _with_pointer(kind: _Opt, grads: torch.Tensor, val_pointers: torch.Tensor, state_dim: int, region, step: int = 1, **kw) -> None:
    region = _resolve_region(region, val_pointers)
    cols = int(grads.shape[1]) + opt_state_dim(kind, int(grads.shape[1]))
    rows = BA.embedding_lookup_by_address(val_pointers, cols, region)
    _fused(kind, grads, rows, step, **kw)
    BA.embedding_update_by_address(val_pointers, rows, 1, region)


def dynamic_emb_sgd_with_pointer(grads, val_pointers, val_type, lr, region=None) -> None:
    _with_pointer(_Opt.SGD, grads, val_pointers, 0, region, learning_rate=lr)


def dynamic_emb_adagrad_with_pointer(grads, valPointers, valType, stateDim, lr, eps, region=None) -> None:
    _with_pointer(_Opt.ADAGRAD, grads, valPointers, stateDim, region, learning_rate=lr, eps=eps)


def dynamic_emb_rowwise_adagrad_with_pointer(grads, valPointers, valType, stateDim, lr, eps, region=None) -> None:
    _with_pointer(_Opt.ROWWISE_ADAGRAD, grads, valPointers, stateDim, region, learning_rate=lr, eps=eps)


def dynamic_emb_adamW_with_pointer(grads, val_pointers, val_type, state_dim, lr, beta1, beta2, eps, weight_decay, iter_num, region=None) -> None:
    _with_pointer(_Opt.ADAM, grads, val_pointers, state_dim, region, int(iter_num), learning_rate=lr, beta1=beta1, beta2=beta2, eps=eps,
                  weight_decay=weight_decay)


def dynamic_emb_Adam_with_pointer(grads, val_pointers, val_type, state_dim, lr, beta1, beta2, eps, weight_decay, iter_num, region=None) -> None:
    """Adam whose ``weight_decay`` enters as decoupled decay, the one form this stack implements."""
    dynamic_emb_adamW_with_pointer(grads, val_pointers, val_type, state_dim, lr, beta1, beta2, eps, weight_decay, iter_num, region)


dynamic_emb_sgd_with_pointer_hybrid = dynamic_emb_sgd_with_pointer
dynamic_emb_adagrad_with_pointer_hybrid = dynamic_emb_adagrad_with_pointer
dynamic_emb_rowwise_adagrad_with_pointer_hybrid = dynamic_emb_rowwise_adagrad_with_pointer
dynamic_emb_adamW_with_pointer_hybrid = dynamic_emb_adamW_with_pointer

__all__ += [n for n in list(globals()) if n.startswith("dynamic_emb_")]


# ----------------------------------------------------------------------------------------------------------------------
# initializers on selected rows of a buffer
# ----------------------------------------------------------------------------------------------------------------------
def _rows_of(buffer: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    if buffer.dim() != 2:
        raise ValueError("buffer must be [rows, dim]")
    return indices.to(device=buffer.device, dtype=torch.int64)


def normal_init(buffer: torch.Tensor, indices: torch.Tensor, curand_state_context: CurandStateContext, mean: float, std_dev: float) -> None:
    idx = _rows_of(buffer, indices)
    z = torch.randn(idx.numel(), buffer.shape[1], generator=curand_state_context.generator(buffer.device), device=buffer.device)
    buffer[idx] = (z * std_dev + mean).to(buffer.dtype)


def truncated_normal_init(buffer: torch.Tensor, indices: torch.Tensor, curand_state_context: CurandStateContext, mean: float, std_dev: float,
                          lower: float, upper: float) -> None:
    """Normal samples redrawn until they fall inside ``[lower, upper]`` (a bounded number of rounds, then clamped)."""
    idx = _rows_of(buffer, indices)
    g = curand_state_context.generator(buffer.device)
    z = torch.randn(idx.numel(), buffer.shape[1], generator=g, device=buffer.device) * std_dev + mean
    for _ in range(32):
        bad = (z < lower) | (z > upper)
        if not bool(bad.any()):
            break
        z = torch.where(bad, torch.randn(z.shape, generator=g, device=buffer.device) * std_dev + mean, z)
    buffer[idx] = z.clamp(lower, upper).to(buffer.dtype)


def uniform_init(buffer: torch.Tensor, indices: torch.Tensor, curand_state_context: CurandStateContext, lower: float, upper: float) -> None:
    idx = _rows_of(buffer, indices)
    u = torch.rand(idx.numel(), buffer.shape[1], generator=curand_state_context.generator(buffer.device), device=buffer.device)
    buffer[idx] = (u * (upper - lower) + lower).to(buffer.dtype)


def const_init(buffer: torch.Tensor, indices: torch.Tensor, value: float) -> None:
    buffer[_rows_of(buffer, indices)] = value


def debug_init(buffer: torch.Tensor, indices: torch.Tensor, keys: torch.Tensor) -> None:
    """Row ``indices[i]`` is filled with ``keys[i] % 100000`` (values a test can predict from the key)."""
    idx = _rows_of(buffer, indices)
    buffer[idx] = (keys.to(buffer.device) % 100000).to(buffer.dtype)[:, None].expand(idx.numel(), buffer.shape[1])

"""Table-batched embedding ops (``csrc/cuda/embedding.cu``): sharded forward over peer pointers,
linearize + sort + run-length-encode, and the fused gradient-gather / segment-sum / optimizer update.

``TbeLayout`` is the device-side description of a group of logical tables and where their rows live
(this GPU or a peer).  The same layout drives the forward (pull rows from the owner) and the
backward (the owner pulls gradients from the sample's GPU).

Behavioural spec: FBGEMM table-batched-embedding "exact" semantics as used by the reference
(``hybrid_torchrec/distributed/batched_embedding_kernel.py:233-443``; NumPy golden in
``cust_op/ascendc_op/ai_core_op/recops_backward_codegen_adagrad_unweighted_exact/v220/README.md:78-135``).
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib

SH_LOCAL, SH_TABLE_WISE, SH_ROW_MOD, SH_ROW_BLOCK = 0, 1, 2, 3
POOL_SUM, POOL_MEAN, POOL_NONE = 0, 1, 2
OPT_SGD, OPT_ROWWISE_ADAGRAD, OPT_ADAGRAD, OPT_ADAM = 0, 1, 2, 3

_SHARD_DTYPE = np.dtype([("kind", "<i4"), ("owner", "<i4"), ("D", "<i4"), ("D_offset", "<i4"),
                         ("rows", "<i8"), ("block", "<i8"), ("ptr_index", "<i8"), ("key_base", "<i8")])


def local_rows(kind: int, rows: int, owner: int, world: int, rank: int) -> int:
    """Number of rows of a logical table that live on ``rank``."""
    if kind == SH_LOCAL:
        return rows
    if kind == SH_TABLE_WISE:
        return rows if owner == rank else 0
    if kind == SH_ROW_MOD:
        return max(0, (rows - rank + world - 1) // world)
    block = (rows + world - 1) // world
    return max(0, min(block, rows - rank * block))


@dataclasses.dataclass
class OptimizerSpec:
    """Sparse optimizer hyper-parameters (one spec per table group)."""
    kind: int = OPT_ROWWISE_ADAGRAD
    lr: float = 0.01
    eps: float = 1e-8
    beta1: float = 0.9
    beta2: float = 0.999
    weight_decay: float = 0.0
    initial_accumulator_value: float = 0.0
    accumulate_step: int = 1          # > 1: sum the row gradients of this many steps, then update once

    def state_elems_per_row(self, dim: int) -> int:
        return {OPT_SGD: 0, OPT_ROWWISE_ADAGRAD: 1, OPT_ADAGRAD: dim, OPT_ADAM: dim}[self.kind]


class TbeLayout:
    """Placement of physical tables across ``world`` ranks, as seen from ``rank``, plus the list of
    features (bag groups) that read them.

    ``kinds[t]`` is one of ``SH_*``; ``owners[t]`` is the owning rank for table-wise tables.
    ``feature_table[f]`` is the table read by feature ``f`` (several features may share a table).
    Each rank stores its rows of all tables back to back in one flat weight buffer;
    ``w_offsets[r, t]`` is the element offset of table ``t`` in rank ``r``'s buffer, which every rank
    can compute without talking.  ``T`` is the number of features: bags are indexed ``f * B + b``.
    """

    def __init__(self, dims: Sequence[int], rows: Sequence[int], kinds: Sequence[int], owners: Sequence[int],
                 world: int, rank: int, feature_table: Optional[Sequence[int]] = None) -> None:
        self.n_tables = len(dims)
        self.dims = [int(d) for d in dims]
        self.rows = [int(r) for r in rows]
        self.kinds = [int(k) for k in kinds]
        self.owners = [int(o) for o in owners]
        self.world, self.rank = int(world), int(rank)
        self.feature_table = list(range(self.n_tables)) if feature_table is None else [int(t) for t in feature_table]
        self.T = len(self.feature_table)
        self.feature_dims = [self.dims[t] for t in self.feature_table]
        self.D_offsets = np.concatenate([[0], np.cumsum(self.feature_dims)]).astype(np.int64)
        self.total_D = int(self.D_offsets[-1])
        self.max_D = max(self.dims) if self.dims else 0
        self.blocks = [(r + world - 1) // world for r in self.rows]
        self.local_rows = np.zeros((world, self.n_tables), dtype=np.int64)
        for r in range(world):
            for t in range(self.n_tables):
                self.local_rows[r, t] = local_rows(self.kinds[t], self.rows[t], self.owners[t], world, r)
        elems = self.local_rows * np.asarray(self.dims, dtype=np.int64)[None, :]
        self.w_offsets = np.zeros((world, self.n_tables), dtype=np.int64)
        if self.n_tables > 1:
            self.w_offsets[:, 1:] = np.cumsum(elems, axis=1)[:, :-1]
        self.local_elems = elems.sum(axis=1)
        # linear key space of this rank: rows of table t are keys [key_cumsum[t], key_cumsum[t+1])
        self.key_cumsum = np.concatenate([[0], np.cumsum(self.local_rows[rank])]).astype(np.int64)
        self.total_local_rows = int(self.key_cumsum[-1])
        self.key_bits = max(1, int(self.total_local_rows + 1).bit_length())
        self._dev = {}

    def table_slice(self, rank: int, t: int):
        """(element offset, local rows) of table ``t`` in ``rank``'s flat weight buffer."""
        return int(self.w_offsets[rank, t]), int(self.local_rows[rank, t])

    # -- device tensors -------------------------------------------------------
    def shard_records(self) -> np.ndarray:
        rec = np.zeros(self.T, dtype=_SHARD_DTYPE)
        for f, t in enumerate(self.feature_table):
            rec[f] = (self.kinds[t], self.owners[t], self.dims[t], int(self.D_offsets[f]), self.rows[t],
                      self.blocks[t], t * self.world, int(self.key_cumsum[t]))
        return rec

    def device_tensors(self, device: torch.device, base_ptrs: Sequence[int], itemsize: int):
        """Upload shard records / pointer table.  ``base_ptrs[r]`` is the device address of rank
        ``r``'s flat weight buffer as mapped in *this* process (peer mapping for r != rank)."""
        ptrs = np.zeros(max(1, self.n_tables * self.world), dtype=np.int64)
        for t in range(self.n_tables):
            for r in range(self.world):
                if base_ptrs[r]:
                    ptrs[t * self.world + r] = int(base_ptrs[r]) + int(self.w_offsets[r, t]) * itemsize
        d = {
            "shards": torch.from_numpy(self.shard_records().view(np.uint8).copy()).to(device),
            "ptrs": torch.from_numpy(ptrs).to(device),
            "key_cumsum": torch.from_numpy(self.key_cumsum.copy()).to(device),
            "w_offsets": torch.from_numpy(self.w_offsets[self.rank].copy()).to(device),
        }
        self._dev = d
        return d


@dataclasses.dataclass
class SortedSegments:
    """Result of linearize + sort + RLE for one batch (all device tensors, no host sync)."""
    sorted_bags: torch.Tensor
    unique_keys: torch.Tensor
    seg_offsets: torch.Tensor
    num_runs: torch.Tensor
    max_runs: int


class SegmentSorter:
    """Reusable workspace: keys/bags staging, CUB temp storage and outputs for up to ``max_nnz`` ids."""

    def __init__(self, max_nnz: int, device: torch.device) -> None:
        self.max_nnz = int(max_nnz)
        n = self.max_nnz
        L = _lib.lib()
        self.temp_bytes = int(L.rb_sort_segments_temp_bytes(n))
        i64 = dict(dtype=torch.int64, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        self.keys = torch.empty(n, **i64)
        self.bags = torch.empty(n, **i32)
        self.keys_sorted = torch.empty(n, **i64)
        self.bags_sorted = torch.empty(n, **i32)
        self.unique = torch.empty(n, **i64)
        self.counts = torch.empty(n + 1, **i32)
        self.seg_offsets = torch.empty(n + 1, **i32)
        self.num_runs = torch.zeros(1, **i32)
        self.temp = torch.empty(self.temp_bytes, dtype=torch.uint8, device=device)
        self.keys_owned: Optional[torch.Tensor] = None       # compaction outputs, allocated on first use
        self.bags_owned: Optional[torch.Tensor] = None
        self.owned_count = torch.zeros(1, **i32)

    def run(self, layout: TbeLayout, dev: dict, indices: torch.Tensor, offsets: Optional[torch.Tensor],
            B_global: int, owned_cap: Optional[int] = None) -> SortedSegments:
        """``owned_cap``: when the ids of all ranks were gathered, a host-side bound on how many of them this rank owns;
        the owned pairs are compacted first and only ``owned_cap`` entries are sorted (an overflow raises the status word)."""
        nnz = indices.numel()
        assert nnz <= self.max_nnz
        L = _lib.lib()
        st = _lib.stream_ptr(indices.device)
        rc = L.rb_tbe_linearize(dev["shards"].data_ptr(), indices.data_ptr(), int(indices.dtype == torch.int64),
                                _lib.ptr(offsets), layout.T, B_global, nnz, layout.world, layout.rank,
                                self.keys.data_ptr(), self.bags.data_ptr(), st)
        _lib.check(rc, "rb_tbe_linearize")
        keys_in, bags_in = self.keys, self.bags
        if owned_cap is not None and owned_cap < nnz:
            if self.keys_owned is None:
                self.keys_owned, self.bags_owned = torch.empty_like(self.keys), torch.empty_like(self.bags)
            rc = L.rb_compact_owned(self.keys.data_ptr(), self.bags.data_ptr(), nnz, self.keys_owned.data_ptr(),
                                    self.bags_owned.data_ptr(), self.owned_count.data_ptr(), int(owned_cap), self.temp.data_ptr(),
                                    self.temp_bytes, _lib.status_tensor(indices.device).data_ptr(), st)
            _lib.check(rc, "rb_compact_owned")
            keys_in, bags_in, nnz = self.keys_owned, self.bags_owned, int(owned_cap)
        rc = L.rb_sort_segments(keys_in.data_ptr(), bags_in.data_ptr(), nnz, layout.key_bits,
                                self.keys_sorted.data_ptr(), self.bags_sorted.data_ptr(), self.unique.data_ptr(),
                                self.counts.data_ptr(), self.seg_offsets.data_ptr(), self.num_runs.data_ptr(),
                                self.temp.data_ptr(), self.temp_bytes, st)
        _lib.check(rc, "rb_sort_segments")
        return SortedSegments(self.bags_sorted, self.unique, self.seg_offsets, self.num_runs, nnz)


def tbe_forward(layout: TbeLayout, dev: dict, indices: torch.Tensor, offsets: Optional[torch.Tensor], B: int,
                pooling: int, w_dtype: torch.dtype, out: torch.Tensor) -> torch.Tensor:
    """Pooled lookup of ``T x B`` bags into ``out[B, >= total_D]`` (row stride = ``out.stride(0)``).

    ``offsets`` is ``None`` for one-hot features (bag ``t*B+b`` holds ``indices[t*B+b]``)."""
    assert out.stride(1) == 1
    out_item = out.element_size()
    vec8_ok = int(all(d % 8 == 0 for d in layout.dims) and (out.stride(0) * out_item) % 16 == 0
                  and out.data_ptr() % 16 == 0)
    rc = _lib.lib().rb_tbe_forward(
        dev["shards"].data_ptr(), dev["ptrs"].data_ptr(), indices.data_ptr(), int(indices.dtype == torch.int64),
        _lib.ptr(offsets), layout.T, B, layout.world, layout.rank, pooling, _lib.dtype_code(w_dtype),
        out.data_ptr(), _lib.dtype_code(out.dtype), out.stride(0), vec8_ok,
        _lib.status_tensor(out.device).data_ptr(), _lib.stream_ptr(out.device))
    _lib.check(rc, "rb_tbe_forward")
    return out


def tbe_sequence(layout: TbeLayout, dev: dict, indices: torch.Tensor, pos_offsets: torch.Tensor,
                 w_dtype: torch.dtype, out: torch.Tensor) -> torch.Tensor:
    """Per-id lookup: ``out[j] = row(indices[j])``; ``pos_offsets[T+1]`` gives each table's id range."""
    rc = _lib.lib().rb_tbe_sequence(
        dev["shards"].data_ptr(), dev["ptrs"].data_ptr(), indices.data_ptr(), int(indices.dtype == torch.int64),
        pos_offsets.data_ptr(), layout.T, indices.numel(), layout.world, layout.rank, _lib.dtype_code(w_dtype),
        out.data_ptr(), _lib.dtype_code(out.dtype), out.stride(0), _lib.status_tensor(out.device).data_ptr(),
        _lib.stream_ptr(out.device))
    _lib.check(rc, "rb_tbe_sequence")
    return out


LONG_CHUNK = 32  # must match csrc/cuda/embedding.cu


class BackwardWorkspace:
    """Scratch of the fused backward: the list of long segments (rows hit by more than
    ``long_threshold`` bags), their chunk work-list and one fp32 accumulation row per long segment.
    ``long_accum`` is all-zero between launches (the kernels restore that themselves)."""

    def __init__(self, device: torch.device, max_nnz: int, max_D: int, long_cap: int = 8192) -> None:
        self.long_cap = int(long_cap)
        self.chunk_cap = int(max_nnz) // LONG_CHUNK + self.long_cap
        self.accum_ld = (int(max_D) + 127) // 128 * 128
        self.long_list = torch.empty(self.long_cap, dtype=torch.int32, device=device)
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)
        self.chunk_list = torch.empty(self.chunk_cap * 2, dtype=torch.int32, device=device)
        self.long_accum = torch.zeros(self.long_cap * self.accum_ld, dtype=torch.float32, device=device)


def tbe_backward_update(layout: TbeLayout, dev: dict, seg: SortedSegments, grad_ptrs: torch.Tensor, ld_g: int,
                        g_dtype: torch.dtype, B_local: int, offsets: Optional[torch.Tensor], pooling: int,
                        weights: torch.Tensor, state1: Optional[torch.Tensor], state2: Optional[torch.Tensor],
                        s_offsets: torch.Tensor, opt: OptimizerSpec, step: int, ws: BackwardWorkspace,
                        long_threshold: int = 256) -> None:
    """Sum gradients per unique owned row (reading each sample's gradient from the GPU that holds it
    through ``grad_ptrs[world]``) and apply the optimizer in place."""
    bc1 = 1.0 - opt.beta1 ** max(step, 1)
    bc2 = 1.0 - opt.beta2 ** max(step, 1)
    rc = _lib.lib().rb_tbe_backward_update(
        dev["shards"].data_ptr(), dev["key_cumsum"].data_ptr(), dev["w_offsets"].data_ptr(), s_offsets.data_ptr(),
        layout.T, layout.n_tables, B_local, layout.world, grad_ptrs.data_ptr(), ld_g, _lib.dtype_code(g_dtype), _lib.ptr(offsets),
        pooling, seg.sorted_bags.data_ptr(), seg.unique_keys.data_ptr(), seg.seg_offsets.data_ptr(),
        seg.num_runs.data_ptr(), seg.max_runs, weights.data_ptr(), _lib.dtype_code(weights.dtype),
        _lib.ptr(state1), _lib.ptr(state2), opt.kind, opt.lr, opt.eps, opt.beta1, opt.beta2, opt.weight_decay,
        bc1, bc2, layout.max_D, ws.long_list.data_ptr(), ws.counters.data_ptr(), ws.chunk_list.data_ptr(),
        ws.long_accum.data_ptr(), ws.long_cap, ws.chunk_cap, ws.accum_ld, long_threshold,
        _lib.num_sms(weights.device), _lib.status_tensor(weights.device).data_ptr(),
        _lib.stream_ptr(weights.device))
    _lib.check(rc, "rb_tbe_backward_update")


def tbe_backward_update_rows(layout: TbeLayout, dev: dict, seg: SortedSegments, grad_rows: torch.Tensor, ld_rows: int,
                             table_dims: torch.Tensor, weights: torch.Tensor, state1: Optional[torch.Tensor],
                             state2: Optional[torch.Tensor], s_offsets: torch.Tensor, opt: OptimizerSpec, step: int,
                             ws: BackwardWorkspace, long_threshold: int = 256) -> None:
    """The same fused segment-sum + optimizer with every gradient row already in local memory (push exchange):
    ``seg.sorted_bags[j]`` is the row of ``grad_rows`` (stride ``ld_rows`` elements) that belongs to sorted entry ``j``."""
    bc1 = 1.0 - opt.beta1 ** max(step, 1)
    bc2 = 1.0 - opt.beta2 ** max(step, 1)
    dummy = dev["key_cumsum"]
    rc = _lib.lib().rb_tbe_backward_update_rows(
        dev["shards"].data_ptr(), dev["key_cumsum"].data_ptr(), dev["w_offsets"].data_ptr(), s_offsets.data_ptr(),
        layout.T, layout.n_tables, 1, 1, dummy.data_ptr(), 0, _lib.dtype_code(grad_rows.dtype), None,
        POOL_SUM, seg.sorted_bags.data_ptr(), seg.unique_keys.data_ptr(), seg.seg_offsets.data_ptr(),
        seg.num_runs.data_ptr(), seg.max_runs, weights.data_ptr(), _lib.dtype_code(weights.dtype),
        _lib.ptr(state1), _lib.ptr(state2), opt.kind, opt.lr, opt.eps, opt.beta1, opt.beta2, opt.weight_decay,
        bc1, bc2, layout.max_D, ws.long_list.data_ptr(), ws.counters.data_ptr(), ws.chunk_list.data_ptr(),
        ws.long_accum.data_ptr(), ws.long_cap, ws.chunk_cap, ws.accum_ld, long_threshold,
        _lib.num_sms(weights.device), _lib.status_tensor(weights.device).data_ptr(),
        _lib.stream_ptr(weights.device), grad_rows.data_ptr(), ld_rows, table_dims.data_ptr())
    _lib.check(rc, "rb_tbe_backward_update_rows")


def pool_rows(rows: torch.Tensor, ld_rows: int, offsets: torch.Tensor, T: int, B: int, f_D: torch.Tensor, f_Doff: torch.Tensor,
              mean: bool, out: torch.Tensor) -> torch.Tensor:
    """``out[b, Doff[f]:Doff[f]+D[f]] = sum or mean over the ids j of bag (f, b) of rows[j, :D[f]]`` (fp32 accumulation)."""
    rc = _lib.lib().rb_pool_rows(rows.data_ptr(), _lib.dtype_code(rows.dtype), ld_rows, offsets.data_ptr(), T, B, f_D.data_ptr(),
                                 f_Doff.data_ptr(), int(mean), out.data_ptr(), _lib.dtype_code(out.dtype), out.stride(0),
                                 _lib.stream_ptr(out.device))
    _lib.check(rc, "rb_pool_rows")
    return out


def gather_rows(src: torch.Tensor, idx: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[i] = src[idx[i]]`` for a 2-D row-major ``src`` (HBM cache -> staging)."""
    if not src.is_cuda:
        res = src.index_select(0, idx)
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert src.is_contiguous() and idx.dtype == torch.int64
    if out is None:
        out = torch.empty((idx.numel(),) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
    row_bytes = src[0].numel() * src.element_size() if src.shape[0] else 0
    if idx.numel() and row_bytes:
        rc = _lib.lib().rb_gather_rows(src.data_ptr(), idx.data_ptr(), idx.numel(), row_bytes, out.data_ptr(),
                                       _lib.stream_ptr(src.device))
        _lib.check(rc, "rb_gather_rows")
    return out


def scatter_rows(src: torch.Tensor, idx: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """``dst[idx[i]] = src[i]`` (staging -> HBM cache)."""
    if not dst.is_cuda:
        dst.index_copy_(0, idx, src)
        return dst
    assert src.is_contiguous() and dst.is_contiguous() and idx.dtype == torch.int64
    row_bytes = dst[0].numel() * dst.element_size() if dst.shape[0] else 0
    if idx.numel() and row_bytes:
        rc = _lib.lib().rb_scatter_rows(src.data_ptr(), idx.data_ptr(), idx.numel(), row_bytes, dst.data_ptr(),
                                        _lib.stream_ptr(dst.device))
        _lib.check(rc, "rb_scatter_rows")
    return dst


# ---------------------------------------------------------------------------
# fp32 PyTorch reference of the whole lookup + exact backward (tests, CPU path)
# ---------------------------------------------------------------------------
def reference_pooled_forward(tables: List[torch.Tensor], indices: torch.Tensor, offsets: torch.Tensor, B: int,
                             pooling: int) -> torch.Tensor:
    outs = []
    off = offsets.tolist()
    for t, w in enumerate(tables):
        rows = []
        for b in range(B):
            ids = indices[off[t * B + b]:off[t * B + b + 1]]
            v = w.float()[ids].sum(0) if ids.numel() else torch.zeros(w.shape[1])
            if pooling == POOL_MEAN and ids.numel():
                v = v / ids.numel()
            rows.append(v)
        outs.append(torch.stack(rows))
    return torch.cat(outs, dim=1)


def copy_rows(src: torch.Tensor, src_idx: torch.Tensor, dst: torch.Tensor, dst_idx: torch.Tensor,
              device: Optional[torch.device] = None) -> None:
    """``dst[dst_idx[i]] = src[src_idx[i]]`` over 2-D row-major tensors.  With ``device`` a CUDA device, either
    tensor may be pinned host memory: the kernel reads / writes it through the unified address space."""
    if device is None or device.type != "cuda":
        dst[dst_idx.to(dst.device)] = src[src_idx.to(src.device)].to(dst.device)
        return
    assert src.is_contiguous() and dst.is_contiguous() and src.shape[1:] == dst.shape[1:] and src.dtype == dst.dtype
    assert (src.is_cuda or src.is_pinned()) and (dst.is_cuda or dst.is_pinned())
    assert src_idx.is_cuda and dst_idx.is_cuda and src_idx.dtype == torch.int64 and dst_idx.dtype == torch.int64
    row_bytes = src[0].numel() * src.element_size()
    rc = _lib.lib().rb_copy_rows(src.data_ptr(), src_idx.data_ptr(), dst.data_ptr(), dst_idx.data_ptr(), src_idx.numel(),
                                 row_bytes, _lib.num_sms(device), _lib.stream_ptr(device))
    _lib.check(rc, "rb_copy_rows")

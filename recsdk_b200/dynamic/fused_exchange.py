"""Multi-GPU lookup of a dynamic (hash-table backed) embedding table on the push exchange.

One ``FusedDynamicExchange`` serves all features that read one table.  Per step, without a host synchronisation and
without a library collective:

    sample side   route each id to ``key % world``; store (key, position) into the owner's dense receive list
    owner side    sort + run-length encode the received keys (one probe per distinct key), admission / find_or_insert in
                  the hash table, then one kernel reads every requested row from local memory by slot and stores it into
                  the requesting GPU's row list (``csrc/cuda/a2a_dynamic.cu``)
    backward      gradient rows are stored into the owner's gradient list; the owner sums them per distinct key from
                  local memory and runs the fused optimizer on the slots

Counts live on the device: owner-side buffers are sized for ``owned_cap`` entries, kernels stop at the received count,
keys beyond it are the empty key, which the table kernels skip.
Reference flow: ``dynamic_emb/distributed/sharding/rw_sharding.py:222-263`` and
``batched_dynamicemb_function.py:344-432`` (unique once per table, batched lookup, update on unique rows).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..ops import _lib
from ..ops import embedding_ops as E
from ..parallel.comm import PeerGroup
from ..parallel.push_exchange import MODE_POOLED, MODE_ROWS, PH_GRADS, PH_PAYLOAD, PH_ROWS, PushExchange
from .key_value_table import KeyValueTable


class FusedDynamicExchange:
    def __init__(self, peer: PeerGroup, table: KeyValueTable, device: torch.device, nnz_cap: int, owned_cap: int,
                 out_dtype: torch.dtype) -> None:
        self.peer, self.table, self.device = peer, table, device
        self.D = table.dim
        if self.D % 8:
            raise ValueError("the fused dynamic exchange needs an embedding dim that is a multiple of 8")
        self.out_dtype = out_dtype
        item = torch.empty(0, dtype=out_dtype).element_size()
        self.px = PushExchange(peer, device, nnz_cap, owned_cap, self.D, out_dtype, nnz_cap * self.D * item)
        cap = self.px.owned_cap
        i64 = dict(dtype=torch.int64, device=device)
        self.slots_u = torch.full((cap,), -1, **i64)
        self.slot_of_pos = torch.full((cap,), -1, **i64)
        self.run_of_sorted = torch.zeros(cap, **i64)
        self.red = torch.zeros(cap, self.D, dtype=torch.float32, device=device)
        self.rows_view = self.px.out_raw[: nnz_cap * self.D * item].view(out_dtype).view(nnz_cap, self.D)
        self._seg: Optional[E.SortedSegments] = None

    # ------------------------------------------------------------------ forward
    def lookup(self, ids: torch.Tensor, offsets: Optional[torch.Tensor], F: int, B: int, training: bool) -> torch.Tensor:
        """ids of all features of the table (feature-major) -> view ``[n, D]`` of the received rows (valid until the next
        call).  ``offsets`` (``F * B + 1``, rebased to start at 0) is given when the caller pools per bag."""
        L = _lib.lib()
        px, t = self.px, self.table
        st = _lib.stream_ptr(self.device)
        n = ids.numel()
        px.join()
        if offsets is None:
            px.route_scatter(ids, None, 1, max(n, 1), None, None, None, 0, want_bags=False)
        else:
            px.route_scatter(ids, offsets, F, B, None, None, None, 0, want_bags=True)
        # ---- owner side
        px.wait(PH_PAYLOAD)
        cap = px.owned_cap
        n_owned = px.n_owned
        _lib.check(L.rb_a2a_pad_keys(px.recv_keys.data_ptr(), n_owned.data_ptr(), cap, st), "rb_a2a_pad_keys")
        seg = px.sort_received(64)
        self._seg = seg
        _lib.check(L.rb_fill_tail_i64(px.unique.data_ptr(), px.num_runs.data_ptr(), cap, -1, st), "rb_fill_tail_i64")
        slots = t.lookup_slots_padded(px.unique, training)
        self.slots_u.copy_(slots)
        _lib.check(L.rb_expand_runs(px.seg_offsets.data_ptr(), px.num_runs.data_ptr(), px.pos_sorted.data_ptr(),
                                    self.slots_u.data_ptr(), cap, self.run_of_sorted.data_ptr(), self.slot_of_pos.data_ptr(), st),
                   "rb_expand_runs")
        tab = t.table
        host_ptr = tab.values_host.data_ptr() if getattr(tab, "values_host", None) is not None else None
        default = float(t.options.eval_initializer_args.value)
        rc = L.rb_a2a_serve_slots(self.slot_of_pos.data_ptr(), px.recv_meta.data_ptr(), n_owned.data_ptr(), cap,
                                  tab.values_hbm.data_ptr(), host_ptr, tab.hbm_rows, tab.row_dim, tab.dim, default,
                                  px.out_p.ctypes.data, _lib.dtype_code(self.out_dtype), self.D, px.ctl.ctypes.data,
                                  px.loc.data_ptr(), px.world, px.rank, _lib.num_sms(self.device), st)
        _lib.check(rc, "rb_a2a_serve_slots")
        # ---- sample side again
        px.wait(PH_ROWS)
        return self.rows_view[:n]

    # ------------------------------------------------------------------ backward
    def backward(self, g: torch.Tensor, mode: int, f_D: torch.Tensor, f_Doff: Optional[torch.Tensor], F: int, B: int,
                 offsets: Optional[torch.Tensor], mean: bool) -> None:
        L = _lib.lib()
        px = self.px
        st = _lib.stream_ptr(self.device)
        if g.dtype != self.out_dtype or g.stride(-1) != 1:
            g = g.to(self.out_dtype).contiguous()
        px.push_grads(g, mode, f_D, f_Doff, F, B, offsets, mean)
        px.wait(PH_GRADS)
        self.red.zero_()
        rc = L.rb_rows_segment_add(px.grad_recv.data_ptr(), _lib.dtype_code(self.out_dtype), px.g_ld,
                                   self.run_of_sorted.data_ptr(), px.pos_sorted.data_ptr(), px.keys_sorted.data_ptr(),
                                   px.owned_cap, self.D, self.red.data_ptr(), st)
        _lib.check(rc, "rb_rows_segment_add")
        self.table.update(self.slots_u, self.red)


class _FusedRowsFn(torch.autograd.Function):
    """Per-id rows of one table group (sequence embeddings)."""

    @staticmethod
    def forward(ctx, anchor: torch.Tensor, ex: FusedDynamicExchange, ids: torch.Tensor, training: bool):
        rows = ex.lookup(ids, None, 1, 1, training)
        ctx.ex, ctx.training, ctx.n = ex, training, ids.numel()
        return rows.clone()          # the exchange buffer is overwritten by the next lookup

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        if ctx.training and ctx.n:
            ex = ctx.ex
            fD = torch.tensor([ex.D], dtype=torch.int32, device=g.device)
            ex.backward(g, MODE_ROWS, fD, None, 1, max(ctx.n, 1), None, False)
        return None, None, None, None


class _FusedPooledFn(torch.autograd.Function):
    """Pooled rows ``[B, F * D]`` of the ``F`` features of one table group."""

    @staticmethod
    def forward(ctx, anchor: torch.Tensor, ex: FusedDynamicExchange, ids: torch.Tensor, offsets: torch.Tensor, F: int, B: int,
                mean: bool, training: bool, out_dtype: torch.dtype):
        rows = ex.lookup(ids, offsets, F, B, training)
        dev = ids.device
        f_D = torch.full((F,), ex.D, dtype=torch.int32, device=dev)
        f_Doff = torch.arange(F, dtype=torch.int32, device=dev) * ex.D
        out = torch.empty(B, F * ex.D, dtype=out_dtype, device=dev)
        E.pool_rows(ex.rows_view, ex.D, offsets, F, B, f_D, f_Doff, mean, out)
        ctx.ex, ctx.training, ctx.mean, ctx.F, ctx.B, ctx.n = ex, training, mean, F, B, ids.numel()
        ctx.save_for_backward(offsets, f_D, f_Doff)
        del rows
        return out

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        offsets, f_D, f_Doff = ctx.saved_tensors
        if ctx.training and ctx.n:
            ctx.ex.backward(g.contiguous(), MODE_POOLED, f_D, f_Doff, ctx.F, ctx.B, offsets, ctx.mean)
        return (None,) * 9


def owned_capacity(nnz_cap: int, world: int, factor: float = 3.0) -> int:
    """Entries an owner's receive list holds: ``factor`` times what one rank sends (keys spread by ``key % world``, hot
    keys land on one owner), never more than everything the job can send."""
    return int(min(world * nnz_cap, (int(factor * nnz_cap) + 8191) // 1024 * 1024))

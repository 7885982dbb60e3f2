"""Host side of the push-based sparse exchange (``csrc/cuda/a2a_push.cu``).

``PushExchange`` owns the peer-mapped buffers of one sharded embedding module (count matrix + flags, the owner-side
receive lists for keys and gradient rows, the requester-side output that owners store into) and issues the kernels:

    route -> scatter            sample side: ids to (owner, key); dense receive lists on the owners, O(owned) entries
    serve_rows                  owner side: local row gather, stores into the requester's output over NVLink
    sort (side stream)          owner side: received keys -> unique rows + segments for the backward
    push_grads -> update_rows   backward: gradient rows stored into the owner's list, segment-sum + optimizer locally

No host synchronisation and no library collective is involved; the counts travel through peer memory.
Reference counterparts: ``cust_op/ascendc_op/ai_core_op/lccl/v220/op_kernel/{gather_all,all2all,all2all_uss}.h``.
"""
from __future__ import annotations

import os
from typing import Optional

import numpy as np
import torch

from ..ops import _lib
from ..ops import embedding_ops as E
from .comm import PeerGroup

PH_COUNTS, PH_PAYLOAD, PH_ROWS, PH_GRADS = 0, 1, 2, 3
MODE_ONE_HOT, MODE_ROWS, MODE_POOLED = 0, 1, 2


class PushExchange:
    def __init__(self, peer: PeerGroup, device: torch.device, nnz_cap: int, owned_cap: int, g_ld: int,
                 g_dtype: torch.dtype, out_bytes: int) -> None:
        """``nnz_cap``: ids this rank sends per step at most; ``owned_cap``: entries its receive list can hold;
        ``g_ld``: elements per gradient row; ``out_bytes``: size of the buffer the owners store rows into."""
        L = _lib.lib()
        self.peer, self.device = peer, device
        self.world, self.rank = peer.world, peer.rank
        self.nnz_cap, self.owned_cap = int(nnz_cap), int(owned_cap)
        self.g_ld, self.g_dtype = int(g_ld), g_dtype
        gsz = torch.empty(0, dtype=g_dtype).element_size()
        al = lambda n: (int(n) + 255) // 256 * 256  # noqa: E731
        self._ctl_bytes = al(int(L.rb_a2a_ctl_ints()) * 4)
        self._keys_bytes = al(self.owned_cap * 8)
        self._grad_bytes = al(self.owned_cap * self.g_ld * gsz)
        self._out_bytes = al(out_bytes)
        total = self._ctl_bytes + 2 * self._keys_bytes + self._grad_bytes + self._out_bytes
        self._buf = peer.alloc(total, zero=True)
        base = np.asarray(self._buf.ptrs, dtype=np.uint64)
        off = 0
        self.ctl = base + np.uint64(off); off += self._ctl_bytes
        self.recv_keys_p = base + np.uint64(off); o_keys = off; off += self._keys_bytes
        self.recv_meta_p = base + np.uint64(off); o_meta = off; off += self._keys_bytes
        self.grad_recv_p = base + np.uint64(off); o_grad = off; off += self._grad_bytes
        self.out_p = base + np.uint64(off); o_out = off
        loc = self._buf.local
        self.recv_keys = loc[o_keys:o_keys + self.owned_cap * 8].view(torch.int64)
        self.recv_meta = loc[o_meta:o_meta + self.owned_cap * 8].view(torch.int64)
        self.grad_recv = loc[o_grad:o_grad + self.owned_cap * self.g_ld * gsz].view(g_dtype)
        self.out_raw = loc[o_out:o_out + out_bytes]
        self.loc = torch.zeros(int(L.rb_a2a_loc_ints()), dtype=torch.int32, device=device)
        self._n_owned_idx = int(L.rb_a2a_loc_n_owned_index())
        i64 = dict(dtype=torch.int64, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        self.entry_key = torch.empty(self.nnz_cap, **i64)
        self.entry_meta = torch.empty(self.nnz_cap, **i64)
        self.entry_dst = torch.empty(self.nnz_cap, **i32)
        self.entry_pos = torch.empty(self.nnz_cap, **i32)
        self.entry_bag = torch.empty(self.nnz_cap, **i32)
        # sort workspace: positions 0..cap-1 are the values carried through the sort
        n = self.owned_cap
        self.iota = torch.arange(n, **i32)
        self.temp_bytes = int(L.rb_sort_segments_temp_bytes(n))
        self.keys_sorted = torch.empty(n, **i64)
        self.pos_sorted = torch.empty(n, **i32)
        self.unique = torch.empty(n, **i64)
        self.counts = torch.empty(n + 1, **i32)
        self.seg_offsets = torch.empty(n + 1, **i32)
        self.num_runs = torch.zeros(1, **i32)
        self.temp = torch.empty(self.temp_bytes, dtype=torch.uint8, device=device)
        # the whole exchange runs on its own stream, so that dense work that does not depend on it (bottom MLP forward
        # and backward) proceeds on the caller's stream meanwhile; single-block wait kernels precede every kernel that
        # needs a peer's data, so no full grid ever spins
        self.stream = torch.cuda.Stream(device)
        self._pending: Optional[torch.cuda.Event] = None      # last work enqueued on the exchange stream
        self.nnz = 0
        self.deterministic = os.environ.get("LCCL_DETERMINISTIC", "0").lower() in ("1", "true")
        self._det_pos = self._det_meta = self._det_keys = None
        torch.cuda.synchronize(device)
        peer.host_barrier()

    @property
    def n_owned(self) -> torch.Tensor:
        """Device scalar: entries in this rank's receive list of the current step."""
        return self.loc[self._n_owned_idx]

    def _st(self) -> int:
        return _lib.stream_ptr(self.device)

    def _status(self) -> int:
        return _lib.status_tensor(self.device).data_ptr()

    # ------------------------------------------------------------------ forward, sample side
    def route_scatter(self, indices: torch.Tensor, offsets: Optional[torch.Tensor], T: int, B: int,
                      shards: Optional[torch.Tensor], key_base_all: Optional[torch.Tensor],
                      feature_table: Optional[torch.Tensor], n_tables: int, want_bags: bool) -> None:
        """ids -> owners' receive lists.  ``shards`` None routes raw 64-bit keys by ``key % world`` (dynamic tables)."""
        L = _lib.lib()
        nnz = indices.numel()
        if nnz > self.nnz_cap:
            raise ValueError("batch holds %d ids, the exchange was sized for %d (max_ids_per_rank)" % (nnz, self.nnz_cap))
        self.nnz = nnz
        ns = _lib.num_sms(self.device)
        rc = L.rb_a2a_route(_lib.ptr(shards), _lib.ptr(key_base_all), _lib.ptr(feature_table), n_tables,
                            indices.data_ptr(), int(indices.dtype == torch.int64), _lib.ptr(offsets), T, B, nnz,
                            self.world, self.rank, self.entry_key.data_ptr(), self.entry_meta.data_ptr(),
                            self.entry_dst.data_ptr(), self.entry_bag.data_ptr() if want_bags else None,
                            self.ctl.ctypes.data, self.loc.data_ptr(), ns, self._status(), self._st())
        _lib.check(rc, "rb_a2a_route")
        self.wait(PH_COUNTS)
        rc = L.rb_a2a_scatter(self.entry_key.data_ptr(), self.entry_meta.data_ptr(), self.entry_dst.data_ptr(),
                              self.entry_pos.data_ptr(), nnz, self.recv_keys_p.ctypes.data, self.recv_meta_p.ctypes.data,
                              self.owned_cap, self.ctl.ctypes.data, self.loc.data_ptr(), self.world, self.rank, ns,
                              self._status(), self.peer.timeout_ms, self._st())
        _lib.check(rc, "rb_a2a_scatter")

    # ------------------------------------------------------------------ forward, owner side
    def serve_rows(self, key_cumsum: torch.Tensor, w_offsets: torch.Tensor, table_dims: torch.Tensor,
                   f_Doff: Optional[torch.Tensor], n_tables: int, T: int, weights: torch.Tensor, out_dtype: torch.dtype,
                   ld_out: int, one_hot: bool, B: int) -> None:
        self.wait(PH_PAYLOAD)
        rc = _lib.lib().rb_a2a_serve_rows(
            self.recv_keys.data_ptr(), self.recv_meta.data_ptr(), self.owned_cap, key_cumsum.data_ptr(), w_offsets.data_ptr(),
            table_dims.data_ptr(), _lib.ptr(f_Doff), n_tables, T, weights.data_ptr(), _lib.dtype_code(weights.dtype),
            self.out_p.ctypes.data, _lib.dtype_code(out_dtype), ld_out, int(one_hot), B, self.ctl.ctypes.data,
            self.loc.data_ptr(), self.world, self.rank, _lib.num_sms(self.device), self._status(), self.peer.timeout_ms,
            self._st())
        _lib.check(rc, "rb_a2a_serve_rows")

    def sort_received(self, key_bits: int) -> E.SortedSegments:
        """Unique owned rows and their segments (the result is first needed in the backward).  Must be ordered after
        ``serve_rows``, which pads the tail of the key list.

        Positions in the receive list are handed out by atomics, so the order of the entries of one row - and with it the
        order of the floating-point additions of its gradient - changes from run to run.  ``LCCL_DETERMINISTIC=1`` (the
        reference's switch for its fused gradient all-to-all, ``lccl/v220/op_kernel/all_uss_deterministic.h``) first
        orders the entries by (source rank, feature, position in the source batch), then sorts stably by row: every
        row's gradients are then summed in an order that depends on the batch only."""
        L = _lib.lib()
        keys_in, vals_in = self.recv_keys, self.iota
        if self.deterministic:
            if self._det_pos is None:
                self._det_meta = torch.empty_like(self.recv_meta)
                self._det_pos = torch.empty_like(self.iota)
            rc = L.rb_sort_pairs_i64_i32(self.recv_meta.data_ptr(), self.iota.data_ptr(), self.owned_cap, 56,
                                         self._det_meta.data_ptr(), self._det_pos.data_ptr(), self.temp.data_ptr(),
                                         self.temp_bytes, self._st())
            _lib.check(rc, "rb_sort_pairs_i64_i32")
            self._det_keys = self.recv_keys.index_select(0, self._det_pos.long())
            keys_in, vals_in = self._det_keys, self._det_pos
        rc = L.rb_sort_segments(keys_in.data_ptr(), vals_in.data_ptr(), self.owned_cap, key_bits,
                                self.keys_sorted.data_ptr(), self.pos_sorted.data_ptr(), self.unique.data_ptr(),
                                self.counts.data_ptr(), self.seg_offsets.data_ptr(), self.num_runs.data_ptr(),
                                self.temp.data_ptr(), self.temp_bytes, self._st())
        _lib.check(rc, "rb_sort_segments")
        return E.SortedSegments(self.pos_sorted, self.unique, self.seg_offsets, self.num_runs, self.owned_cap)

    # ------------------------------------------------------------------ stream choreography
    def fork(self) -> "torch.cuda.StreamContext":
        """Context manager: the exchange stream, ordered after everything enqueued so far on the current stream."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self.stream.wait_event(ev)
        return torch.cuda.stream(self.stream)

    def mark(self) -> torch.cuda.Event:
        """Record (on the exchange stream, inside ``fork()``) an event that ``join`` or a consumer waits for."""
        ev = torch.cuda.Event()
        ev.record(self.stream)
        self._pending = ev
        return ev

    def join(self) -> None:
        """The current stream waits for everything enqueued on the exchange stream."""
        if self._pending is not None:
            torch.cuda.current_stream(self.device).wait_event(self._pending)
            self._pending = None

    def wait(self, phase: int) -> None:
        rc = _lib.lib().rb_a2a_wait(self.ctl.ctypes.data, self.loc.data_ptr(), phase, self.world, self.rank, self._status(),
                                    self.peer.timeout_ms, self._st())
        _lib.check(rc, "rb_a2a_wait")

    # ------------------------------------------------------------------ backward
    def push_grads(self, dout: torch.Tensor, mode: int, f_D: torch.Tensor, f_Doff: Optional[torch.Tensor], T: int, B: int,
                   offsets: Optional[torch.Tensor] = None, mean: bool = False) -> None:
        assert dout.stride(-1) == 1 and dout.dtype == self.g_dtype
        rc = _lib.lib().rb_a2a_push_grads(
            self.entry_meta.data_ptr(), self.entry_dst.data_ptr(), self.entry_pos.data_ptr(),
            self.entry_bag.data_ptr() if mode == MODE_POOLED else None, _lib.ptr(offsets), self.nnz, f_D.data_ptr(),
            _lib.ptr(f_Doff), T, B, mode, int(mean), dout.data_ptr(), _lib.dtype_code(dout.dtype), dout.stride(0),
            self.grad_recv_p.ctypes.data, self.g_ld, self.ctl.ctypes.data, self.loc.data_ptr(), self.world, self.rank,
            _lib.num_sms(self.device), self._st())
        _lib.check(rc, "rb_a2a_push_grads")

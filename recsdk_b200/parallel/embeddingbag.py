"""Sharded ``EmbeddingBagCollection`` on the fused peer-memory kernels.

Every rank keeps its shard of every table in one flat weight buffer.  With more than one GPU a train step is the push
exchange of ``push_exchange.py`` / ``csrc/cuda/a2a_push.cu``:

* ``input_dist``   route every local id to its owner and store (key, position) into the owner's dense receive list
                   (counts travel through peer memory, no host sync); the owner gathers the requested rows from its
                   own HBM and stores them straight into the requester's output - for one-hot features that is the
                   feature-interaction input ``[B_local, sum(D)]``, for variable-length bags a per-id row list that the
                   requester pools; the owner also sorts its received keys on a side stream for the backward,
* ``forward``      wait for the rows of all owners (one flag per owner),
* ``backward``     store the gradient row of every id into the owner's gradient list, then one kernel per owner
                   segment-sums per unique row from local memory and applies the sparse optimizer in place.

Sharding types: table-wise, row-wise (round-robin ``id % world`` like the reference's bucketize,
``hybrid_torchrec/src/ids_process/bucketize.cpp:46,66``, or contiguous blocks) and data-parallel (on several GPUs a
data-parallel table is stored row-wise: same numerics, one update per row instead of a replicated one).
The module contract (``input_dist`` / ``compute_and_output_dist`` / ``forward``) follows
``hybrid_torchrec/distributed/embeddingbag.py:481-693``.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Dict, List, Optional

import numpy as np
import torch
from torch import nn

from ..modules.embedding_configs import EmbeddingBagConfig, PoolingType, data_type_to_dtype
from ..modules.embedding_modules import TableDict
from ..ops import _lib
from ..ops import embedding_ops as E
from ..optim import FusedOptimizerStub
from ..sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor
from ..utils import trace
from .comm import PeerGroup, ShardingEnv
from .push_exchange import MODE_ONE_HOT, MODE_POOLED, PH_GRADS, PH_ROWS, PushExchange


@dataclasses.dataclass
class ParameterSharding:
    sharding_type: str = "row_wise"          # table_wise | row_wise | data_parallel
    compute_kernel: str = "fused"
    ranks: Optional[List[int]] = None        # owner for table_wise
    row_partition: str = "mod"               # mod (id % world) | block


_KIND = {"table_wise": E.SH_TABLE_WISE, "data_parallel": E.SH_LOCAL}


def _kind_of(ps: ParameterSharding) -> int:
    if ps.sharding_type == "row_wise":
        return E.SH_ROW_MOD if ps.row_partition == "mod" else E.SH_ROW_BLOCK
    if ps.sharding_type in _KIND:
        return _KIND[ps.sharding_type]
    raise NotImplementedError("sharding type %r is not supported" % ps.sharding_type)


@dataclasses.dataclass
class EmbeddingDistContext:
    """What ``input_dist`` hands to ``compute_and_output_dist``."""
    indices: torch.Tensor
    offsets: Optional[torch.Tensor]
    B_local: int
    segments: Optional[E.SortedSegments] = None
    global_offsets: Optional[torch.Tensor] = None
    one_hot: bool = False
    served: Optional[torch.cuda.Event] = None
    sorted: Optional[torch.cuda.Event] = None


class _LookupFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchor: torch.Tensor, mod: "ShardedEmbeddingBagCollection", dctx: EmbeddingDistContext):
        out = mod._lookup(dctx)
        ctx.mod, ctx.dctx = mod, dctx
        return out

    @staticmethod
    def backward(ctx, dout: torch.Tensor):
        ctx.mod._backward_update(ctx.dctx, dout)
        return None, None, None


class ShardedEmbeddingBagCollection(nn.Module):
    split_dist = True      # callers may run ``input_dist`` early and ``compute_and_output_dist(ctx)`` when the rows are needed

    def __init__(self, tables: List[EmbeddingBagConfig], plan: Dict[str, ParameterSharding], env: ShardingEnv,
                 device: torch.device, optimizer_spec: Optional[E.OptimizerSpec] = None,
                 peer: Optional[PeerGroup] = None, out_dtype: torch.dtype = torch.bfloat16,
                 max_local_batch: int = 0, max_ids_per_rank: int = 0, one_hot: bool = False,
                 init_weights: bool = True) -> None:
        super().__init__()
        if not tables:
            raise ValueError("need at least one table")
        self.env, self.device, self.out_dtype = env, device, out_dtype
        self.world, self.rank = env.world_size, env.rank
        self.tables = list(tables)
        self.opt = optimizer_spec or E.OptimizerSpec()
        self.one_hot = one_hot
        dts = {t.data_type for t in tables}
        if len(dts) != 1:
            raise ValueError("all tables of one collection must share a data type")
        self.w_dtype = data_type_to_dtype(tables[0].data_type)
        pools = {t.pooling for t in tables}
        if len(pools) != 1:
            raise ValueError("all tables of one collection must share a pooling type")
        self.pooling = {PoolingType.SUM: E.POOL_SUM, PoolingType.MEAN: E.POOL_MEAN}[tables[0].pooling]
        if self.pooling == E.POOL_MEAN and self.world > 1 and not one_hot:
            pass  # mean pooling divides by the bag length, known from the gathered offsets
        self.feature_names: List[str] = []
        feature_table: List[int] = []
        for ti, t in enumerate(tables):
            for f in t.feature_names:
                self.feature_names.append(f)
                feature_table.append(ti)
        kinds, owners = [], []
        for t in tables:
            ps = plan.get(t.name, ParameterSharding("row_wise" if self.world > 1 else "data_parallel"))
            k = _kind_of(ps)
            if self.world == 1:
                k = E.SH_LOCAL
            elif k == E.SH_LOCAL:
                k = E.SH_ROW_MOD          # several GPUs: a data-parallel table is stored row-wise (one update per row)
            kinds.append(k)
            owners.append((ps.ranks[0] if ps.ranks else 0) if k == E.SH_TABLE_WISE else 0)
        self.plan = plan
        self._kinds, self._owners, self._feature_table = kinds, owners, feature_table
        self.layout = E.TbeLayout([t.embedding_dim for t in tables], [t.num_embeddings for t in tables], kinds,
                                  owners, self.world, self.rank, feature_table)
        for d in self.layout.dims:
            if d % 8:
                raise ValueError("embedding_dim must be a multiple of 8 (16-byte row vectors)")
        self.peer = peer
        if self.world > 1 and peer is None:
            raise ValueError("world_size > 1 needs a PeerGroup")
        itemsize = torch.empty(0, dtype=self.w_dtype).element_size()
        max_elems = int(self.layout.local_elems.max())
        # owners read their rows locally and push them, so the weights need no peer mapping
        flat = torch.empty(max(int(self.layout.local_elems[self.rank]), 1), dtype=self.w_dtype, device=device)
        base_ptrs = [0] * self.world
        base_ptrs[self.rank] = flat.data_ptr()
        self.weights = flat
        del max_elems
        self.dev = self.layout.device_tensors(device, base_ptrs, itemsize)
        # optimizer state
        L = self.layout
        if self.opt.kind == E.OPT_ROWWISE_ADAGRAD:
            self.state1 = torch.full((max(L.total_local_rows, 1),), self.opt.initial_accumulator_value,
                                     dtype=torch.float32, device=device)
            self.state2 = None
            self.s_offsets = torch.from_numpy(L.key_cumsum[:-1].copy()).to(device)
        elif self.opt.kind in (E.OPT_ADAGRAD, E.OPT_ADAM):
            n = max(int(L.local_elems[self.rank]), 1)
            self.state1 = torch.full((n,), self.opt.initial_accumulator_value if self.opt.kind == E.OPT_ADAGRAD else 0.0,
                                     dtype=torch.float32, device=device)
            self.state2 = torch.zeros(n, dtype=torch.float32, device=device) if self.opt.kind == E.OPT_ADAM else None
            self.s_offsets = self.dev["w_offsets"]
        else:
            self.state1 = self.state2 = None
            self.s_offsets = self.dev["w_offsets"]
        self._step = 0
        # per-table parameter views (state_dict / user access); updates are fused in backward
        self.embedding_bags = TableDict()
        for ti, t in enumerate(tables):
            off, rows = L.table_slice(self.rank, ti)
            holder = nn.Module()
            w = nn.Parameter(self.weights[off:off + rows * t.embedding_dim].view(rows, t.embedding_dim),
                             requires_grad=False)
            w._in_backward_optimizers = True  # type: ignore[attr-defined]
            holder.weight = w
            self.embedding_bags[t.name] = holder
        if init_weights:
            self.reset_parameters()
        self._anchor = nn.Parameter(torch.zeros(1, device=device))   # makes autograd call our backward
        self._anchor._in_backward_optimizers = True  # type: ignore[attr-defined]
        self._bwd_ws: Optional[E.BackwardWorkspace] = None
        self._sorter: Optional[E.SegmentSorter] = None
        self._px: Optional[PushExchange] = None
        self._px_one_hot = False
        self.owned_cap_factor = float(os.environ.get("RECSDK_B200_OWNED_CAP_FACTOR", "3.0"))
        self._caps = (0, 0)
        self.max_local_batch, self.max_ids_per_rank = max_local_batch, max_ids_per_rank
        self.fused_optimizer = FusedOptimizerStub([h.weight for h in self.embedding_bags.values()], self.opt)

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def reset_parameters(self, seed: Optional[int] = None) -> None:
        """Uniform(-1/sqrt(rows), 1/sqrt(rows)) per table.  Values are a pure function of
        (seed, table, global row), so any sharding of the same model starts identically."""
        for ti, t in enumerate(self.tables):
            w = self.embedding_bags[t.name].weight
            if w.numel() == 0:
                continue
            if t.init_fn is not None:
                t.init_fn(w)
                continue
            lo, hi = t.get_weight_init_min(), t.get_weight_init_max()
            if seed is None:
                w.uniform_(lo, hi)
                continue
            rows = self.global_rows_of(ti)
            D = t.embedding_dim
            d = torch.arange(D, device=self.device, dtype=torch.int64)
            mix = (seed * 1000003 + ti * 7919 + 12345) & 0x7FFFFFFF
            chunk = max(1, (1 << 24) // D)
            for r0 in range(0, rows.numel(), chunk):        # bounded temporaries for 1e8-row tables
                x = rows[r0:r0 + chunk, None] * D + d[None, :] + mix
                x = ((x >> 16) ^ x) * 0x45D9F3B & 0xFFFFFFFF
                x = ((x >> 16) ^ x) * 0x45D9F3B & 0xFFFFFFFF
                x = (x >> 16) ^ x
                u = x.to(torch.float32) * (1.0 / 4294967296.0)
                w[r0:r0 + chunk].copy_((lo + (hi - lo) * u).to(w.dtype))

    @torch.no_grad()
    def load_from_unsharded(self, ebc: nn.Module) -> None:
        """Copy this rank's rows out of an unsharded collection that holds full tables."""
        for ti, t in enumerate(self.tables):
            w = self.embedding_bags[t.name].weight
            if w.numel() == 0:
                continue
            full = ebc.embedding_bags[t.name].weight.detach()
            rows = self.global_rows_of(ti).to(full.device)
            w.copy_(full.index_select(0, rows).to(device=w.device, dtype=w.dtype))

    @torch.no_grad()
    def full_table(self, name: str) -> torch.Tensor:
        """Debug / test helper: the whole logical table gathered on every rank (fp32, host)."""
        import torch.distributed as dist

        ti = [t.name for t in self.tables].index(name)
        t = self.tables[ti]
        w = self.embedding_bags[name].weight.detach().float().cpu()
        rows = self.global_rows_of(ti).cpu()
        full = torch.zeros(t.num_embeddings, t.embedding_dim)
        if self.world == 1 or self.layout.kinds[ti] == E.SH_LOCAL:
            full[rows] = w
            return full
        parts = [None] * self.world
        dist.all_gather_object(parts, (rows, w), group=self.env.process_group)
        for r_rows, r_w in parts:
            if r_rows.numel():
                full[r_rows] = r_w
        return full

    def global_rows_of(self, ti: int) -> torch.Tensor:
        """Global row id of every local row of table ``ti`` on this rank."""
        L = self.layout
        n = int(L.local_rows[self.rank, ti])
        r = torch.arange(n, device=self.device, dtype=torch.int64)
        k = L.kinds[ti]
        if k == E.SH_ROW_MOD:
            return r * self.world + self.rank
        if k == E.SH_ROW_BLOCK:
            return r + self.rank * L.blocks[ti]
        return r

    # ------------------------------------------------------------ workspaces
    def _ensure_capacity(self, B_local: int, nnz_local: int, one_hot: bool) -> None:
        if self.world == 1:
            cap_b = max(self.max_local_batch, B_local)
            cap_n = max(self.max_ids_per_rank, nnz_local)
            if self._sorter is not None and self._caps[0] >= cap_b and self._caps[1] >= cap_n:
                return
            cap_n = (cap_n + 1) // 2 * 2
            self._caps = (cap_b, cap_n)
            self._sorter = E.SegmentSorter(cap_n, self.device)
            self._bwd_ws = E.BackwardWorkspace(self.device, cap_n, self.layout.max_D)
            return
        if self._px is not None:
            if B_local > self._caps[0] or nnz_local > self._caps[1] or one_hot != self._px_one_hot:
                raise ValueError("batch (%d samples, %d ids, one_hot=%s) exceeds what the exchange buffers were sized for "
                                 "(%d samples, %d ids, one_hot=%s): pass max_local_batch / max_ids_per_rank"
                                 % (B_local, nnz_local, one_hot, self._caps[0], self._caps[1], self._px_one_hot))
            return
        # Peer buffers are allocated collectively, so every rank must arrive at the same sizes: take the maximum over ranks
        # of the first batch (one host-side exchange, set-up only) unless the caller gave explicit bounds.
        import torch.distributed as dist

        cap_b, cap_n = max(self.max_local_batch, B_local), max(self.max_ids_per_rank, nnz_local)
        t = torch.tensor([cap_b, cap_n, 0 if self.max_ids_per_rank else 1], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.env.process_group)
        cap_b, cap_n, guessed = int(t[0]), int(t[1]), bool(t[2])
        if guessed and not one_hot:
            cap_n = int(cap_n * 1.5) + 1024         # variable-length bags: head-room over the first batch
        cap_n = (cap_n + 7) // 8 * 8
        self._caps = (cap_b, cap_n)
        L = self.layout
        owned = self._owned_cap(cap_b * self.world, cap_n, one_hot)
        out_item = torch.empty(0, dtype=self.out_dtype).element_size()
        w_item = torch.empty(0, dtype=self.w_dtype).element_size()
        self._row_ld = (L.max_D + 7) // 8 * 8
        out_bytes = cap_b * L.total_D * out_item if one_hot else cap_n * self._row_ld * w_item
        self._px = PushExchange(self.peer, self.device, cap_n, owned, self._row_ld, self.out_dtype, out_bytes)
        self._px_one_hot = one_hot
        self._bwd_ws = E.BackwardWorkspace(self.device, owned, L.max_D)
        i32 = dict(dtype=torch.int32, device=self.device)
        self._f_D = torch.tensor(L.feature_dims, **i32)
        self._f_Doff = torch.tensor([int(x) for x in L.D_offsets[:-1]], **i32)
        self._table_dims = torch.tensor(L.dims, **i32)
        self._feature_table_dev = torch.tensor(L.feature_table, **i32)
        kb = np.zeros((self.world, L.n_tables), dtype=np.int64)
        if L.n_tables > 1:
            kb[:, 1:] = np.cumsum(L.local_rows, axis=1)[:, :-1]
        self._key_base_all = torch.from_numpy(kb).to(self.device)
        if one_hot:
            self._out_view = self._px.out_raw[: cap_b * L.total_D * out_item].view(self.out_dtype).view(cap_b, L.total_D)
        else:
            self._rows_view = self._px.out_raw[: cap_n * self._row_ld * w_item].view(self.w_dtype).view(cap_n, self._row_ld)

    def _owned_cap(self, Bg: int, nnz_cap: int, one_hot: bool) -> int:
        """Capacity of this rank's receive list.  One-hot: all ids of the table-wise tables it owns plus ``owned_cap_factor``
        times the fair share of the row-wise ones (hot ids cluster on a few residues).  Variable-length bags:
        ``owned_cap_factor`` times the ids one rank sends.  Never more than everything the job can send.  A step that
        would exceed it sets ``RB_ERR_CAPACITY`` (polled by the train pipelines, which raise)."""
        factor = self.owned_cap_factor
        if not one_hot:
            return int(min(self.world * nnz_cap, (int(factor * nnz_cap) + 8191) // 1024 * 1024))
        need = [0.0] * self.world            # the same list on every rank: it depends on the plan only
        for f in range(self.layout.T):
            ti = self._feature_table[f]
            if self._kinds[ti] == E.SH_TABLE_WISE:
                need[self._owners[ti]] += Bg
            else:
                for r in range(self.world):
                    need[r] += factor * Bg / self.world
        return int(min(self.layout.T * Bg, (int(max(need)) + 8191) // 1024 * 1024))

    # ------------------------------------------------------------ input dist
    def input_dist(self, features: KeyedJaggedTensor) -> EmbeddingDistContext:
        assert features.keys() == self.feature_names, "feature order must match the table configs"
        B = features.stride()
        idx = features.values()
        if idx.dtype not in (torch.int64, torch.int32):
            idx = idx.long()
        idx = idx.contiguous()
        one_hot = self.one_hot or bool(getattr(features, "one_hot", False))
        offsets = None if one_hot else features.offsets().contiguous()
        nnz = idx.numel()
        self._ensure_capacity(B, nnz, one_hot)
        dctx = EmbeddingDistContext(idx, offsets, B, one_hot=one_hot)
        L = self.layout
        if self.world == 1:
            dctx.segments = self._sorter.run(L, self.dev, idx, offsets, B)
            dctx.global_offsets = offsets
            return dctx
        px = self._px
        px.join()                       # the previous step's update (exchange stream) is ordered before this step
        trace.mark("emb.input_dist")
        with px.fork():
            px.route_scatter(idx, offsets, L.T, B, self.dev["shards"], self._key_base_all, self._feature_table_dev,
                             L.n_tables, want_bags=not one_hot)
            if one_hot:
                px.serve_rows(self.dev["key_cumsum"], self.dev["w_offsets"], self._table_dims, self._f_Doff, L.n_tables, L.T,
                              self.weights, self.out_dtype, L.total_D, True, B)
            else:
                px.serve_rows(self.dev["key_cumsum"], self.dev["w_offsets"], self._table_dims, None, L.n_tables, L.T,
                              self.weights, self.w_dtype, self._row_ld, False, B)
            dctx.served = px.mark()
            if self.training and torch.is_grad_enabled():
                dctx.segments = px.sort_received(L.key_bits)
                dctx.sorted = px.mark()
        return dctx

    # --------------------------------------------------------------- compute
    def _lookup(self, dctx: EmbeddingDistContext) -> torch.Tensor:
        L = self.layout
        if self.world == 1:
            out = torch.empty(dctx.B_local, L.total_D, dtype=self.out_dtype, device=self.device)
            trace.mark("emb.lookup")
            E.tbe_forward(L, self.dev, dctx.indices, dctx.offsets, dctx.B_local, self.pooling, self.w_dtype, out)
            trace.mark("dense.forward")
            return out
        trace.mark("emb.wait_rows")
        torch.cuda.current_stream(self.device).wait_event(dctx.served)
        self._px.wait(PH_ROWS)
        if dctx.one_hot:
            out = self._out_view[: dctx.B_local]
        else:
            out = torch.empty(dctx.B_local, L.total_D, dtype=self.out_dtype, device=self.device)
            E.pool_rows(self._rows_view, self._row_ld, dctx.offsets, L.T, dctx.B_local, self._f_D, self._f_Doff,
                        self.pooling == E.POOL_MEAN, out)
        trace.mark("dense.forward")
        return out

    def _backward_update(self, dctx: EmbeddingDistContext, dout: torch.Tensor) -> None:
        self._step += 1
        self.opt.lr = self.fused_optimizer.param_groups[0]["lr"]
        if self.world == 1:
            g = dout if dout.is_contiguous() else dout.contiguous()
            ptrs = torch.tensor([g.data_ptr()], dtype=torch.int64, device=self.device) \
                if not torch.cuda.is_current_stream_capturing() else self._static_ptr(g)
            E.tbe_backward_update(self.layout, self.dev, dctx.segments, ptrs, g.stride(0), g.dtype, dctx.B_local,
                                  dctx.global_offsets, self.pooling, self.weights, self.state1, self.state2,
                                  self.s_offsets, self.opt, self._step, self._bwd_ws)
            return
        px = self._px
        L = self.layout
        if dctx.segments is None:
            raise RuntimeError("backward through a lookup whose input_dist ran without gradients enabled")
        g = dout if (dout.stride(-1) == 1 and dout.dtype == self.out_dtype) else dout.to(self.out_dtype).contiguous()
        trace.mark("emb.grad_push")
        # Exchange stream (already past this step's sort, which must be complete on this rank before any peer can be
        # released into the next step): push the gradient rows to their owners, wait for everyone's rows, update.  The
        # caller's stream goes straight on with the rest of the dense backward.
        with px.fork():
            if dctx.one_hot:
                px.push_grads(g, MODE_ONE_HOT, self._f_D, self._f_Doff, L.T, dctx.B_local)
            else:
                px.push_grads(g, MODE_POOLED, self._f_D, self._f_Doff, L.T, dctx.B_local, dctx.offsets,
                              self.pooling == E.POOL_MEAN)
            px.wait(PH_GRADS)
            E.tbe_backward_update_rows(L, self.dev, dctx.segments, px.grad_recv, px.g_ld, self._table_dims, self.weights,
                                       self.state1, self.state2, self.s_offsets, self.opt, self._step, self._bwd_ws)
            px.mark()
        if g.is_cuda:
            g.record_stream(px.stream)
        trace.mark("dense.backward_rest")

    def join_exchange(self) -> None:
        """Order the current stream after the sparse update that runs on the exchange stream (end of a step)."""
        if self._px is not None:
            self._px.join()

    def _static_ptr(self, g: torch.Tensor) -> torch.Tensor:
        # under CUDA-graph capture the gradient tensor's address is stable across replays
        t = torch.empty(1, dtype=torch.int64, device=self.device)
        t.fill_(g.data_ptr())
        return t

    def compute_and_output_dist(self, dctx: EmbeddingDistContext) -> KeyedTensor:
        out = _LookupFn.apply(self._anchor, self, dctx)
        return KeyedTensor(self.feature_names, self.layout.feature_dims, out)

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        return self.compute_and_output_dist(self.input_dist(features))

    # ------------------------------------------------------------- utilities
    def embedding_bag_configs(self) -> List[EmbeddingBagConfig]:
        return self.tables

    def pooled_dim(self) -> int:
        return self.layout.total_D

    def table_weight(self, name: str) -> torch.Tensor:
        return self.embedding_bags[name].weight

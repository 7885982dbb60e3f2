"""Sharded ``EmbeddingBagCollection`` on the fused peer-memory kernels.

Every rank keeps its shard of every table in one flat, peer-mapped weight buffer.  A train step does

* ``input_dist``   push this rank's ids (and bag offsets) into every peer's gathered-id buffer and cross
                   a device barrier; linearize + sort + run-length-encode the ids this rank owns,
* ``forward``      one kernel pulls the rows of the local batch from whichever GPU owns them and writes
                   the pooled result ``[B_local, sum(D)]`` (no id all-to-all, no pooled all-to-all),
* ``backward``     publish the pooled-output gradient in a peer-mapped buffer, barrier, then one kernel
                   per owner: pull the gradients of every bag that touched an owned row from the GPU
                   that holds the sample, segment-sum them and apply the sparse optimizer in place.

Sharding types: table-wise, row-wise (round-robin ``id % world`` like the reference's bucketize,
``hybrid_torchrec/src/ids_process/bucketize.cpp:46,66``, or contiguous blocks) and data-parallel
(replicated; gradients of a replicated table are summed by the owner-pull kernel on every rank).
The module contract (``input_dist`` / ``compute_and_output_dist`` / ``forward``) follows
``hybrid_torchrec/distributed/embeddingbag.py:481-693``.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import numpy as np
import torch
from torch import nn

from ..modules.embedding_configs import EmbeddingBagConfig, PoolingType, data_type_to_dtype
from ..ops import _lib
from ..ops import embedding_ops as E
from ..optim import FusedOptimizerStub
from ..sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor
from ..utils import trace
from .comm import PeerGroup, ShardingEnv


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
        if self.world > 1:
            self._wbuf = peer.alloc(max(max_elems, 1) * itemsize)
            base_ptrs = self._wbuf.ptrs
            flat = self._wbuf.local.view(self.w_dtype)
        else:
            flat = torch.empty(max(max_elems, 1), dtype=self.w_dtype, device=device)
            self._wbuf = None
            base_ptrs = [flat.data_ptr()]
        self.weights = flat
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
        self.embedding_bags = nn.ModuleDict()
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
        self._gather_ids: Optional[object] = None
        self._gather_offs: Optional[object] = None
        self._grad_buf: Optional[object] = None
        self._grad_ptrs: Optional[torch.Tensor] = None
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
    def _ensure_capacity(self, B_local: int, nnz_local: int) -> None:
        cap_b = max(self.max_local_batch, B_local)
        cap_n = max(self.max_ids_per_rank, nnz_local)
        if self._sorter is not None and self._caps[0] >= cap_b and self._caps[1] >= cap_n:
            return
        cap_n = (cap_n + 1) // 2 * 2
        self._caps = (cap_b, cap_n)
        T = self.layout.T
        self._sorter = E.SegmentSorter(cap_n * self.world, self.device)
        self._bwd_ws = E.BackwardWorkspace(self.device, cap_n * self.world, self.layout.max_D)
        if self.world > 1:
            self._gather_ids = self.peer.alloc(self.world * cap_n * 8)
            self._gather_offs = self.peer.alloc(self.world * (T * cap_b + 2) * 8)
            self._grad_buf = self.peer.alloc(cap_b * self.layout.total_D * 2 if self.out_dtype != torch.float32
                                             else cap_b * self.layout.total_D * 4)
            self._grad_ptrs = self._grad_buf.ptr_tensor(self.device)

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
        self._ensure_capacity(B, nnz)
        dctx = EmbeddingDistContext(idx, offsets, B)
        T = self.layout.T
        if self.world == 1:
            dctx.segments = self._sorter.run(self.layout, self.dev, idx, offsets, B)
            dctx.global_offsets = offsets
            return dctx
        # --- multi-GPU: gather everyone's ids (and offsets) into every rank, then barrier
        if not one_hot:
            raise NotImplementedError("multi-GPU fused path currently takes one-hot (fixed-length-1) features; "
                                      "use the collective backend for variable-length bags")
        if idx.dtype != torch.int64:
            idx = idx.long()
        cap_b, _ = self._caps
        assert B == cap_b or self.max_local_batch == 0 or B <= cap_b
        Bg = B * self.world
        row_bytes = B * 8
        trace.mark("emb.id_push")
        self.peer.allgather_push_2d(self._gather_ids, idx.view(T, B), Bg * 8, self.rank * row_bytes)
        trace.mark("emb.id_barrier")
        self.peer.barrier()
        trace.mark("emb.sort")
        gathered = self._gather_ids.local.view(torch.int64)[: T * Bg]
        dctx.segments = self._sorter.run(self.layout, self.dev, gathered, None, Bg, owned_cap=self._owned_cap(Bg))
        trace.mark("emb.sort_done")
        return dctx

    def _owned_cap(self, Bg: int) -> int:
        """Bound on the ids of a gathered one-hot batch that this rank owns: all ids of its table-wise tables, twice the
        fair share of the row-wise ones (hot ids cluster on a few residues), everything of replicated tables."""
        exp = 0.0
        for f in range(self.layout.T):
            ti = self._feature_table[f]
            k = self._kinds[ti]
            if k == E.SH_TABLE_WISE:
                exp += Bg if self._owners[ti] == self.rank else 0
            elif k in (E.SH_ROW_MOD, E.SH_ROW_BLOCK):
                exp += 2.0 * Bg / self.world
            else:
                exp += Bg
        return int(min(self.layout.T * Bg, (int(exp) + 8191) // 1024 * 1024))

    # --------------------------------------------------------------- compute
    def _lookup(self, dctx: EmbeddingDistContext) -> torch.Tensor:
        out = torch.empty(dctx.B_local, self.layout.total_D, dtype=self.out_dtype, device=self.device)
        trace.mark("emb.lookup")
        E.tbe_forward(self.layout, self.dev, dctx.indices, dctx.offsets, dctx.B_local, self.pooling, self.w_dtype, out)
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
        trace.mark("emb.grad_publish")
        gb = self._grad_buf.local.view(dout.dtype)[: dout.numel()].view(dout.shape)
        if dout.data_ptr() != gb.data_ptr():           # the consumer may already have written into the published buffer
            gb.copy_(dout)
        trace.mark("emb.grad_barrier")
        self.peer.barrier()
        trace.mark("emb.backward_update")
        E.tbe_backward_update(self.layout, self.dev, dctx.segments, self._grad_ptrs, self.layout.total_D, dout.dtype,
                              dctx.B_local, None, self.pooling, self.weights, self.state1, self.state2,
                              self.s_offsets, self.opt, self._step, self._bwd_ws)
        trace.mark("dense.backward_rest")

    def _static_ptr(self, g: torch.Tensor) -> torch.Tensor:
        # under CUDA-graph capture the gradient tensor's address is stable across replays
        t = torch.empty(1, dtype=torch.int64, device=self.device)
        t.fill_(g.data_ptr())
        return t

    def compute_and_output_dist(self, dctx: EmbeddingDistContext) -> KeyedTensor:
        out = _LookupFn.apply(self._anchor, self, dctx)
        if self.world > 1:
            out._grad_out_buffer = self._grad_buf.local.view(out.dtype)[: out.numel()].view(out.shape)
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

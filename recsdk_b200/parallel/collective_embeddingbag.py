"""Sharded ``EmbeddingBagCollection`` on ``torch.distributed`` collectives (gloo on CPU, NCCL on GPU).

This is the classic three-stage flow the reference inherits from TorchRec
(``hybrid_torchrec/distributed/embeddingbag.py:514-693``, ``sharding/hybrid_rw_sharding.py``):

* ``input_dist``   bucketize the local KJT by owner rank (row-wise: ``id % world`` or contiguous blocks,
                   table-wise: the owning rank) with the native bucketize op, exchange the per-bucket
                   lengths and then the ids with ``all_to_all_single``;
* ``post_input_dist``  (hash tables only) map raw ids to local slots with the owner's ``IdsMapper`` and
                   de-duplicate them (fused unique + lookup, optionally table-parallel);
* lookup           pool this rank's rows for the *global* batch;
* ``output_dist``  all-to-all of the partial pooled rows + sum over source shards (= reduce-scatter).

The sparse update is applied inside backward ("exact" semantics: gradients are first summed per unique
row, then SGD / Adagrad / row-wise Adagrad / Adam is applied once per row).  It runs everywhere PyTorch
runs, is the numerical oracle of the fused GPU path, and is the "NCCL-only" baseline on GPUs.
"""
from __future__ import annotations

import dataclasses
import os
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist
from torch import nn

from ..host import host
from ..modules.embedding_configs import EmbeddingBagConfig, PoolingType, data_type_to_dtype
from ..modules.embedding_modules import TableDict
from ..ops import embedding_ops as E
from ..optim import FusedOptimizerStub
from ..sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor
from .comm import ShardingEnv
from .embeddingbag import ParameterSharding, _kind_of


def _env_threads(name: str, default: int = 6) -> int:
    try:
        return max(1, min(12, int(os.environ.get(name, default))))
    except ValueError:
        return default


class _AllToAll(torch.autograd.Function):
    """Differentiable ``all_to_all_single`` with explicit split sizes along dim 0."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, out_splits: List[int], in_splits: List[int], pg):
        ctx.pg, ctx.out_splits, ctx.in_splits = pg, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=pg)
        return out

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        gi = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(gi, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.pg)
        return gi, None, None, None


def apply_sparse_update(weight: torch.Tensor, state: Dict[str, torch.Tensor], rows: torch.Tensor, grads: torch.Tensor,
                        opt: E.OptimizerSpec, step: int) -> None:
    """Exact sparse update: ``grads[i]`` belongs to ``rows[i]``; duplicates are summed first.
    Reference math: NumPy golden in ``recops_backward_codegen_adagrad_unweighted_exact/v220/README.md:78-135``
    and ``dynamic_emb/csrc/ops/Rowwise_adagrad_update/rowwise_adagrad_update.cpp:51-98``."""
    if rows.numel() == 0:
        return
    uniq, inv = torch.unique(rows, return_inverse=True)
    g = torch.zeros(uniq.numel(), weight.shape[1], dtype=torch.float32, device=weight.device)
    g.index_add_(0, inv, grads.float())
    w = weight.data[uniq].float()
    if opt.kind == E.OPT_SGD:
        w = w - opt.lr * (g + opt.weight_decay * w)
    elif opt.kind == E.OPT_ROWWISE_ADAGRAD:
        acc = state["state1"]
        a = acc[uniq] + (g * g).mean(dim=1)
        acc[uniq] = a
        w = w - opt.lr * g / (a.sqrt() + opt.eps)[:, None]
    elif opt.kind == E.OPT_ADAGRAD:
        acc = state["state1"]
        a = acc[uniq] + g * g
        acc[uniq] = a
        w = w - opt.lr * g / (a.sqrt() + opt.eps)
    else:
        m, v = state["state1"], state["state2"]
        gg = g + opt.weight_decay * w
        mm = opt.beta1 * m[uniq] + (1 - opt.beta1) * gg
        vv = opt.beta2 * v[uniq] + (1 - opt.beta2) * gg * gg
        m[uniq], v[uniq] = mm, vv
        bc1, bc2 = 1 - opt.beta1 ** step, 1 - opt.beta2 ** step
        w = w - (opt.lr / bc1) * mm / ((vv / bc2).sqrt() + opt.eps)
    weight.data[uniq] = w.to(weight.dtype)


class _PooledLookup(torch.autograd.Function):
    """Pooled lookup of one table shard whose sparse update happens in backward."""

    @staticmethod
    def forward(ctx, anchor, mod, ti: int, rows: torch.Tensor, offsets: torch.Tensor, mean: bool, n_bags: int):
        w = mod.embedding_bags[mod.tables[ti].name].weight
        if rows.numel():
            out = torch.nn.functional.embedding_bag(rows, w.data.float(), offsets[:-1], mode="mean" if mean else "sum",
                                                    include_last_offset=False)
        else:
            out = torch.zeros(n_bags, w.shape[1], dtype=torch.float32, device=w.device)
        ctx.mod, ctx.ti, ctx.mean = mod, ti, mean
        ctx.save_for_backward(rows, offsets)
        return out

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        rows, offsets = ctx.saved_tensors
        mod, ti = ctx.mod, ctx.ti
        lengths = offsets[1:] - offsets[:-1]
        bag = torch.repeat_interleave(torch.arange(lengths.numel(), device=rows.device), lengths)
        gr = g[bag]
        if ctx.mean:
            gr = gr / lengths[bag].clamp(min=1).to(gr.dtype)[:, None]
        mod._apply_update(ti, rows, gr)
        return None, None, None, None, None, None, None


@dataclasses.dataclass
class DistState:
    """One batch's way through the five input-distribution stages of one sharded module (split -> lengths all-to-all ->
    id all-to-all -> id mapping -> device copy).  Host tensors throughout; futures / work handles of the stage in flight."""
    module: Any
    features: Any
    F: int
    B: int
    orig_lengths: Optional[torch.Tensor] = None
    split_future: Any = None
    send_lengths: Optional[torch.Tensor] = None
    send_ids: Optional[torch.Tensor] = None
    recv_lengths: Optional[torch.Tensor] = None
    recv_ids: Optional[torch.Tensor] = None
    ids_work: Any = None
    post_future: Any = None
    mapped_ids: Optional[torch.Tensor] = None


class CollectiveShardedEmbeddingBagCollection(nn.Module):
    def __init__(self, tables: List[EmbeddingBagConfig], plan: Dict[str, ParameterSharding], env: ShardingEnv,
                 device: torch.device, optimizer_spec: Optional[E.OptimizerSpec] = None, hashed: bool = False,
                 out_dtype: torch.dtype = torch.float32, init_weights: bool = True,
                 input_env: Optional[ShardingEnv] = None) -> None:
        """``input_env``: optional host-side (gloo) environment; when given, the id exchange of ``input_dist`` runs on
        it with CPU tensors, so it can be issued from a background thread ahead of time without interleaving with the
        device collectives of the running step."""
        super().__init__()
        self.tables, self.env, self.device = list(tables), env, torch.device(device)
        self.world, self.rank, self.pg = env.world_size, env.rank, env.process_group
        self.input_pg = input_env.process_group if input_env is not None else None
        self._prepared: Dict[int, tuple] = {}
        self._pending: Dict[int, list] = {}          # gradient accumulation: table -> [rows, grads, passes]
        self._prefetch_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.opt = optimizer_spec or E.OptimizerSpec()
        self.hashed, self.out_dtype = hashed, out_dtype
        self.feature_names: List[str] = []
        self.feature_table: List[int] = []
        for ti, t in enumerate(tables):
            for f in t.feature_names:
                self.feature_names.append(f)
                self.feature_table.append(ti)
        self.kinds, self.owners = [], []
        for t in tables:
            ps = plan.get(t.name, ParameterSharding("row_wise" if self.world > 1 else "data_parallel"))
            k = E.SH_LOCAL if self.world == 1 else _kind_of(ps)
            if hashed and k not in (E.SH_ROW_MOD, E.SH_LOCAL):
                # the reference's hash tables accept row-wise and data-parallel only
                # (hybrid_torchrec/distributed/hash_embeddingbag.py:148-155)
                raise NotImplementedError("hash embedding tables support row_wise (mod) and data_parallel sharding")
            self.kinds.append(k)
            self.owners.append((ps.ranks[0] if ps.ranks else 0) if k == E.SH_TABLE_WISE else 0)
        self.layout = E.TbeLayout([t.embedding_dim for t in tables], [t.num_embeddings for t in tables], self.kinds,
                                  self.owners, self.world, self.rank, self.feature_table)
        self.embedding_bags = TableDict()
        self.state: List[Dict[str, torch.Tensor]] = []
        for ti, t in enumerate(tables):
            rows = int(self.layout.local_rows[self.rank, ti])
            holder = nn.Module()
            w = nn.Parameter(torch.empty(rows, t.embedding_dim, dtype=data_type_to_dtype(t.data_type), device=self.device),
                             requires_grad=False)
            w._in_backward_optimizers = True  # type: ignore[attr-defined]
            holder.weight = w
            self.embedding_bags[t.name] = holder
            st: Dict[str, torch.Tensor] = {}
            if self.opt.kind == E.OPT_ROWWISE_ADAGRAD:
                st["state1"] = torch.full((rows,), self.opt.initial_accumulator_value, device=self.device)
            elif self.opt.kind == E.OPT_ADAGRAD:
                st["state1"] = torch.full((rows, t.embedding_dim), self.opt.initial_accumulator_value, device=self.device)
            elif self.opt.kind == E.OPT_ADAM:
                st["state1"] = torch.zeros(rows, t.embedding_dim, device=self.device)
                st["state2"] = torch.zeros(rows, t.embedding_dim, device=self.device)
            self.state.append(st)
        self.mappers = [host().IdsMapper(max(1, int(self.layout.local_rows[self.rank, ti]))) for ti in range(len(tables))] \
            if hashed else None
        self._anchor = nn.Parameter(torch.zeros(1, device=self.device))
        self._anchor._in_backward_optimizers = True  # type: ignore[attr-defined]
        self._step = 0
        self._in_pool = ThreadPoolExecutor(max_workers=_env_threads("INPUT_DIST_THREADS"))
        self._post_pool = ThreadPoolExecutor(max_workers=_env_threads("POST_INPUT_THREADS"))
        self.fused_optimizer = FusedOptimizerStub([h.weight for h in self.embedding_bags.values()], self.opt)
        if init_weights:
            self.reset_parameters()

    # ----------------------------------------------------------------- parameters
    @torch.no_grad()
    def reset_parameters(self) -> None:
        for t in self.tables:
            w = self.embedding_bags[t.name].weight
            if w.numel():
                if t.init_fn is not None:
                    t.init_fn(w)
                else:
                    w.uniform_(t.get_weight_init_min(), t.get_weight_init_max())

    def global_rows_of(self, ti: int) -> torch.Tensor:
        n = int(self.layout.local_rows[self.rank, ti])
        r = torch.arange(n, dtype=torch.int64)
        k = self.kinds[ti]
        if k == E.SH_ROW_MOD:
            return r * self.world + self.rank
        if k == E.SH_ROW_BLOCK:
            return r + self.rank * self.layout.blocks[ti]
        return r

    @torch.no_grad()
    def load_from_unsharded(self, ebc: nn.Module) -> None:
        if self.hashed:
            return  # slots are assigned on first sight; nothing to copy
        for ti, t in enumerate(self.tables):
            w = self.embedding_bags[t.name].weight
            if w.numel():
                full = ebc.embedding_bags[t.name].weight.detach()
                w.copy_(full.index_select(0, self.global_rows_of(ti).to(full.device)).to(w.device, w.dtype))

    @torch.no_grad()
    def full_table(self, name: str) -> torch.Tensor:
        ti = [t.name for t in self.tables].index(name)
        t = self.tables[ti]
        w = self.embedding_bags[name].weight.detach().float().cpu()
        rows = self.global_rows_of(ti)
        full = torch.zeros(t.num_embeddings, t.embedding_dim)
        if self.world == 1 or self.kinds[ti] == E.SH_LOCAL:
            full[rows] = w
            return full
        parts = [None] * self.world
        dist.all_gather_object(parts, (rows, w), group=self.pg)
        for r_rows, r_w in parts:
            if r_rows.numel():
                full[r_rows] = r_w
        return full

    def embedding_bag_configs(self) -> List[EmbeddingBagConfig]:
        return self.tables

    def table_weight(self, name: str) -> torch.Tensor:
        return self.embedding_bags[name].weight

    # ----------------------------------------------------------------- input dist
    def _bucketize(self, features: KeyedJaggedTensor):
        """CPU native bucketize: (new_lengths [W, F*B], new_indices, permute).  Table-wise and replicated
        tables are expressed as block sizes so that every id of the feature lands in one bucket."""
        F, B = len(self.feature_names), features.stride()
        lengths = features.lengths().cpu().numpy().astype(np.int64)
        values = features.values().cpu().numpy().astype(np.int64)
        if all(self.kinds[self.feature_table[f]] in (E.SH_ROW_MOD,) for f in range(F)):
            # hash tables keep the raw id (the owner maps it to a slot); plain tables send the local row
            nl, ni, _, perm = host().block_bucketize_sparse_features(lengths, values, None, F, B, self.world, None,
                                                                     not self.hashed)
            return torch.from_numpy(nl).view(self.world, F * B), torch.from_numpy(ni), torch.from_numpy(perm)
        # general case: per-feature destination function evaluated in PyTorch
        off = np.concatenate([[0], np.cumsum(lengths)])
        feat = np.repeat(np.arange(F), [int(off[(f + 1) * B] - off[f * B]) for f in range(F)])
        dest = np.zeros(values.shape[0], dtype=np.int64)
        local = values.copy()
        for f in range(F):
            ti = self.feature_table[f]
            sel = feat == f
            k = self.kinds[ti]
            if k == E.SH_ROW_MOD:
                dest[sel] = values[sel] % self.world
                if not self.hashed:
                    local[sel] = values[sel] // self.world
            elif k == E.SH_ROW_BLOCK:
                blk = self.layout.blocks[ti]
                dest[sel] = np.minimum(values[sel] // blk, self.world - 1)
                local[sel] = values[sel] - dest[sel] * blk
            elif k == E.SH_TABLE_WISE:
                dest[sel] = self.owners[ti]
            else:
                dest[sel] = self.rank
        bag = np.repeat(np.arange(F * B), lengths)
        key = dest * (F * B) + bag
        order = np.argsort(key, kind="stable")
        nl = np.bincount(key, minlength=self.world * F * B).astype(np.int64)
        perm = np.empty_like(order)
        perm[order] = np.arange(order.size)
        return torch.from_numpy(nl).view(self.world, F * B), torch.from_numpy(local[order]), torch.from_numpy(perm)

    def input_dist(self, features: KeyedJaggedTensor):
        """Returns the KJT of ids this rank owns for the global batch: lengths ``[W_src, F, B]`` and ids."""
        assert features.keys() == self.feature_names
        F, B = len(self.feature_names), features.stride()
        new_lengths, new_ids, _perm = self._in_pool.submit(self._bucketize, features).result()
        if self.world == 1:
            return new_lengths.view(1, F, B).to(self.device), new_ids.to(self.device), B
        host_side = self.input_pg is not None
        xdev, xpg = (torch.device("cpu"), self.input_pg) if host_side else (self.device, self.pg)
        send_lengths = new_lengths.to(xdev).contiguous()
        recv_lengths = torch.empty_like(send_lengths)
        dist.all_to_all_single(recv_lengths, send_lengths, group=xpg)              # splits: F*B per rank
        in_splits = new_lengths.sum(dim=1).tolist()
        out_splits = recv_lengths.view(self.world, -1).sum(dim=1).tolist()
        send_ids = new_ids.to(xdev)
        recv_ids = send_ids.new_empty(int(sum(out_splits)))
        dist.all_to_all_single(recv_ids, send_ids, out_splits, in_splits, group=xpg)
        if host_side and not self.hashed:
            recv_lengths, recv_ids = recv_lengths.to(self.device, non_blocking=True), recv_ids.to(self.device, non_blocking=True)
        elif host_side:
            recv_lengths = recv_lengths.to(self.device, non_blocking=True)         # ids stay on the host for the id mapper
        return recv_lengths.view(self.world, F, B), recv_ids, B

    def post_input_dist(self, lengths: torch.Tensor, ids: torch.Tensor):
        """Hash tables: raw ids -> local slots (fused unique + lookup per table, table-parallel when
        ``ENABLE_PARALLEL_GLOBAL_UNIQUE=1``)."""
        if not self.hashed:
            return ids
        W, F, B = lengths.shape
        per_feature = lengths.sum(dim=2)                                 # [W, F]
        ids_np = ids.cpu().numpy().astype(np.int64)
        # positions of each table's ids inside the (source, feature)-major id list
        seg = per_feature.reshape(-1).cpu().numpy()
        seg_off = np.concatenate([[0], np.cumsum(seg)])
        tab_pos: List[List[np.ndarray]] = [[] for _ in self.tables]
        for s in range(W):
            for f in range(F):
                tab_pos[self.feature_table[f]].append(np.arange(seg_off[s * F + f], seg_off[s * F + f + 1]))
        pos = [np.concatenate(p) if p else np.zeros(0, dtype=np.int64) for p in tab_pos]
        per_table = [ids_np[p] for p in pos]
        if os.environ.get("ENABLE_PARALLEL_GLOBAL_UNIQUE", "0") == "1":
            res = self._post_pool.submit(host().parallel_unique_hash_out, self.mappers, per_table).result()
        else:
            res = [self.mappers[t].ids2indices_unique_out(per_table[t]) for t in range(len(self.tables))]
        out = np.empty_like(ids_np)
        for t, p in enumerate(pos):
            out[p] = res[t][0]
        return torch.from_numpy(out).to(ids.device)

    # ----------------------------------------------------------------- compute
    def _allgather_var(self, t: torch.Tensor) -> torch.Tensor:
        """All-gather of tensors whose first dimension differs per rank."""
        n = torch.tensor([t.shape[0]], dtype=torch.int64, device=t.device)
        sizes = [torch.zeros_like(n) for _ in range(self.world)]
        dist.all_gather(sizes, n, group=self.pg)
        sizes = [int(x.item()) for x in sizes]
        cap = max(max(sizes), 1)
        pad = t.new_zeros((cap,) + tuple(t.shape[1:]))
        pad[: t.shape[0]] = t
        outs = [torch.empty_like(pad) for _ in range(self.world)]
        dist.all_gather(outs, pad, group=self.pg)
        return torch.cat([o[:k] for o, k in zip(outs, sizes)])

    def _apply_update(self, ti: int, rows: torch.Tensor, grads: torch.Tensor) -> None:
        self.opt.lr = self.fused_optimizer.param_groups[0]["lr"]
        if self.world > 1 and self.kinds[ti] == E.SH_LOCAL:
            # replicated table: every replica applies the gradient of the global batch
            rows, grads = self._allgather_var(rows), self._allgather_var(grads.contiguous())
        k = max(int(getattr(self.opt, "accumulate_step", 1)), 1)
        if k > 1:
            # gradient accumulation (the reference's GradientAccumulator, hybrid_torchrec/distributed/
            # batched_embedding_kernel.py:111-230): keep the row gradients of k backward passes, then one exact update
            pend = self._pending.setdefault(ti, [[], [], 0])
            pend[0].append(rows)
            pend[1].append(grads.detach().float())
            pend[2] += 1
            if pend[2] < k:
                return
            rows, grads = torch.cat(pend[0]), torch.cat(pend[1])
            self._pending.pop(ti)
        apply_sparse_update(self.embedding_bags[self.tables[ti].name].weight, self.state[ti], rows, grads, self.opt,
                            max(self._step, 1))

    def compute_and_output_dist(self, lengths: torch.Tensor, ids: torch.Tensor, B: int,
                                orig_lengths: Optional[torch.Tensor] = None) -> KeyedTensor:
        self._step += 1
        W, F, _ = lengths.shape
        per_feature = lengths.sum(dim=2).reshape(-1).tolist()
        flat_len = lengths.reshape(W * F, B)
        pooled = []                                   # per feature: [W*B, D]
        chunks = torch.split(ids, per_feature) if ids.numel() else [ids] * (W * F)
        for f in range(F):
            ti = self.feature_table[f]
            t = self.tables[ti]
            rows = torch.cat([chunks[s * F + f] for s in range(W)])
            ln = torch.cat([flat_len[s * F + f] for s in range(W)])
            off = torch.zeros(W * B + 1, dtype=torch.int64, device=ids.device)
            torch.cumsum(ln, 0, out=off[1:])
            # shards pool with SUM; MEAN divides by the full bag length after the reduce below
            pooled.append(_PooledLookup.apply(self._anchor, self, ti, rows, off, False, W * B))
        partial = torch.cat(pooled, dim=1)            # [W*B, total_D], rows grouped by source rank
        if self.world == 1:
            out = partial
        else:
            recv = _AllToAll.apply(partial, [B] * self.world, [B] * self.world, self.pg)
            out = recv.view(self.world, B, -1).sum(dim=0)
        if orig_lengths is not None and any(t.pooling == PoolingType.MEAN for t in self.tables):
            scale = torch.ones(B, out.shape[1], dtype=out.dtype, device=out.device)
            col = 0
            for f in range(F):
                t = self.tables[self.feature_table[f]]
                if t.pooling == PoolingType.MEAN:
                    scale[:, col:col + t.embedding_dim] = 1.0 / orig_lengths[f].clamp(min=1).to(out.dtype)[:, None]
                col += t.embedding_dim
            out = out * scale
        return KeyedTensor(self.feature_names, self.layout.feature_dims, out.to(self.out_dtype))

    # ----------------------------------------------------------------- staged input dist (multi-line host pipeline)
    def stage_split(self, features: KeyedJaggedTensor) -> "DistState":
        """Stage 1 of 5: bucketize the batch's ids by owner rank on the input thread pool (returns at once)."""
        assert features.keys() == self.feature_names
        st = DistState(module=self, features=features, F=len(self.feature_names), B=features.stride())
        st.orig_lengths = features.lengths().view(st.F, st.B)
        st.split_future = self._in_pool.submit(self._bucketize, features)
        return st

    def stage_send_lengths(self, st: "DistState") -> torch.Tensor:
        """The ``[W, F*B]`` lengths this rank sends (waits for the bucketize future)."""
        st.send_lengths, st.send_ids, _ = st.split_future.result()
        st.split_future = None
        return st.send_lengths

    def stage_exchange_ids(self, st: "DistState", recv_lengths: torch.Tensor):
        """Stage 3 of 5: start the id all-to-all on the host process group (asynchronous; ``st.ids_work``)."""
        st.recv_lengths = recv_lengths.view(self.world, -1)
        if self.world == 1:
            st.recv_ids, st.ids_work = st.send_ids, None
            return
        in_splits = st.send_lengths.sum(dim=1).tolist()
        out_splits = st.recv_lengths.sum(dim=1).tolist()
        st.recv_ids = st.send_ids.new_empty(int(sum(out_splits)))
        st.ids_work = dist.all_to_all_single(st.recv_ids, st.send_ids.contiguous(), out_splits, in_splits,
                                             group=self.input_pg if self.input_pg is not None else self.pg, async_op=True)

    def stage_post_input(self, st: "DistState") -> None:
        """Stage 4 of 5: raw ids -> local slots on the post-input pool (hash tables; identity otherwise)."""
        if st.ids_work is not None:
            st.ids_work.wait()
            st.ids_work = None
        lengths3 = st.recv_lengths.view(self.world, st.F, st.B)
        if self.hashed:
            st.post_future = self._post_pool.submit(self.post_input_dist, lengths3, st.recv_ids)
        else:
            st.mapped_ids = st.recv_ids

    def stage_to_device(self, st: "DistState", device_features: KeyedJaggedTensor, stream=None) -> None:
        """Stage 5 of 5: pinned host buffers -> device on ``stream``; registers the result for ``forward``."""
        if st.post_future is not None:
            st.mapped_ids = st.post_future.result()
            st.post_future = None
        cuda = self.device.type == "cuda"

        def up(t: torch.Tensor) -> torch.Tensor:
            if not cuda:
                return t
            return t.pin_memory().to(self.device, non_blocking=True)

        if cuda and stream is not None:
            with torch.cuda.stream(stream):
                lengths, ids, orig = up(st.recv_lengths), up(st.mapped_ids), up(st.orig_lengths)
                ev = torch.cuda.Event()
                ev.record(stream)
        else:
            lengths, ids, orig, ev = up(st.recv_lengths), up(st.mapped_ids), up(st.orig_lengths), None
        self._prepared[id(device_features)] = (lengths.view(self.world, st.F, st.B), ids, st.B, orig, ev)

    # ----------------------------------------------------------------- pipelining
    def _prepare(self, features: KeyedJaggedTensor):
        lengths, ids, B = self.input_dist(features)
        ids = self.post_input_dist(lengths, ids)
        orig = features.lengths().view(len(self.feature_names), B).to(self.device)
        return lengths, ids.to(self.device), B, orig

    def prefetch(self, features: KeyedJaggedTensor) -> None:
        """Run input distribution and id mapping for a batch that ``forward`` will consume later (matched by the
        identity of ``features``).  Device work goes to a side stream; ``forward`` makes the compute stream wait."""
        if self._prefetch_stream is not None:
            self._prefetch_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._prefetch_stream):
                ctx = self._prepare(features)
                ev = torch.cuda.Event()
                ev.record(self._prefetch_stream)
        else:
            ctx, ev = self._prepare(features), None
        self._prepared[id(features)] = ctx + (ev,)

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        ctx = self._prepared.pop(id(features), None)
        if ctx is None:
            lengths, ids, B, orig = self._prepare(features)
        else:
            lengths, ids, B, orig, ev = ctx
            if ev is not None:
                torch.cuda.current_stream(self.device).wait_event(ev)
        return self.compute_and_output_dist(lengths, ids, B, orig)

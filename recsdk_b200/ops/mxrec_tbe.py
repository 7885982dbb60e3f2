"""``torch.ops.mxrec.split_embedding_codegen_lookup_*_function``: the FBGEMM-TBE-shaped training lookups of the reference.

One flat weight buffer holds every table (``weights_offsets[f]`` is the element offset of the table read by feature ``f``,
``D_offsets`` the output columns of each feature, ``hash_size_cumsum`` the running row count of the tables).  The forward is
the pooled (sum / mean) or per-id lookup; the backward sums the output gradient per touched row and applies the optimizer
to ``dev_weights`` and the momentum buffers in place, so no dense weight gradient ever exists
(``cust_op/framework/torch_plugin/torch_library/split_embedding_codegen_forward_unweighted/``:
``backward_codegen_adagrad_unweighted_exact.cpp:45-283``, ``backward_codegen_adam_unweighted_exact.cpp``,
``backward_codegen_sgd_unweighted_exact.cpp``, ``backward_codegen_rowwise_adagrad_unweighted_exact.cpp:411-466``, the
``*_grad_aggregation.cpp`` variants; update formulas: ``ai_core_op/recops_backward_codegen_adagrad_unweighted_exact/v220/
README.md:78-135`` and the Adam / SGD sections after it).

On a GPU, when every table starts on a 16-byte boundary and has a width that is a multiple of 8, the work is done by the
library's fused kernels (``rb_tbe_forward`` and sort + ``rb_tbe_backward_update``: segment sum per unique row and optimizer
in one launch).  Every other case (CPU, odd widths, per-id output, multi-step aggregation, ``use_optimize=False``) runs the
same math as PyTorch index operations.

Multi-step accumulation: with ``use_optimize=False`` the per-row gradient sums are added to ``grad_accumulate[t]`` (one
``[rows_t, D_t]`` fp32 buffer per table) and the weights stay as they are; the next call with ``use_optimize=True`` adds the
stored rows to its own sums, clears them and updates once.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import embedding_ops as E

_SGD, _ROWWISE, _ADAGRAD, _ADAM = E.OPT_SGD, E.OPT_ROWWISE_ADAGRAD, E.OPT_ADAGRAD, E.OPT_ADAM


class _Geometry:
    """Tables and features decoded from the FBGEMM argument list (host integers; cached by the caller's tensors)."""

    def __init__(self, dev_weights, weights_offsets, D_offsets, hash_size_cumsum, rows_per_table) -> None:
        w_off = [int(x) for x in weights_offsets.tolist()]
        d_off = [int(x) for x in D_offsets.tolist()]
        self.F = len(w_off)
        self.feature_dims = [d_off[f + 1] - d_off[f] for f in range(self.F)]
        self.D_offsets = d_off
        self.total_D = d_off[-1]
        starts = sorted(set(w_off))
        self.table_start = starts
        self.feature_table = [starts.index(o) for o in w_off]
        self.n_tables = len(starts)
        self.dims = [0] * self.n_tables
        for f, t in enumerate(self.feature_table):
            self.dims[t] = self.feature_dims[f]
        rows = [0] * self.n_tables
        if rows_per_table is not None:
            rp = [int(x) for x in rows_per_table.tolist()]
            for f, t in enumerate(self.feature_table):
                rows[t] = rp[f] if len(rp) == self.F else rp[t]
        elif hash_size_cumsum is not None and hash_size_cumsum.numel() == self.F + 1:
            hs = [int(x) for x in hash_size_cumsum.tolist()]
            for f, t in enumerate(self.feature_table):
                rows[t] = max(rows[t], hs[f + 1] - hs[f])
        for t in range(self.n_tables):
            if rows[t] <= 0:
                end = starts[t + 1] if t + 1 < self.n_tables else dev_weights.numel()
                rows[t] = (end - starts[t]) // self.dims[t]
        self.rows = rows
        self.row_cumsum = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
        self.packed = all(starts[t] + rows[t] * self.dims[t] == starts[t + 1] for t in range(self.n_tables - 1)) and starts[0] == 0

    def table_view(self, flat: torch.Tensor, t: int, offsets: Optional[Sequence[int]] = None) -> torch.Tensor:
        s = self.table_start[t] if offsets is None else int(offsets[t])
        return flat[s: s + self.rows[t] * self.dims[t]].view(self.rows[t], self.dims[t])


def _forward(geo: _Geometry, dev_weights, idx, offsets, pooling_mode: int, max_D: int, out_dtype=torch.float32):
    B = (offsets.numel() - 1) // geo.F
    tables = [geo.table_view(dev_weights, t) for t in geo.feature_table]
    if pooling_mode == 2:
        off = offsets.tolist()
        out = torch.zeros(idx.numel(), max_D, dtype=out_dtype, device=dev_weights.device)
        for f in range(geo.F):
            a, b = off[f * B], off[(f + 1) * B]
            out[a:b, : geo.feature_dims[f]] = tables[f][idx[a:b]].to(out_dtype)
        return out
    if _cuda_ok(geo, dev_weights) and out_dtype in (torch.float32, torch.float16, torch.bfloat16):
        layout, dev = _cuda_layout(geo, dev_weights)
        out = torch.empty(B, geo.total_D, dtype=out_dtype, device=dev_weights.device)
        E.tbe_forward(layout, dev, idx, offsets, B, pooling_mode, dev_weights.dtype, out)
        return out
    lengths = (offsets[1:] - offsets[:-1]).long()
    bag_of = torch.repeat_interleave(torch.arange(geo.F * B, device=idx.device), lengths)
    off = offsets.tolist()
    out = torch.zeros(B, geo.total_D, dtype=torch.float32, device=dev_weights.device)
    for f in range(geo.F):
        a, b = off[f * B], off[(f + 1) * B]
        if a == b:
            continue
        rows = tables[f][idx[a:b].long()].float()
        if pooling_mode == 1:
            rows = rows / lengths[bag_of[a:b]].clamp(min=1).float()[:, None]
        out[:, geo.D_offsets[f]: geo.D_offsets[f + 1]].index_add_(0, bag_of[a:b] - f * B, rows)
    return out.to(out_dtype)


# ------------------------------------------------------------------------------------------------ fused GPU path
_LAYOUTS: Dict[Tuple, Tuple] = {}
_WORK: Dict[Tuple, Tuple] = {}


def _cuda_ok(geo: _Geometry, dev_weights: torch.Tensor) -> bool:
    item = dev_weights.element_size()
    return (dev_weights.is_cuda and dev_weights.dtype in (torch.float16, torch.bfloat16, torch.float32)
            and all(d % 8 == 0 for d in geo.dims) and all((s * item) % 16 == 0 for s in geo.table_start)
            and dev_weights.data_ptr() % 16 == 0)


def _cuda_layout(geo: _Geometry, dev_weights: torch.Tensor):
    """Single-rank ``TbeLayout`` over the caller's buffer; the pointer and offset tables follow ``weights_offsets`` so gaps
    between tables are allowed."""
    key = (dev_weights.data_ptr(), dev_weights.device.index, tuple(geo.table_start), tuple(geo.rows), tuple(geo.feature_table),
           tuple(geo.dims))
    hit = _LAYOUTS.get(key)
    if hit is None:
        layout = E.TbeLayout(geo.dims, geo.rows, [E.SH_LOCAL] * geo.n_tables, [0] * geo.n_tables, 1, 0, geo.feature_table)
        dev = layout.device_tensors(dev_weights.device, [dev_weights.data_ptr()], dev_weights.element_size())
        item = dev_weights.element_size()
        ptrs = np.asarray([dev_weights.data_ptr() + s * item for s in geo.table_start], dtype=np.int64)
        dev["ptrs"] = torch.from_numpy(ptrs).to(dev_weights.device)
        dev["w_offsets"] = torch.tensor(geo.table_start, dtype=torch.int64, device=dev_weights.device)
        if len(_LAYOUTS) > 64:
            _LAYOUTS.clear()
        hit = _LAYOUTS[key] = (layout, dev)
    return hit


def _workspace(device: torch.device, nnz: int, max_D: int):
    cap = max(1024, 1 << (int(nnz) - 1).bit_length())
    key = (device.index, max_D)
    hit = _WORK.get(key)
    if hit is None or hit[0] < cap:
        hit = _WORK[key] = (cap, E.SegmentSorter(cap, device), E.BackwardWorkspace(device, cap, max_D))
    return hit[1], hit[2]


def _table_offsets(geo: _Geometry, per_feature: torch.Tensor) -> List[int]:
    """FBGEMM passes state offsets per feature; the kernels want them per table."""
    vals = [int(x) for x in per_feature.tolist()]
    if len(vals) == geo.n_tables and geo.n_tables != geo.F:
        return vals
    out = [0] * geo.n_tables
    for f, t in enumerate(geo.feature_table):
        out[t] = vals[f]
    return out


def _backward_cuda(geo, grad, dev_weights, idx, offsets, pooling_mode, kind, m1, m1_off, m2, hp) -> None:
    layout, dev = _cuda_layout(geo, dev_weights)
    B = (offsets.numel() - 1) // geo.F
    sorter, ws = _workspace(dev_weights.device, idx.numel(), layout.max_D)
    seg = sorter.run(layout, dev, idx, offsets, B)
    g = grad if grad.is_contiguous() else grad.contiguous()
    ptrs = torch.tensor([g.data_ptr()], dtype=torch.int64, device=g.device)
    if m1_off is not None:
        s_off = torch.tensor(_table_offsets(geo, m1_off), dtype=torch.int64, device=g.device)
    elif kind == _ROWWISE:
        s_off = torch.from_numpy(geo.row_cumsum[:-1].copy()).to(g.device)
    else:
        s_off = dev["w_offsets"]
    opt = E.OptimizerSpec(kind=kind, lr=hp["lr"], eps=hp.get("eps", 0.0), beta1=hp.get("beta1", 0.9), beta2=hp.get("beta2", 0.999),
                          weight_decay=hp.get("weight_decay", 0.0) if kind == _SGD else 0.0)
    E.tbe_backward_update(layout, dev, seg, ptrs, g.stride(0), g.dtype, B, offsets, pooling_mode, dev_weights, m1, m2, s_off, opt,
                          max(int(hp.get("iter", 1)), 1), ws)


# ------------------------------------------------------------------------------------------------ PyTorch statement
def row_gradients(geo: _Geometry, grad, idx, offsets, pooling_mode: int):
    """Per table: ``(unique_rows, summed_grad[len(unique_rows), D_t])`` in fp32 (``None`` for tables no id touches)."""
    B = (offsets.numel() - 1) // geo.F
    lengths = (offsets[1:] - offsets[:-1]).long()
    bag_of = torch.repeat_interleave(torch.arange(geo.F * B, device=idx.device), lengths)            # [nnz]
    off = offsets.tolist()
    per_table: List[List[Tuple[torch.Tensor, torch.Tensor]]] = [[] for _ in range(geo.n_tables)]
    for f, t in enumerate(geo.feature_table):
        a, b = off[f * B], off[(f + 1) * B]
        if a == b:
            continue
        if pooling_mode == 2:
            g = grad[a:b, : geo.feature_dims[f]].float()
        else:
            bags = bag_of[a:b]
            g = grad[bags - f * B, geo.D_offsets[f]: geo.D_offsets[f + 1]].float()
            if pooling_mode == 1:
                g = g / lengths[bags].clamp(min=1).float()[:, None]
        per_table[t].append((idx[a:b].long(), g))
    out: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = []
    for t in range(geo.n_tables):
        if not per_table[t]:
            out.append(None)
            continue
        ids = torch.cat([p[0] for p in per_table[t]])
        gs = torch.cat([p[1] for p in per_table[t]])
        uniq, inv = torch.unique(ids, return_inverse=True)
        acc = torch.zeros(uniq.numel(), geo.dims[t], dtype=torch.float32, device=grad.device)
        acc.index_add_(0, inv, gs)
        out.append((uniq, acc))
    return out


def apply_rows(kind: int, w: torch.Tensor, rows: torch.Tensor, g: torch.Tensor, m1, m2, hp) -> None:
    """Update ``w[rows]`` (a ``[rows_t, D]`` view of the flat buffer) with the summed gradients ``g``; ``m1`` / ``m2`` are views
    of the momentum buffers with the same leading dimension."""
    lr, eps = hp["lr"], hp.get("eps", 0.0)
    wr = w[rows].float()
    if kind == _SGD:
        wr = wr - lr * (g + hp.get("weight_decay", 0.0) * wr)
    elif kind == _ROWWISE:
        st = m1[rows].float() + (g * g).mean(dim=1)
        m1[rows] = st.to(m1.dtype)
        wr = wr - (lr / (st.sqrt() + eps))[:, None] * g
    elif kind == _ADAGRAD:
        st = m1[rows].float() + g * g
        m1[rows] = st.to(m1.dtype)
        wr = wr - lr * g / (st.sqrt() + eps)
    else:
        b1, b2, it = hp["beta1"], hp["beta2"], max(int(hp.get("iter", 1)), 1)
        a = b1 * m1[rows].float() + (1 - b1) * g
        v = b2 * m2[rows].float() + (1 - b2) * g * g
        m1[rows], m2[rows] = a.to(m1.dtype), v.to(m2.dtype)
        wr = wr - lr * (a / (1 - b1 ** it)) / ((v / (1 - b2 ** it)).sqrt() + eps)
    w[rows] = wr.to(w.dtype)


def _state_view(geo: _Geometry, kind: int, buf: Optional[torch.Tensor], offs: Optional[List[int]], t: int):
    if buf is None or kind == _SGD:
        return None
    s = geo.table_start[t] if offs is None else offs[t]
    if kind == _ROWWISE:
        s = int(geo.row_cumsum[t]) if offs is None else offs[t]
        return buf[s: s + geo.rows[t]]
    return buf[s: s + geo.rows[t] * geo.dims[t]].view(geo.rows[t], geo.dims[t])


def _backward_torch(geo, grad, dev_weights, idx, offsets, pooling_mode, kind, m1, m1_off, m2, m2_off, hp, grad_accumulate,
                    use_optimize: bool):
    sums = row_gradients(geo, grad, idx, offsets, pooling_mode)
    o1 = None if m1_off is None else _table_offsets(geo, m1_off)
    o2 = None if m2_off is None else _table_offsets(geo, m2_off)
    for t, item in enumerate(sums):
        acc_buf = None
        if grad_accumulate is not None and t < len(grad_accumulate) and grad_accumulate[t].numel() >= geo.rows[t] * geo.dims[t]:
            acc_buf = grad_accumulate[t].view(-1)[: geo.rows[t] * geo.dims[t]].view(geo.rows[t], geo.dims[t])
        if not use_optimize:
            if item is not None and acc_buf is not None:
                acc_buf.index_add_(0, item[0], item[1].to(acc_buf.dtype))
            continue
        if acc_buf is not None:
            pending = torch.nonzero(acc_buf.abs().sum(dim=1) > 0).flatten()
            if pending.numel():
                rows_now = pending if item is None else torch.unique(torch.cat([pending, item[0]]))
                g = acc_buf[rows_now].float()
                if item is not None:
                    g[torch.searchsorted(rows_now, item[0])] += item[1]
                acc_buf[pending] = 0
                item = (rows_now, g)
        if item is None:
            continue
        apply_rows(kind, geo.table_view(dev_weights, t), item[0], item[1], _state_view(geo, kind, m1, o1, t),
                   _state_view(geo, kind, m2, o2, t), hp)
    return sums


# ------------------------------------------------------------------------------------------------ autograd + schemas
def _hyper(kind: int, kw: dict) -> dict:
    hp = {"lr": float(kw.get("learning_rate", 0.0)), "eps": float(kw.get("eps", 0.0)), "iter": int(kw.get("iter", 1) or 1)}
    if kind == _ADAM:
        hp.update(beta1=float(kw.get("beta1", 0.0)), beta2=float(kw.get("beta2", 0.0)))
    return hp


def backward_update(kind: int, grad_output: torch.Tensor, kw: dict) -> List[Optional[Tuple[torch.Tensor, torch.Tensor]]]:
    """Shared body of the autograd backward and of the raw ``split_embedding_backward_codegen_*`` ops.  Returns the per-table
    row gradients when the PyTorch statement ran (``[]`` after the fused kernels, which never materialise them)."""
    dev_weights = kw["dev_weights"]
    geo = _Geometry(dev_weights, kw["weights_offsets"], kw["D_offsets"], kw.get("hash_size_cumsum"), kw.get("rows_per_table"))
    idx = kw["hash_indices"] if kw.get("hash_indices") is not None else kw["indices"]
    offsets = kw["offsets"].long()
    use_optimize = bool(kw.get("use_optimize", True))
    acc = kw.get("grad_accumulate")
    acc = acc if acc else None
    m1, m2 = kw.get("momentum1_dev"), kw.get("momentum2_dev")
    m1_off, m2_off = kw.get("momentum1_offsets"), kw.get("momentum2_offsets")
    hp = _hyper(kind, kw)
    same_state = m2_off is None or m1_off is None or torch.equal(m1_off.cpu(), m2_off.cpu())
    states_fp32 = all(x is None or x.dtype == torch.float32 for x in (m1, m2))
    if (use_optimize and acc is None and kw["pooling_mode"] != 2 and _cuda_ok(geo, dev_weights) and same_state and states_fp32
            and grad_output.dtype in (torch.float32, torch.float16, torch.bfloat16) and not kw.get("_want_rows", False)):
        _backward_cuda(geo, grad_output, dev_weights, idx, offsets, kw["pooling_mode"], kind,
                       None if kind == _SGD else m1, None if kind == _SGD else m1_off, m2 if kind == _ADAM else None, hp)
        return []
    return _backward_torch(geo, grad_output, dev_weights, idx.long(), offsets, kw["pooling_mode"], kind, m1, m1_off, m2, m2_off, hp,
                           acc, use_optimize)


class _Lookup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, placeholder, kind: int, kw: dict):
        dev_weights = kw["dev_weights"]
        geo = _Geometry(dev_weights, kw["weights_offsets"], kw["D_offsets"], kw.get("hash_size_cumsum"), kw.get("rows_per_table"))
        idx = kw["hash_indices"] if kw.get("hash_indices") is not None else kw["indices"]
        ctx.kind, ctx.kw = kind, kw
        out_dtype = {0: torch.float32, 1: torch.float16, 5: torch.bfloat16}.get(int(kw.get("output_dtype", 0)), torch.float32)
        return _forward(geo, dev_weights, idx, kw["offsets"].long(), int(kw["pooling_mode"]), int(kw["max_D"]), out_dtype)

    @staticmethod
    def backward(ctx, grad_output):
        # aggregation variants: the rows of earlier steps are found through their non-zero sums in ``grad_accumulate``, so the
        # ``*_multi_step`` id lists are not needed
        with torch.no_grad():
            backward_update(ctx.kind, grad_output, ctx.kw)
        return None, None, None


_COMMON_HEAD = ("Tensor placeholder_autograd_tensor, Tensor(a!) dev_weights, Tensor(b!) uvm_weights, Tensor lxu_cache_weights, "
                "Tensor weights_placements, Tensor weights_offsets, Tensor D_offsets, SymInt total_D, SymInt max_D, "
                "Tensor hash_size_cumsum, int total_hash_size_bits, Tensor indices, Tensor offsets, {multi}int pooling_mode, "
                "Tensor? indice_weights, Tensor? feature_requires_grad, Tensor lxu_cache_locations, bool gradient_clipping, "
                "float max_gradient, bool stochastic_rounding, ")
_M1 = "Tensor momentum1_dev, Tensor momentum1_uvm, Tensor momentum1_placements, Tensor momentum1_offsets, "
_M2 = "Tensor momentum2_dev, Tensor momentum2_uvm, Tensor momentum2_placements, Tensor momentum2_offsets, "
_UNIQ = ("Tensor[]? grad_accumulate=None, Tensor? grad_accumulate_offsets=None, Tensor? hash_indices=None, Tensor? unique_ids=None, "
         "Tensor? unique_offsets=None, Tensor? unique_inverse=None, Tensor? table_grad_accumulate_offsets=None, ")
_UNIQ_MULTI = ("Tensor? table_offsets_multi=None, Tensor? unique_multi_step=None, Tensor? unique_offset_multi_step=None, "
               "Tensor? unique_inverse_multi_step=None, ")
_VBE = ("int output_dtype=0, Tensor? B_offsets=None, Tensor? vbe_output_offsets_feature_rank=None, "
        "Tensor? vbe_B_offsets_rank_per_feature=None, SymInt max_B=-1, SymInt max_B_feature_rank=-1, SymInt vbe_output_size=-1, "
        "bool is_experimental=False, bool use_uniq_cache_locations_bwd=False, bool use_homogeneous_placements=False, "
        "Tensor? uvm_cache_stats=None, Tensor? prev_iter_dev=None, ")
_TAIL = "bool apply_global_weight_decay=False, float gwd_lower_bound=0, bool use_optimize=True, Tensor? rows_per_table=None"


def lookup_schemas() -> Dict[str, Tuple[int, str]]:
    """name -> (optimizer kind, schema); argument order as in the reference's ``m.def`` strings."""
    out: Dict[str, Tuple[int, str]] = {}
    for agg in (False, True):
        sfx = "_grad_aggregation" if agg else ""
        head = _COMMON_HEAD.format(multi="Tensor indices_multi_step, Tensor offsets_multi_step, " if agg else "")
        uniq = _UNIQ + (_UNIQ_MULTI if agg else "")
        out["split_embedding_codegen_lookup_adagrad_function" + sfx] = (
            _ADAGRAD, head + _M1 + uniq + "float eps=0, float learning_rate=0, " + _VBE + "int iter=0, " + _TAIL)
        out["split_embedding_codegen_lookup_adam_function" + sfx] = (
            _ADAM, head + _M1 + _M2 + uniq + "float eps=0, float learning_rate=0, float beta1=0, float beta2=0, float weight_decay=0, "
            "int iter=0, " + _VBE + _TAIL)
        out["split_embedding_codegen_lookup_sgd_function" + sfx] = (
            _SGD, head + uniq + "float learning_rate=0, " + _VBE + "int iter=0, " + _TAIL)
    out["split_embedding_codegen_lookup_rowwise_adagrad_function"] = (
        _ROWWISE, _COMMON_HEAD.format(multi="") + _M1 + "float eps=0, float learning_rate=0, float weight_decay=0.0, "
        "int weight_decay_mode=0, float max_norm=0.0, " + _VBE + "int iter=0, bool apply_global_weight_decay=False, "
        "float gwd_lower_bound=0, bool mixed_D=True, " + _UNIQ + "Tensor? rows_per_table=None")
    return out


def _arg_names(schema_args: str) -> List[str]:
    return [a.strip().split("=")[0].split()[-1] for a in schema_args.split(",")]


def make_lookup(kind: int, schema_args: str):
    names = _arg_names(schema_args)

    def fn(*args):
        kw = dict(zip(names, args))
        return _Lookup.apply(kw["placeholder_autograd_tensor"], kind, kw)

    return fn


_RAW_HEAD = ("Tensor grad_output, Tensor(a!) dev_weights, Tensor(b!) uvm_weights, Tensor lxu_cache_weights, Tensor weights_placements, "
             "Tensor weights_offsets, Tensor D_offsets, SymInt max_D, Tensor hash_size_cumsum, int total_hash_size_bits, Tensor indices, "
             "Tensor offsets, {multi}int pooling_mode, Tensor lxu_cache_locations, int unused_, int max_segment_length_per_warp, "
             "bool stochastic_rounding, int info_B_num_bits, int info_B_mask_int64, bool use_uniq_cache_locations, "
             "bool use_homogeneous_placements, ")
_RAW_UNIQ = ("Tensor[] grad_accumulate, Tensor grad_accumulate_offsets, Tensor? hash_indices=None, Tensor? unique_ids=None, "
             "Tensor? unique_offsets=None, Tensor? unique_inverse=None, Tensor? offset_per_key=None, "
             "Tensor? table_grad_accumulate_offsets=None, ")


def raw_backward_schemas() -> Dict[str, Tuple[int, str]]:
    """name -> (optimizer kind, schema).  The ``*_grad_aggregation`` forms carry the id lists of the accumulated steps and
    their unique results (``backward_codegen_{adagrad,adam,sgd}_unweighted_exact_grad_aggregation.cpp`` of the reference); the
    rows of earlier steps are found through their non-zero sums in ``grad_accumulate``, so those lists are accepted and unused."""
    out: Dict[str, Tuple[int, str]] = {}
    for agg in (False, True):
        sfx = "_grad_aggregation" if agg else ""
        head = _RAW_HEAD.format(multi="Tensor indices_multi_step, Tensor offsets_multi_step, " if agg else "")
        uniq = _RAW_UNIQ + (_UNIQ_MULTI if agg else "")
        out["split_embedding_backward_codegen_adagrad_unweighted_exact_cuda" + sfx] = (
            _ADAGRAD, head + _M1 + uniq + "float eps=0, float learning_rate=0, bool use_optimize=True")
        out["split_embedding_backward_codegen_adam_unweighted_exact_cuda" + sfx] = (
            _ADAM, head + _M1 + _M2 + uniq + "float eps=0, float learning_rate=0, float beta1=0, float beta2=0, int iter=0, "
            "bool use_optimize=True")
        out["split_embedding_backward_codegen_sgd_unweighted_exact_cuda" + sfx] = (
            _SGD, head + uniq + "float learning_rate=0, bool use_optimize=True")
    out["split_embedding_backward_codegen_rowwise_adagrad_unweighted_exact_cuda"] = (
        _ROWWISE, _RAW_HEAD.format(multi="") + _M1 + _RAW_UNIQ + "float eps=0, float learning_rate=0, bool use_optimize=True")
    return out


def make_raw_backward(kind: int, schema_args: str):
    """Returns the summed row gradients: ``[len(unique_ids), max_D]`` in the caller's unique order when ``unique_ids`` is given
    (table-major, ``unique_offsets[t]`` the start of table ``t``), else a dense gradient the size of ``dev_weights``."""
    names = _arg_names(schema_args)

    def fn(*args):
        kw = dict(zip(names, args))
        kw["_want_rows"] = True
        dev_weights = kw["dev_weights"]
        geo = _Geometry(dev_weights, kw["weights_offsets"], kw["D_offsets"], kw.get("hash_size_cumsum"), None)
        sums = backward_update(kind, kw["grad_output"], kw)
        max_D = int(kw["max_D"])
        uniq = kw.get("unique_ids")
        if uniq is not None and uniq.numel():
            out = torch.zeros(uniq.numel(), max_D, dtype=torch.float32, device=dev_weights.device)
            uo = kw["unique_offsets"].tolist()
            for t, item in enumerate(sums):
                if item is None:
                    continue
                seg = uniq[uo[t]: uo[t + 1]].long()
                order = torch.argsort(seg)
                pos = order[torch.searchsorted(seg[order], item[0])] + uo[t]
                out[pos, : geo.dims[t]] = item[1]
            return out
        out = torch.zeros(dev_weights.numel(), dtype=torch.float32, device=dev_weights.device)
        for t, item in enumerate(sums):
            if item is not None:
                geo.table_view(out, t)[item[0]] = item[1]
        return out

    return fn

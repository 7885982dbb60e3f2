"""Invokers of the table-batched training lookups: argument records -> ``torch.ops.mxrec.split_embedding_codegen_lookup_*``.

The reference's batched-embedding module does not call its lookup operators directly; it fills ``HybridCommonArgs`` (the flat
weight buffer and its layout, the batch, and the host-computed ``hash_indices`` / ``unique_*`` tensors that replace the raw
ids), an ``OptimizerArgs`` record and ``Momentum`` records, and hands them to ``lookup_adagrad.invoke`` /
``lookup_adam.invoke`` / ``lookup_sgd.invoke`` or their ``invoke_grad_aggregation`` forms
(``hybrid_torchrec/hybrid_lookup_invoke/hybrid_lookup_{args,adagrad,adam,sgd}.py``).  The same records and entry points are
kept here for code written against that layer; the operators behind them are this package's (``ops/mxrec_tbe.py``).
Weights live in one device buffer in this package, so the host-weights branch of the reference's invokers has no
counterpart: a non-empty ``host_weights`` is refused.
"""
from __future__ import annotations

import dataclasses
import types
from typing import Any, Dict, List, Optional

import torch

from . import mxrec_tbe  # noqa: F401  (registers the operators)


@dataclasses.dataclass
class VBEMetadata:
    B_offsets: Optional[torch.Tensor] = None
    output_offsets_feature_rank: Optional[torch.Tensor] = None
    B_offsets_rank_per_feature: Optional[torch.Tensor] = None
    max_B: int = -1
    max_B_feature_rank: int = -1
    output_size: int = -1


@dataclasses.dataclass
class Momentum:
    dev: torch.Tensor
    host: torch.Tensor
    uvm: torch.Tensor
    offsets: torch.Tensor
    placements: torch.Tensor


@dataclasses.dataclass
class OptimizerArgs:
    stochastic_rounding: bool = False
    gradient_clipping: bool = False
    max_gradient: float = 1.0
    max_norm: float = 0.0
    learning_rate: float = 0.01
    eps: float = 1e-8
    beta1: float = 0.9
    beta2: float = 0.999
    weight_decay: float = 0.0
    weight_decay_mode: int = 0
    eta: float = 0.0
    momentum: float = 0.0
    counter_halflife: int = -1
    adjustment_iter: int = -1
    adjustment_ub: float = 1.0
    learning_rate_mode: int = -1
    grad_sum_decay: int = -1
    tail_id_threshold: float = 0.0
    is_tail_id_thresh_ratio: int = 0
    total_hash_size: int = 0
    weight_norm_coefficient: float = 0.0
    lower_bound: float = 0.0
    regularization_mode: int = 0


@dataclasses.dataclass
class HybridCommonArgs:
    placeholder_autograd_tensor: torch.Tensor
    dev_weights: torch.Tensor
    host_weights: torch.Tensor
    uvm_weights: torch.Tensor
    lxu_cache_weights: torch.Tensor
    weights_placements: torch.Tensor
    weights_offsets: torch.Tensor
    D_offsets: torch.Tensor
    total_D: int
    max_D: int
    hash_size_cumsum: torch.Tensor
    rows_per_table: Optional[torch.Tensor]
    total_hash_size_bits: int
    indices: torch.Tensor
    offsets: torch.Tensor
    hash_indices: Optional[torch.Tensor]
    unique_indices: Optional[torch.Tensor]
    unique_offset: Optional[torch.Tensor]
    unique_inverse: Optional[torch.Tensor]
    hash_indices2address: Optional[torch.Tensor]
    pooling_mode: int
    indice_weights: Optional[torch.Tensor]
    feature_requires_grad: Optional[torch.Tensor]
    lxu_cache_locations: torch.Tensor
    uvm_cache_stats: Optional[torch.Tensor]
    output_dtype: int
    vbe_metadata: VBEMetadata
    is_experimental: bool
    use_uniq_cache_locations_bwd: bool
    use_homogeneous_placements: bool
    learning_rate: float
    table_grad_accumulate_offsets: Optional[torch.Tensor]
    grad_accumulate: Optional[List[torch.Tensor]]
    grad_accumulate_offsets: Optional[torch.Tensor]
    use_optimize: bool


@dataclasses.dataclass
class HybridCommonArgsAggregation(HybridCommonArgs):
    table_offsets_multi: Optional[torch.Tensor] = None
    indices_multi_step: Optional[torch.Tensor] = None
    offsets_multi_step: Optional[torch.Tensor] = None
    unique_multi_step: Optional[torch.Tensor] = None
    unique_offset_multi_step: Optional[torch.Tensor] = None
    unique_inverse_multi_step: Optional[torch.Tensor] = None


def check_unique_valid(common_args: HybridCommonArgs) -> None:
    """``unique_indices[unique_offset[t] + unique_inverse[j]]`` must give back ``hash_indices[j]`` for every id ``j`` of every
    table ``t`` (a debugging aid of the reference, ``hybrid_lookup_adagrad.py:22-49``)."""
    a = common_args
    if a.hash_indices is None or a.unique_indices is None:
        return
    offsets, uo = a.offsets.cpu(), a.unique_offset.cpu()
    B = (offsets.numel() - 1) // a.weights_offsets.numel()
    uniq, inv, parts = a.unique_indices.cpu(), a.unique_inverse.cpu(), []
    for t in range(uo.numel() - 1):
        lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
        parts.append(uniq[int(uo[t]):].index_select(0, inv[lo:hi]))
    if not bool((torch.cat(parts) == a.hash_indices.cpu()).all()):
        raise RuntimeError("unique_indices / unique_offset / unique_inverse do not reproduce hash_indices")


def _learning_rate(a: HybridCommonArgs, o: OptimizerArgs) -> float:
    lr = getattr(a, "learning_rate", None)
    return float(o.learning_rate if lr is None else lr)


def _common_kwargs(a: HybridCommonArgs, o: OptimizerArgs, iteration: int) -> Dict[str, Any]:
    if a.host_weights is not None and a.host_weights.numel() > 0:
        raise NotImplementedError("weights live in one device buffer here: host_weights must be empty")
    v = a.vbe_metadata or VBEMetadata()
    return dict(
        placeholder_autograd_tensor=a.placeholder_autograd_tensor, dev_weights=a.dev_weights, uvm_weights=a.uvm_weights,
        lxu_cache_weights=a.lxu_cache_weights, weights_placements=a.weights_placements, weights_offsets=a.weights_offsets,
        D_offsets=a.D_offsets, total_D=a.total_D, max_D=a.max_D, hash_size_cumsum=a.hash_size_cumsum, rows_per_table=a.rows_per_table,
        total_hash_size_bits=a.total_hash_size_bits, indices=a.hash_indices if a.hash_indices is not None else a.indices,
        offsets=a.offsets, hash_indices=a.hash_indices, unique_ids=a.unique_indices, unique_offsets=a.unique_offset,
        unique_inverse=a.unique_inverse, pooling_mode=a.pooling_mode, indice_weights=a.indice_weights,
        feature_requires_grad=a.feature_requires_grad, lxu_cache_locations=a.lxu_cache_locations, uvm_cache_stats=a.uvm_cache_stats,
        B_offsets=v.B_offsets, vbe_output_offsets_feature_rank=v.output_offsets_feature_rank,
        vbe_B_offsets_rank_per_feature=v.B_offsets_rank_per_feature, max_B=v.max_B, max_B_feature_rank=v.max_B_feature_rank,
        vbe_output_size=v.output_size, gradient_clipping=o.gradient_clipping, max_gradient=o.max_gradient,
        stochastic_rounding=o.stochastic_rounding, learning_rate=_learning_rate(a, o), iter=int(iteration), output_dtype=a.output_dtype,
        is_experimental=a.is_experimental, use_uniq_cache_locations_bwd=a.use_uniq_cache_locations_bwd,
        use_homogeneous_placements=a.use_homogeneous_placements, use_optimize=a.use_optimize, grad_accumulate=a.grad_accumulate,
        grad_accumulate_offsets=a.grad_accumulate_offsets, table_grad_accumulate_offsets=a.table_grad_accumulate_offsets)


def _aggregation_kwargs(a: HybridCommonArgsAggregation) -> Dict[str, Any]:
    return dict(table_offsets_multi=a.table_offsets_multi, indices_multi_step=a.indices_multi_step, offsets_multi_step=a.offsets_multi_step,
                unique_multi_step=a.unique_multi_step, unique_offset_multi_step=a.unique_offset_multi_step,
                unique_inverse_multi_step=a.unique_inverse_multi_step)


def _momentum_kwargs(i: int, m: Momentum) -> Dict[str, Any]:
    return {"momentum%d_dev" % i: m.dev, "momentum%d_uvm" % i: m.uvm, "momentum%d_offsets" % i: m.offsets,
            "momentum%d_placements" % i: m.placements}


def _adagrad(common_args, optimizer_args, momentum1, iteration=0, apply_global_weight_decay=False, prev_iter_dev=None,
             gwd_lower_bound=0.0) -> torch.Tensor:
    kw = _common_kwargs(common_args, optimizer_args, iteration)
    kw.update(_momentum_kwargs(1, momentum1), eps=optimizer_args.eps, prev_iter_dev=prev_iter_dev,
              apply_global_weight_decay=apply_global_weight_decay, gwd_lower_bound=gwd_lower_bound)
    return torch.ops.mxrec.split_embedding_codegen_lookup_adagrad_function(**kw)


def _adagrad_agg(common_args, optimizer_args, momentum1, iteration=0, apply_global_weight_decay=False, prev_iter_dev=None,
                 gwd_lower_bound=0.0) -> torch.Tensor:
    kw = _common_kwargs(common_args, optimizer_args, iteration)
    kw.update(_momentum_kwargs(1, momentum1), eps=optimizer_args.eps, prev_iter_dev=prev_iter_dev,
              apply_global_weight_decay=apply_global_weight_decay, gwd_lower_bound=gwd_lower_bound, **_aggregation_kwargs(common_args))
    return torch.ops.mxrec.split_embedding_codegen_lookup_adagrad_function_grad_aggregation(**kw)


def _adam_kwargs(common_args, optimizer_args, momentum1, momentum2, iteration) -> Dict[str, Any]:
    kw = _common_kwargs(common_args, optimizer_args, iteration)
    kw.update(_momentum_kwargs(1, momentum1), **_momentum_kwargs(2, momentum2), eps=optimizer_args.eps, beta1=optimizer_args.beta1,
              beta2=optimizer_args.beta2, weight_decay=optimizer_args.weight_decay)
    return kw


def _adam(common_args, optimizer_args, momentum1, momentum2, iteration=0, **_unused) -> torch.Tensor:
    return torch.ops.mxrec.split_embedding_codegen_lookup_adam_function(**_adam_kwargs(common_args, optimizer_args, momentum1, momentum2, iteration))


def _adam_agg(common_args, optimizer_args, momentum1, momentum2, iteration=0, **_unused) -> torch.Tensor:
    kw = _adam_kwargs(common_args, optimizer_args, momentum1, momentum2, iteration)
    kw.update(_aggregation_kwargs(common_args))
    return torch.ops.mxrec.split_embedding_codegen_lookup_adam_function_grad_aggregation(**kw)


def _sgd(common_args, optimizer_args, iteration=0, **_unused) -> torch.Tensor:
    return torch.ops.mxrec.split_embedding_codegen_lookup_sgd_function(**_common_kwargs(common_args, optimizer_args, iteration))


def _sgd_agg(common_args, optimizer_args, iteration=0, **_unused) -> torch.Tensor:
    kw = _common_kwargs(common_args, optimizer_args, iteration)
    kw.update(_aggregation_kwargs(common_args))
    return torch.ops.mxrec.split_embedding_codegen_lookup_sgd_function_grad_aggregation(**kw)


# the reference's sub-modules, as namespaces: ``lookup_adagrad.invoke(...)``, ``lookup_adagrad.invoke_grad_aggregation(...)`` etc.
lookup_adagrad = types.SimpleNamespace(invoke=_adagrad, invoke_grad_aggregation=_adagrad_agg, check_unique_valid=check_unique_valid)
lookup_adam = types.SimpleNamespace(invoke=_adam, invoke_grad_aggregation=_adam_agg)
lookup_sgd = types.SimpleNamespace(invoke=_sgd, invoke_grad_aggregation=_sgd_agg)
lookup_args = types.SimpleNamespace(HybridCommonArgs=HybridCommonArgs, HybridCommonArgsAggregation=HybridCommonArgsAggregation,
                                    OptimizerArgs=OptimizerArgs, Momentum=Momentum, VBEMetadata=VBEMetadata)

__all__ = ["VBEMetadata", "Momentum", "OptimizerArgs", "HybridCommonArgs", "HybridCommonArgsAggregation", "check_unique_valid",
           "lookup_adagrad", "lookup_adam", "lookup_sgd", "lookup_args"]

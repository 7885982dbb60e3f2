"""Optimizer objects of the dynamic-embedding API: table-level classes (``update(hashtables, indices, grads)``) and the
row-level "V2" classes (``fused_update(grads, values)`` on ``[n, dim + state]`` rows), with the argument dictionaries the
checkpoint's ``*_opt_args.json`` files hold.

The fused update normally runs inside the backward (``KeyValueTable.update`` -> the table's in-place optimizer kernel); these
classes give user code the reference's handles for the same formulas: changing the learning rate, exporting / restoring the
optimizer arguments, updating rows it has gathered itself.  Row layout: ``[embedding | state]`` with Adam ``m, v`` (2 x dim),
Adagrad ``G`` (dim), row-wise Adagrad one accumulator padded to 16 bytes, SGD none.  Adam applies decoupled weight decay.
Reference: ``dynamic_emb/distributed/optimizers/base_dynamicemb_optimizer.py:38-220``, ``sgd_*:44-162``, ``adam_*:45-263``,
``adagrad_*:46-203``, ``rowwise_adagrad_*:46-217``.
"""
from __future__ import annotations

import abc
import copy
import dataclasses
from typing import Any, Dict, List, Optional

import torch

from .dynamicemb_config import EmbOptimType
from .hkv import OptimizerType, opt_state_dim


@dataclasses.dataclass
class OptimizerArgs:
    learning_rate: float = 0.01
    weight_decay: float = 0.0
    eps: float = 1e-8
    initial_accumulator_value: float = 0.0
    momentum: float = 0.0
    beta1: float = 0.9
    beta2: float = 0.999
    other: dict = dataclasses.field(default_factory=dict)


def string_to_opt_type(optimizer_str: str) -> EmbOptimType:
    try:
        return EmbOptimType(optimizer_str)
    except ValueError as e:
        raise ValueError("'%s' is not a valid EmbOptimType." % optimizer_str) from e


def get_required_arg(args: Dict[str, Any], key: str) -> Any:
    if key not in args:
        raise ValueError("Input args does not contain required optimizer argument: %s" % key)
    return args[key]


# ----------------------------------------------------------------------------------------------------------------------
# shared formulas on [n, dim + state] rows (fp32 math, written back in the rows' dtype)
# ----------------------------------------------------------------------------------------------------------------------
def _apply(kind: OptimizerType, grads: torch.Tensor, values: torch.Tensor, a: OptimizerArgs, step: int) -> None:
    D = grads.shape[1]
    if values.shape[0] != grads.shape[0] or values.shape[1] < D + opt_state_dim(kind, D):
        raise ValueError("values must be [%d, >= %d] for gradients %s" % (grads.shape[0], D + opt_state_dim(kind, D), tuple(grads.shape)))
    g = grads.float()
    w = values[:, :D].float()
    if kind == OptimizerType.SGD:
        w = w - a.learning_rate * (g + a.weight_decay * w)
    elif kind == OptimizerType.ROWWISE_ADAGRAD:
        acc = values[:, D].float() + (g * g).mean(dim=1)
        w = w - a.learning_rate * g / (acc.sqrt()[:, None] + a.eps)
        values[:, D] = acc.to(values.dtype)
    elif kind == OptimizerType.ADAGRAD:
        acc = values[:, D:2 * D].float() + g * g
        w = w - a.learning_rate * g / (acc.sqrt() + a.eps)
        values[:, D:2 * D] = acc.to(values.dtype)
    else:
        m = a.beta1 * values[:, D:2 * D].float() + (1 - a.beta1) * g
        v = a.beta2 * values[:, 2 * D:3 * D].float() + (1 - a.beta2) * g * g
        t = max(int(step), 1)
        w = w * (1 - a.learning_rate * a.weight_decay) - (a.learning_rate / (1 - a.beta1 ** t)) * m / ((v / (1 - a.beta2 ** t)).sqrt() + a.eps)
        values[:, D:2 * D] = m.to(values.dtype)
        values[:, 2 * D:3 * D] = v.to(values.dtype)
    values[:, :D] = w.to(values.dtype)


class BaseDynamicEmbeddingOptimizerV2(abc.ABC):
    KIND: OptimizerType = OptimizerType.SGD
    NAME = "sgd"

    def __init__(self, opt_args: OptimizerArgs) -> None:
        self._opt_args: OptimizerArgs = copy.deepcopy(opt_args)
        self._iterations = 0

    # -- updates -----------------------------------------------------------------------------------------------------
    def update(self, grads: torch.Tensor, embs: torch.Tensor, states: Optional[torch.Tensor]) -> None:
        """Embeddings and states in two tensors (``states`` may be None for SGD); both updated in place."""
        D = grads.shape[1]
        sd = self.get_state_dim(D)
        rows = torch.cat([embs, states[:, :sd]], dim=1) if sd else embs.clone()
        _apply(self.KIND, grads, rows, self._opt_args, self._iterations)
        embs.copy_(rows[:, :D])
        if sd:
            states[:, :sd].copy_(rows[:, D:D + sd])

    def fused_update(self, grads: torch.Tensor, values: torch.Tensor) -> None:
        """``values``: rows ``[embedding | state]`` (device memory), updated in place."""
        with torch.no_grad():
            _apply(self.KIND, grads, values, self._opt_args, self._iterations)

    def fused_update_hybrid(self, grads: torch.Tensor, values: torch.Tensor) -> None:
        """Same rows when part of them lives in the host-mapped value tier: the arithmetic does not differ."""
        self.fused_update(grads, values)

    def fused_update_with_pointer(self, grads: torch.Tensor, value_ptr: torch.Tensor, value_type=None, region=None) -> None:
        """fp32 rows addressed by ``value_ptr`` (e.g. from ``HKVTable.find_pointers``).  ``region`` - the tensor that holds the
        rows, or its ``(first, one-past-last)`` byte addresses - is required: row IO by address is bounds-checked here."""
        if region is None:
            raise ValueError("fused_update_with_pointer needs region= the rows' tensor or its (lo, hi) addresses (they are checked)")
        from ..ops import by_address as BA

        D = grads.shape[1]
        cols = D + self.get_state_dim(D)
        rows = BA.embedding_lookup_by_address(value_ptr, cols, region)
        self.fused_update(grads, rows)
        BA.embedding_update_by_address(value_ptr, rows, 1, region)

    def fused_update_with_pointer_hybrid(self, grads: torch.Tensor, value_ptr: torch.Tensor, value_type=None, region=None) -> None:
        self.fused_update_with_pointer(grads, value_ptr, value_type, region)

    # -- arguments ---------------------------------------------------------------------------------------------------
    def get_state_dim(self, emb_dim: int) -> int:
        return opt_state_dim(self.KIND, emb_dim)

    def set_learning_rate(self, new_lr: float) -> None:
        self._opt_args.learning_rate = new_lr

    def get_initial_optim_states(self) -> float:
        return self._opt_args.initial_accumulator_value

    def set_initial_optim_states(self, value: float) -> None:
        self._opt_args.initial_accumulator_value = value

    def step(self) -> None:
        self._iterations += 1

    def get_opt_args(self) -> Dict[str, Any]:
        a = self._opt_args
        out: Dict[str, Any] = {"opt_type": self.NAME, "lr": a.learning_rate}
        if self.KIND in (OptimizerType.ADAGRAD, OptimizerType.ROWWISE_ADAGRAD):
            out.update(eps=a.eps, initial_accumulator_value=a.initial_accumulator_value)
        elif self.KIND == OptimizerType.ADAM:
            out.update(iters=self._iterations, beta1=a.beta1, beta2=a.beta2, eps=a.eps, weight_decay=a.weight_decay)
        return out

    def set_opt_args(self, args: Dict[str, Any]) -> None:
        a = self._opt_args
        a.learning_rate = get_required_arg(args, "lr")
        if self.KIND in (OptimizerType.ADAGRAD, OptimizerType.ROWWISE_ADAGRAD):
            a.eps = get_required_arg(args, "eps")
            a.initial_accumulator_value = get_required_arg(args, "initial_accumulator_value")
        elif self.KIND == OptimizerType.ADAM:
            self._iterations = get_required_arg(args, "iters")
            a.beta1, a.beta2 = get_required_arg(args, "beta1"), get_required_arg(args, "beta2")
            a.eps, a.weight_decay = get_required_arg(args, "eps"), get_required_arg(args, "weight_decay")


class SGDDynamicEmbeddingOptimizerV2(BaseDynamicEmbeddingOptimizerV2):
    KIND, NAME = OptimizerType.SGD, "sgd"


class AdamDynamicEmbeddingOptimizerV2(BaseDynamicEmbeddingOptimizerV2):
    KIND, NAME = OptimizerType.ADAM, "adam"


class AdagradDynamicEmbeddingOptimizerV2(BaseDynamicEmbeddingOptimizerV2):
    KIND, NAME = OptimizerType.ADAGRAD, "exact_adagrad"


class RowWiseAdagradDynamicEmbeddingOptimizerV2(BaseDynamicEmbeddingOptimizerV2):
    KIND, NAME = OptimizerType.ROWWISE_ADAGRAD, "exact_row_wise_adagrad"


# ----------------------------------------------------------------------------------------------------------------------
# table-level classes: the optimizer state lives behind the embedding in every row of the table
# ----------------------------------------------------------------------------------------------------------------------
class BaseDynamicEmbeddingOptimizer(abc.ABC):
    KIND: OptimizerType = OptimizerType.SGD
    NAME = "exact_sgd"
    STATES: tuple = ()

    def __init__(self, opt_args: OptimizerArgs, table_options: List[Any], hashtables: List[Any]) -> None:
        self._opt_args: OptimizerArgs = copy.deepcopy(opt_args)
        self._table_options = list(table_options)
        self._hashtables = list(hashtables)
        self._num_tables = len(self._hashtables)
        for ht in self._hashtables:
            if OptimizerType(ht.optimizer) != self.KIND:
                raise ValueError("table rows are laid out for %s, not for %s" % (OptimizerType(ht.optimizer).name, self.KIND.name))
        # the state shares the rows of the embedding tables: every state name maps to the same handles
        self._state_dict: Dict[str, List[Any]] = {n: self._hashtables for n in self.STATES}
        self._table_state_map: Dict[int, int] = {id(ht): i for i, ht in enumerate(self._hashtables)}
        self._iterations = 0

    def get_state_by_name(self, state_name: str):
        return self._state_dict.get(state_name)

    def get_state(self):
        return self._state_dict

    def state_names(self) -> List[str]:
        return list(self._state_dict.keys())

    def table_state_map(self) -> Dict[int, int]:
        return self._table_state_map

    def set_learning_rate(self, new_lr) -> None:
        self._opt_args.learning_rate = new_lr

    def update(self, hashtables: List[Any], indices: List[torch.Tensor], grads: List[torch.Tensor]) -> None:
        """``indices[i]``: keys of table ``hashtables[i]`` (absent keys are skipped), ``grads[i]`` their summed gradients."""
        for ht in hashtables:
            if id(ht) not in self._table_state_map:
                raise ValueError("DynamicEmb ERROR: Hashtable %r not found in _table_state_map in class %s." % (ht, type(self).__name__))
        self._iterations += 1
        a = self._opt_args
        for ht, keys, g in zip(hashtables, indices, grads):
            slots, _found = ht.find(keys)
            ht.update(slots, g, a.learning_rate, a.eps, a.beta1, a.beta2, a.weight_decay, self._iterations)

    get_opt_args = BaseDynamicEmbeddingOptimizerV2.get_opt_args
    set_opt_args = BaseDynamicEmbeddingOptimizerV2.set_opt_args


class SGDDynamicEmbeddingOptimizer(BaseDynamicEmbeddingOptimizer):
    KIND, NAME, STATES = OptimizerType.SGD, "exact_sgd", ()


class AdamDynamicEmbeddingOptimizer(BaseDynamicEmbeddingOptimizer):
    KIND, NAME, STATES = OptimizerType.ADAM, "adam", ("m", "v")


class AdagradDynamicEmbeddingOptimizer(BaseDynamicEmbeddingOptimizer):
    KIND, NAME, STATES = OptimizerType.ADAGRAD, "exact_adagrad", ("Gt",)


class RowWiseAdagradDynamicEmbeddingOptimizer(BaseDynamicEmbeddingOptimizer):
    KIND, NAME, STATES = OptimizerType.ROWWISE_ADAGRAD, "exact_row_wise_adagrad", ("Gt",)


_V2 = {OptimizerType.SGD: SGDDynamicEmbeddingOptimizerV2, OptimizerType.ADAM: AdamDynamicEmbeddingOptimizerV2,
       OptimizerType.ADAGRAD: AdagradDynamicEmbeddingOptimizerV2, OptimizerType.ROWWISE_ADAGRAD: RowWiseAdagradDynamicEmbeddingOptimizerV2}


def create_optimizer(optimizer_type, opt_args: Optional[OptimizerArgs] = None) -> BaseDynamicEmbeddingOptimizerV2:
    """Row-level optimizer object for an ``OptimizerType`` or an ``EmbOptimType``."""
    if isinstance(optimizer_type, EmbOptimType):
        from .dynamicemb_config import convert_optimizer_type

        optimizer_type = convert_optimizer_type(optimizer_type)
    return _V2[OptimizerType(optimizer_type)](opt_args or OptimizerArgs())

"""Optimizers: fused flat dense Adam/SGD, ``apply_optimizer_in_backward`` for embedding tables, and
the ``CombinedOptimizer`` / ``KeyedOptimizerWrapper`` glue of the reference's user flow
(``docs/en/torch/torch_rec_v1/03_quick_start/quick_start.md:239-262``).  Gradient-accumulating sparse
optimizers mirror ``torchrec1.2.0_npu.patch:899-924`` (``AccumulateAdagrad/SGD/Adam``).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterable, List, Optional, Type

import torch
from torch import nn

from ..ops import dense_ops

_ALLOWED_IN_BACKWARD = (torch.optim.SGD, torch.optim.Adam, torch.optim.Adagrad)


class AccumulateAdagrad(torch.optim.Adagrad):
    def __init__(self, params, use_accumulate: bool = False, accumulate_step: int = 1, **kw) -> None:
        super().__init__(params, **kw)
        self.use_accumulate, self.accumulate_step = use_accumulate, accumulate_step


class AccumulateSGD(torch.optim.SGD):
    def __init__(self, params, use_accumulate: bool = False, accumulate_step: int = 1, **kw) -> None:
        super().__init__(params, **kw)
        self.use_accumulate, self.accumulate_step = use_accumulate, accumulate_step


class AccumulateAdam(torch.optim.Adam):
    def __init__(self, params, use_accumulate: bool = False, accumulate_step: int = 1, **kw) -> None:
        super().__init__(params, **kw)
        self.use_accumulate, self.accumulate_step = use_accumulate, accumulate_step


def apply_optimizer_in_backward(optimizer_class: Type[torch.optim.Optimizer], params: Iterable[nn.Parameter],
                                optimizer_kwargs: Dict[str, Any]) -> None:
    """Mark embedding parameters so that their update is fused into the backward of the lookup.

    Only SGD, Adam and Adagrad (and their accumulate variants) are accepted, as in the reference's
    TorchRec patch (``torchrec1.2.0_npu.patch:823-824``).
    """
    if not issubclass(optimizer_class, _ALLOWED_IN_BACKWARD):
        raise ValueError("apply_optimizer_in_backward supports torch.optim.{SGD, Adam, Adagrad}, got %s" % optimizer_class)
    for p in params:
        p._optimizer_classes = [optimizer_class]  # type: ignore[attr-defined]
        p._optimizer_kwargs = [dict(optimizer_kwargs)]  # type: ignore[attr-defined]
        p._in_backward_optimizers = True  # type: ignore[attr-defined]


class FusedOptimizerStub(torch.optim.Optimizer):
    """Optimizer whose update already happened inside the backward kernel: ``step`` is a no-op, but
    hyper-parameters stay editable through ``param_groups`` (learning-rate schedules)."""

    def __init__(self, params: List[nn.Parameter], spec) -> None:
        self.spec = spec
        super().__init__(params if params else [torch.zeros(1)], {"lr": spec.lr})

    def step(self, closure=None):  # noqa: ARG002
        self.spec.lr = self.param_groups[0]["lr"]
        return None

    def zero_grad(self, set_to_none: bool = True) -> None:  # noqa: ARG002
        return None


class FusedDenseOptimizer(torch.optim.Optimizer):
    """Adam or SGD over modules that expose ``flat_param / flat_grad / flat_shadow`` (``FusedMLP``-style)
    with one kernel launch per module, plus a stock PyTorch optimizer for any remaining parameters."""

    def __init__(self, module: nn.Module, kind: str = "adam", lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, grad_scale: float = 1.0) -> None:
        self.kind, self.betas, self.eps, self.weight_decay = kind, betas, eps, weight_decay
        self.grad_scale = grad_scale
        self.flat_modules = [m for m in module.modules() if hasattr(m, "flat_param") and hasattr(m, "flat_grad")]
        flat_ids = {id(m.flat_param) for m in self.flat_modules}
        rest = [p for p in module.parameters() if id(p) not in flat_ids and p.requires_grad
                and not getattr(p, "_in_backward_optimizers", False)]
        self.rest = rest
        params = [m.flat_param for m in self.flat_modules] + rest
        super().__init__(params if params else [torch.zeros(1)], {"lr": lr})
        if rest:
            if kind == "adam":
                self._rest_opt = torch.optim.Adam(rest, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                                  capturable=all(p.is_cuda for p in rest))
            else:
                self._rest_opt = torch.optim.SGD(rest, lr=lr, weight_decay=weight_decay)
        else:
            self._rest_opt = None
        self._step = 0
        self._hyper: Optional[torch.Tensor] = None
        self._hyper_lr = lr
        self._m: Dict[int, torch.Tensor] = {}
        self._v: Dict[int, torch.Tensor] = {}

    @torch.no_grad()
    def step(self, closure=None):  # noqa: ARG002
        self._step += 1
        lr = self.param_groups[0]["lr"]
        hyper = None
        if self.kind == "adam" and self.flat_modules and self.flat_modules[0].flat_param.is_cuda:
            dev = self.flat_modules[0].flat_param.device
            if self._hyper is None or self._hyper.device != dev:
                self._hyper = torch.tensor([lr, 1.0, 1.0, float(self._step - 1)], dtype=torch.float32, device=dev)
                self._hyper_lr = lr
            if lr != self._hyper_lr:      # learning-rate change: host write, outside any graph capture
                self._hyper[0:1].fill_(lr)
                self._hyper_lr = lr
            hyper = self._hyper
            dense_ops.adam_tick(hyper, self.betas[0], self.betas[1])
        for mod in self.flat_modules:
            p, g = mod.flat_param.data, mod.flat_grad
            shadow = getattr(mod, "flat_shadow", None)
            if self.kind == "adam":
                key = id(mod)
                if key not in self._m or self._m[key].device != p.device:
                    self._m[key] = torch.zeros_like(p)
                    self._v[key] = torch.zeros_like(p)
                dense_ops.adam_flat(p, g, self._m[key], self._v[key], shadow, lr, self.betas[0], self.betas[1], self.eps,
                                    self.weight_decay, self._step, self.grad_scale, hyper)
            else:
                dense_ops.sgd_flat(p, g, shadow, lr, self.weight_decay, self.grad_scale)
        if self._rest_opt is not None:
            for gq in self._rest_opt.param_groups:
                gq["lr"] = lr
            self._rest_opt.step()
        return None

    def zero_grad(self, set_to_none: bool = True) -> None:
        for mod in self.flat_modules:
            mod.flat_grad.zero_()
        if self._rest_opt is not None:
            self._rest_opt.zero_grad(set_to_none=set_to_none)


class KeyedOptimizerWrapper(torch.optim.Optimizer):
    """``KeyedOptimizerWrapper(named_params, lambda params: Optimizer(params))``."""

    def __init__(self, params: Dict[str, nn.Parameter], optim_factory: Callable[[List[nn.Parameter]], torch.optim.Optimizer]) -> None:
        self.named = dict(params)
        self._inner = optim_factory(list(self.named.values())) if self.named else None
        super().__init__(list(self.named.values()) or [torch.zeros(1)], {})

    def step(self, closure=None):
        return self._inner.step(closure) if self._inner is not None else None

    def zero_grad(self, set_to_none: bool = True) -> None:
        if self._inner is not None:
            self._inner.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return self._inner.state_dict() if self._inner is not None else {}

    def load_state_dict(self, sd) -> None:
        if self._inner is not None:
            self._inner.load_state_dict(sd)


class CombinedOptimizer:
    """Steps a list of optimizers together (fused sparse stubs + dense optimizers)."""

    def __init__(self, optims: List[Any]) -> None:
        self.optims = [o for o in optims if o is not None]

    @property
    def param_groups(self):
        out = []
        for o in self.optims:
            out += getattr(o, "param_groups", [])
        return out

    def step(self, closure=None):
        for o in self.optims:
            o.step()
        return None

    def zero_grad(self, set_to_none: bool = True) -> None:
        for o in self.optims:
            o.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return {str(i): o.state_dict() for i, o in enumerate(self.optims) if hasattr(o, "state_dict")}

    def load_state_dict(self, sd) -> None:
        for i, o in enumerate(self.optims):
            if str(i) in sd and hasattr(o, "load_state_dict"):
                o.load_state_dict(sd[str(i)])

"""Dense MLP blocks.

``FusedMLP`` keeps fp32 master weights and a 16-bit shadow copy in flat buffers and runs every layer
(forward, input-gradient with the ReLU mask fused, weight-gradient with split-K) on the tcgen05 GEMM.
Weight gradients are accumulated straight into a flat fp32 gradient buffer (``flat_grad``), which is
what the fused dense optimizer and the fused gradient all-reduce consume; autograd never sees
per-parameter ``.grad`` tensors for these layers.

``MLP`` is the plain fp32 ``nn.Linear`` stack used on CPU.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
from torch import nn

from ..ops import _lib
from ..ops import dense_ops, gemm


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class MLP(nn.Module):
    """fp32 reference MLP: Linear(+ReLU) per layer; ``final_activation`` controls the last layer."""

    def __init__(self, in_features: int, layer_sizes: Sequence[int], final_activation: bool = True,
                 bias: bool = True, device=None) -> None:
        super().__init__()
        layers: List[nn.Module] = []
        k = in_features
        for i, n in enumerate(layer_sizes):
            layers.append(nn.Linear(k, n, bias=bias, device=device))
            if i + 1 < len(layer_sizes) or final_activation:
                layers.append(nn.ReLU())
            k = n
        self.net = nn.Sequential(*layers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(x)


class _FusedMLPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, mlp: "FusedMLP", grad_premasked: bool, _flat: torch.Tensor, grad_mode: bool = True):
        acts = [x]
        L = mlp.num_layers
        for l in range(L):
            relu = mlp.relu[l]
            y = gemm.gemm16(acts[-1], mlp.w16[l], bias=mlp.b32[l], epi=gemm.EPI_RELU if relu else gemm.EPI_NONE)
            acts.append(y)
        ctx.mlp = mlp
        # A backward will follow this forward.  ``needs_input_grad`` stays true for the parameters under ``torch.no_grad()``
        # (and grad mode always reads "off" inside a Function), so the caller passes the grad mode it ran under: an
        # evaluation pass must not leave the counter raised, or the gradient-ready hook would never fire again.
        ctx.counted = bool(grad_mode) and any(ctx.needs_input_grad)
        if ctx.counted:
            mlp._pending_backward += 1
        ctx.grad_premasked = grad_premasked
        ctx.x_needs_grad = x.requires_grad
        ctx.save_for_backward(*acts)
        return acts[-1]

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        mlp: FusedMLP = ctx.mlp
        acts = ctx.saved_tensors
        L = mlp.num_layers
        dz = dy if dy.stride(-1) == 1 else dy.contiguous()
        if mlp.relu[L - 1] and not ctx.grad_premasked:
            dz = dz * (acts[L] > 0).to(dz.dtype)
        nsm = _lib.num_sms(dz.device) if dz.is_cuda else 148
        dx = None
        bias_done = False            # this layer's bias gradient already came out of the GEMM that produced dz
        for l in range(L - 1, -1, -1):
            x_l = acts[l]
            M = x_l.shape[0]
            N, Kp = mlp.w16[l].shape
            gemm.gemm16(dz, x_l, a_mn=True, b_mn=True, out=mlp.wgrad[l], epi=gemm.EPI_F32_ATOMIC,
                        splits=gemm.pick_splits(N, Kp, M, nsm))
            if mlp.bgrad[l] is not None and not bias_done:
                dense_ops.colsum16(dz, mlp.bgrad[l])
            bias_done = False
            if l > 0:
                # dz of layer l-1 and, in the same epilogue, its column sums (= that layer's bias gradient)
                cs = mlp.bgrad[l - 1] if dz.is_cuda else None
                bias_done = cs is not None
                if mlp.relu[l - 1]:
                    dz = gemm.gemm16(dz, mlp.w16[l], b_mn=True, epi=gemm.EPI_RELU_MASK, aux=x_l, colsum_out=cs)
                else:
                    dz = gemm.gemm16(dz, mlp.w16[l], b_mn=True, colsum_out=cs)
            elif ctx.x_needs_grad:
                dx = gemm.gemm16(dz, mlp.w16[l], b_mn=True)
        if ctx.counted:
            mlp._pending_backward -= 1
        if mlp._grad_ready_hook is not None and mlp._pending_backward <= 0:
            mlp._pending_backward = 0
            mlp._grad_ready_hook(mlp)          # every weight gradient of this module is enqueued: its all-reduce may start
        return dx, None, None, None, None


class FusedMLP(nn.Module):
    """16-bit MLP on the tcgen05 GEMM with fp32 master weights.

    ``in_features`` is padded up to a multiple of 8 (``in_padded``); callers feed ``[B, in_padded]``
    activations (padding columns zero).  ``weight(l)`` / ``bias(l)`` return fp32 views of layer ``l``.
    """

    ALIGN = 64

    def __init__(self, in_features: int, layer_sizes: Sequence[int], final_activation: bool = True,
                 bias: bool = True, device=None, dtype: torch.dtype = torch.bfloat16) -> None:
        super().__init__()
        self.in_features = in_features
        self.in_padded = _round_up(in_features, 8)
        self.layer_sizes = list(layer_sizes)
        self.num_layers = len(self.layer_sizes)
        self.compute_dtype = dtype
        self.relu = [(i + 1 < self.num_layers) or final_activation for i in range(self.num_layers)]
        self.has_bias = bias
        for n in self.layer_sizes[:-1]:
            if n % 8:
                raise ValueError("hidden sizes must be multiples of 8")
        self._shapes = []
        k_true, k_pad = in_features, self.in_padded
        off = 0
        for n in self.layer_sizes:
            w_off = off
            off += _round_up(n * k_pad, self.ALIGN)
            b_off = off
            off += _round_up(n, self.ALIGN) if bias else 0
            self._shapes.append((n, k_true, k_pad, w_off, b_off))
            k_true, k_pad = n, _round_up(n, 8)
        self.flat_param = nn.Parameter(torch.zeros(off, dtype=torch.float32, device=device))
        self.register_buffer("flat_shadow", torch.zeros(off, dtype=dtype, device=device), persistent=False)
        self.register_buffer("flat_grad", torch.zeros(off, dtype=torch.float32, device=device), persistent=False)
        self._pending_backward = 0
        self._grad_ready_hook = None
        self.reset_parameters()

    def set_grad_ready_hook(self, hook) -> None:
        """``hook(module)`` runs at the end of this module's backward, once the last weight-gradient GEMM of the step is
        enqueued (a module applied several times per step fires after its last backward)."""
        self._grad_ready_hook = hook

    # -- views ----------------------------------------------------------------
    def _build_views(self) -> None:
        self.w16, self.b32, self.wgrad, self.bgrad, self.w32 = [], [], [], [], []
        for (n, _k, kp, w_off, b_off) in self._shapes:
            self.w32.append(self.flat_param.data[w_off:w_off + n * kp].view(n, kp))
            self.w16.append(self.flat_shadow[w_off:w_off + n * kp].view(n, kp))
            self.wgrad.append(self.flat_grad[w_off:w_off + n * kp].view(n, kp))
            if self.has_bias:
                self.b32.append(self.flat_param.data[b_off:b_off + n])
                self.bgrad.append(self.flat_grad[b_off:b_off + n])
            else:
                self.b32.append(None)
                self.bgrad.append(None)

    def _apply(self, fn, *args, **kwargs):
        out = super()._apply(fn, *args, **kwargs)
        if self.flat_shadow.dtype != self.compute_dtype:
            self.flat_shadow = self.flat_shadow.to(self.compute_dtype)
        if self.flat_grad.dtype != torch.float32:
            self.flat_grad = self.flat_grad.float()
        self._build_views()
        self.sync_shadow()
        return out

    def set_grad_buffer(self, buf: torch.Tensor) -> None:
        """Re-home the flat gradient buffer (e.g. into peer-mapped memory for the fused all-reduce)."""
        assert buf.numel() == self.flat_grad.numel() and buf.dtype == torch.float32
        buf.copy_(self.flat_grad)
        self.flat_grad = buf
        self._build_views()

    def weight(self, l: int) -> torch.Tensor:
        n, k, _kp, _w, _b = self._shapes[l]
        return self.w32[l][:, :k]

    def bias(self, l: int) -> Optional[torch.Tensor]:
        return self.b32[l]

    def weight_grad(self, l: int) -> torch.Tensor:
        n, k, _kp, _w, _b = self._shapes[l]
        return self.wgrad[l][:, :k]

    def bias_grad(self, l: int) -> Optional[torch.Tensor]:
        return self.bgrad[l]

    @torch.no_grad()
    def reset_parameters(self) -> None:
        self._build_views()
        for l, (n, k, kp, _w, _b) in enumerate(self._shapes):
            self.w32[l].zero_()
            bound = 1.0 / math.sqrt(k)
            self.w32[l][:, :k].uniform_(-bound, bound)
            if self.has_bias:
                self.b32[l].uniform_(-bound, bound)
        self.sync_shadow()

    @torch.no_grad()
    def load_from_linears(self, linears: Sequence[nn.Linear]) -> None:
        """Copy weights from ``nn.Linear`` layers (tests: identical initialisation for both paths)."""
        for l, lin in enumerate(linears):
            self.w32[l].zero_()
            self.weight(l).copy_(lin.weight.detach().float())
            if self.has_bias and lin.bias is not None:
                self.b32[l].copy_(lin.bias.detach().float())
        self.sync_shadow()

    @torch.no_grad()
    def sync_shadow(self) -> None:
        self.flat_shadow.copy_(self.flat_param.data.to(self.flat_shadow.dtype))

    def zero_grad_buffers(self) -> None:
        self.flat_grad.zero_()

    def forward(self, x: torch.Tensor, grad_premasked: bool = False) -> torch.Tensor:
        """``x`` is ``[B, in_padded]`` in the compute dtype.  ``grad_premasked`` promises that the
        incoming gradient of a ReLU-terminated MLP is already multiplied by the ReLU mask."""
        assert x.shape[1] == self.in_padded, "expected %d (padded) input columns" % self.in_padded
        return _FusedMLPFn.apply(x, self, grad_premasked, self.flat_param, torch.is_grad_enabled())

"""Dense-side helper kernels (``csrc/cuda/dense_misc.cu``) with PyTorch references for CPU tensors."""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib


def bce_head(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], labels: torch.Tensor, inv_batch: float,
             logits: Optional[torch.Tensor], loss_sum: torch.Tensor, dh: Optional[torch.Tensor],
             dw: Optional[torch.Tensor], db: Optional[torch.Tensor], relu_mask: bool = False) -> None:
    """Final ``K -> 1`` linear layer + BCE-with-logits loss + backward in one pass.

    Accumulates ``loss_sum += mean-scaled loss``, ``dw += ...``, ``db += ...`` and writes ``dh``.
    ``inv_batch`` is 1 / (global batch) so gradients are those of the global mean loss.
    """
    if not h.is_cuda:
        z = h.float() @ w.float() + (bias.float() if bias is not None else 0.0)
        y = labels.float()
        loss = torch.clamp(z, min=0) - z * y + torch.log1p(torch.exp(-z.abs()))
        loss_sum += loss.sum() * inv_batch
        dz = (torch.sigmoid(z) - y) * inv_batch
        if logits is not None:
            logits.copy_(z)
        if dh is not None:
            g = dz[:, None] * w.float()[None, :]
            if relu_mask:
                g = g * (h.float() > 0)
            dh.copy_(g.to(dh.dtype))
        if dw is not None:
            dw += dz @ h.float()
        if db is not None:
            db += dz.sum()
        return
    B, K = h.shape
    assert h.dtype == torch.bfloat16 and h.stride(1) == 1 and w.dtype == torch.float32
    rc = _lib.lib().rb_bce_head(h.data_ptr(), h.stride(0), B, K, w.data_ptr(), _lib.ptr(bias), labels.data_ptr(),
                                float(inv_batch), _lib.ptr(logits), loss_sum.data_ptr(), _lib.ptr(dh),
                                dh.stride(0) if dh is not None else 0, _lib.ptr(dw), _lib.ptr(db), int(relu_mask),
                                _lib.num_sms(h.device), _lib.stream_ptr(h.device))
    _lib.check(rc, "rb_bce_head")


def colsum16(a: torch.Tensor, out: torch.Tensor) -> None:
    """``out[n] += sum_m a[m, n]`` (fp32 accumulation of a bf16/fp16 matrix)."""
    if not a.is_cuda:
        out += a.float().sum(0)
        return
    rc = _lib.lib().rb_colsum16(a.data_ptr(), a.stride(0), a.shape[0], a.shape[1], int(a.dtype == torch.bfloat16),
                                out.data_ptr(), _lib.stream_ptr(a.device))
    _lib.check(rc, "rb_colsum16")


def adam_flat(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, shadow: Optional[torch.Tensor],
              lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
              grad_scale: float = 1.0, hyper: Optional[torch.Tensor] = None) -> None:
    """Adam on flat buffers.  With ``hyper`` (device float[4] = lr, 1-b1^t, 1-b2^t, t; advanced by
    ``adam_tick``) the learning rate and bias corrections are read on the device, which keeps a
    captured CUDA graph correct across replays."""
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    if not p.is_cuda:
        gi = g * grad_scale + weight_decay * p
        m.mul_(beta1).add_(gi, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(gi, gi, value=1 - beta2)
        p.sub_((lr / bc1) * m / ((v / bc2).sqrt() + eps))
        if shadow is not None:
            shadow.copy_(p.to(shadow.dtype))
        return
    rc = _lib.lib().rb_adam_flat(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), _lib.ptr(shadow),
                                 int(shadow is None or shadow.dtype == torch.bfloat16), p.numel(), lr, beta1, beta2, eps,
                                 weight_decay, bc1, bc2, grad_scale, _lib.ptr(hyper), _lib.num_sms(p.device),
                                 _lib.stream_ptr(p.device))
    _lib.check(rc, "rb_adam_flat")


def adam_tick(hyper: torch.Tensor, beta1: float, beta2: float) -> None:
    rc = _lib.lib().rb_adam_tick(hyper.data_ptr(), beta1, beta2, _lib.stream_ptr(hyper.device))
    _lib.check(rc, "rb_adam_tick")


def sgd_flat(p: torch.Tensor, g: torch.Tensor, shadow: Optional[torch.Tensor], lr: float, weight_decay: float = 0.0,
             grad_scale: float = 1.0) -> None:
    if not p.is_cuda:
        p.sub_(lr * (g * grad_scale + weight_decay * p))
        if shadow is not None:
            shadow.copy_(p.to(shadow.dtype))
        return
    rc = _lib.lib().rb_sgd_flat(p.data_ptr(), g.data_ptr(), _lib.ptr(shadow),
                                int(shadow is None or shadow.dtype == torch.bfloat16), p.numel(), lr, weight_decay,
                                grad_scale, _lib.num_sms(p.device), _lib.stream_ptr(p.device))
    _lib.check(rc, "rb_sgd_flat")


def cast_pad(src: torch.Tensor, cols_pad: int, dtype: torch.dtype = torch.bfloat16,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 ``[rows, cols]`` -> 16-bit ``[rows, cols_pad]`` with zero padding columns."""
    rows, cols = src.shape
    if out is None:
        out = torch.empty(rows, cols_pad, dtype=dtype, device=src.device)
    if not src.is_cuda:
        out.zero_()
        out[:, :cols] = src.to(dtype)
        return out
    assert src.dtype == torch.float32 and src.stride(1) == 1
    rc = _lib.lib().rb_cast_pad_f32_to_16(src.data_ptr(), src.stride(0), rows, cols, out.data_ptr(), out.stride(0),
                                          cols_pad, int(dtype == torch.bfloat16), _lib.num_sms(src.device),
                                          _lib.stream_ptr(src.device))
    _lib.check(rc, "rb_cast_pad_f32_to_16")
    return out

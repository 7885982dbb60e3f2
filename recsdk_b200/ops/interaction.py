"""Pairwise dot interaction (DLRM) on ``csrc/cuda/interaction.cu`` with an fp32 PyTorch reference.

``R[b] = [ x0[b] | <X_i, X_j> for 0 <= j < i < F | zero pad ]`` where ``X = [x0 | xs]``.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib


def interaction_out_cols(F: int, D: int, pad_to: int = 8) -> int:
    n = D + F * (F - 1) // 2
    return (n + pad_to - 1) // pad_to * pad_to


def _tri_index(F: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    i, j = torch.tril_indices(F, F, offset=-1, device=device)
    return i, j


def dot_interaction_ref(x0: torch.Tensor, xs: torch.Tensor, F: int, out_cols: int) -> torch.Tensor:
    B, D = x0.shape
    X = torch.cat([x0.float().unsqueeze(1), xs.float().reshape(B, F - 1, D)], dim=1)
    Z = torch.bmm(X, X.transpose(1, 2))
    i, j = _tri_index(F, x0.device)
    tri = Z[:, i, j]
    out = torch.zeros(B, out_cols, dtype=torch.float32, device=x0.device)
    out[:, :D] = x0.float()
    out[:, D:D + tri.shape[1]] = tri
    return out


def dot_interaction_bwd_ref(x0: torch.Tensor, xs: torch.Tensor, dR: torch.Tensor, F: int):
    B, D = x0.shape
    X = torch.cat([x0.float().unsqueeze(1), xs.float().reshape(B, F - 1, D)], dim=1)
    i, j = _tri_index(F, x0.device)
    dZ = torch.zeros(B, F, F, dtype=torch.float32, device=x0.device)
    dZ[:, i, j] = dR.float()[:, D:D + i.numel()]
    dZs = dZ + dZ.transpose(1, 2)
    dX = torch.bmm(dZs, X)
    dX[:, 0, :] += dR.float()[:, :D]
    return dX[:, 0, :].contiguous(), dX[:, 1:, :].reshape(B, (F - 1) * D).contiguous()


def dot_interaction_fwd(x0: torch.Tensor, xs: torch.Tensor, F: int, out: torch.Tensor) -> torch.Tensor:
    """x0 [B,D], xs [B,(F-1)*D] (bf16, unit inner stride) -> out [B, out_cols] bf16."""
    B, D = x0.shape
    if not x0.is_cuda:
        out.copy_(dot_interaction_ref(x0, xs, F, out.shape[1]).to(out.dtype))
        return out
    assert x0.dtype == torch.bfloat16 and xs.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert x0.stride(1) == 1 and xs.stride(1) == 1 and out.stride(1) == 1
    assert x0.stride(0) % 8 == 0 and xs.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
    rc = _lib.lib().rb_dot_interaction_fwd(x0.data_ptr(), x0.stride(0), xs.data_ptr(), xs.stride(0), B, F, D,
                                           out.data_ptr(), out.stride(0), out.shape[1], _lib.num_sms(x0.device),
                                           _lib.stream_ptr(x0.device))
    _lib.check(rc, "rb_dot_interaction_fwd")
    return out


def dot_interaction_bwd(x0: torch.Tensor, xs: torch.Tensor, dR: torch.Tensor, F: int, dx0: torch.Tensor,
                        dxs: torch.Tensor, mask_x0: bool = False) -> None:
    """``mask_x0``: ``x0`` is a ReLU output; return ``dx0 * (x0 > 0)`` (the gradient of its pre-activation)."""
    B, D = x0.shape
    if not x0.is_cuda:
        a, b = dot_interaction_bwd_ref(x0, xs, dR, F)
        if mask_x0:
            a = a * (x0.float() > 0)
        dx0.copy_(a.to(dx0.dtype))
        dxs.copy_(b.to(dxs.dtype))
        return
    assert dR.stride(1) == 1 and dx0.stride(1) == 1 and dxs.stride(1) == 1
    rc = _lib.lib().rb_dot_interaction_bwd(x0.data_ptr(), x0.stride(0), xs.data_ptr(), xs.stride(0), dR.data_ptr(),
                                           dR.stride(0), dR.shape[1], B, F, D, dx0.data_ptr(), dx0.stride(0),
                                           dxs.data_ptr(), dxs.stride(0), int(mask_x0), _lib.num_sms(x0.device),
                                           _lib.stream_ptr(x0.device))
    _lib.check(rc, "rb_dot_interaction_bwd")


class DotInteractionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x0: torch.Tensor, xs: torch.Tensor, F: int, out_cols: int, mask_x0: bool = False):
        out = torch.empty(x0.shape[0], out_cols, dtype=x0.dtype, device=x0.device)
        dot_interaction_fwd(x0, xs, F, out)
        ctx.save_for_backward(x0, xs)
        ctx.F, ctx.mask_x0 = F, mask_x0
        # a producer may nominate the buffer its gradient should be written into (e.g. a peer-mapped buffer that other
        # GPUs read): saves the consumer a copy
        ctx.grad_buffer = getattr(xs, "_grad_out_buffer", None)
        return out

    @staticmethod
    def backward(ctx, dR: torch.Tensor):
        x0, xs = ctx.saved_tensors
        dx0 = torch.empty_like(x0)
        gb = ctx.grad_buffer
        dxs = gb if (gb is not None and gb.shape == xs.shape and gb.dtype == xs.dtype and gb.is_contiguous()) else torch.empty_like(xs)
        dot_interaction_bwd(x0, xs, dR if dR.stride(1) == 1 else dR.contiguous(), ctx.F, dx0, dxs, ctx.mask_x0)
        return dx0, dxs, None, None, None


def dot_interaction(x0: torch.Tensor, xs: torch.Tensor, F: int, out_cols: int, mask_x0: bool = False) -> torch.Tensor:
    """``mask_x0=True`` promises that ``x0`` comes out of a ReLU; its returned gradient is then already
    multiplied by the ReLU mask (the producing MLP can skip its own masking pass)."""
    return DotInteractionFunction.apply(x0, xs, F, out_cols, mask_x0)

"""Fused model-level ops (``csrc/cuda/model_ops.cu``): sampled-softmax loss, DCN v2 cross combine, multi-slice concat.
Each has a plain PyTorch statement for CPU tensors, which is also the oracle of its GPU test."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib, gemm


# ----------------------------------------------------------------------------- sampled softmax
class _SampledSoftmaxFn(torch.autograd.Function):
    """loss = sum_rows( logsumexp([<h, e_pos>, h @ E_neg^T]) - <h, e_pos> ) * scale, with every gradient produced by the
    same pass over the logits.  The loss is the root of the backward pass (its incoming gradient is taken as 1)."""

    @staticmethod
    def forward(ctx, h: torch.Tensor, e_pos: torch.Tensor, e_neg: torch.Tensor, scale: float):
        M, d = h.shape
        N = e_neg.shape[0]
        logits = gemm.gemm16(h, e_neg)                                  # [M, N] bf16 on the tcgen05 GEMM
        dh = torch.empty_like(h)
        de = torch.empty_like(e_pos)
        loss = torch.zeros(1, dtype=torch.float32, device=h.device)
        rc = _lib.lib().rb_sampled_softmax(h.data_ptr(), e_pos.data_ptr(), h.stride(0), e_pos.stride(0), d, logits.data_ptr(),
                                           logits.stride(0), N, M, float(scale), dh.data_ptr(), de.data_ptr(), dh.stride(0),
                                           de.stride(0), loss.data_ptr(), None, _lib.stream_ptr(h.device))
        _lib.check(rc, "rb_sampled_softmax")
        ctx.save_for_backward(h, e_neg, logits, dh, de)                 # logits now hold d loss / d logits
        return loss.squeeze(0)

    @staticmethod
    def backward(ctx, _gloss):
        h, e_neg, dlogits, dh, de = ctx.saved_tensors
        # d h = dL @ E_neg + dpos * e_pos ; d E_neg = dL^T @ h
        dh_total = gemm.gemm16(dlogits, e_neg, b_mn=True)
        dh_total += dh
        dneg32 = torch.zeros(e_neg.shape, dtype=torch.float32, device=h.device)
        gemm.gemm16(dlogits, h, a_mn=True, b_mn=True, out=dneg32, epi=gemm.EPI_F32_ATOMIC,
                    splits=gemm.pick_splits(e_neg.shape[0], e_neg.shape[1], h.shape[0]))
        return dh_total, de, dneg32.to(e_neg.dtype), None


def sampled_softmax_loss(h: torch.Tensor, e_pos: torch.Tensor, e_neg: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``h`` [M, d] query vectors, ``e_pos`` [M, d] embeddings of the true next items, ``e_neg`` [N, d] shared sampled
    negatives -> scalar ``scale * sum_i (logsumexp([h_i . e_pos_i, h_i . e_neg_*]) - h_i . e_pos_i)``."""
    ok = (h.is_cuda and h.dtype == torch.bfloat16 and e_pos.dtype == torch.bfloat16 and e_neg.dtype == torch.bfloat16
          and h.shape[1] % 8 == 0 and e_neg.shape[0] % 8 == 0 and e_neg.shape[0] <= 2048 and h.shape[0] > 0)
    if not ok:
        pos = (h.float() * e_pos.float()).sum(-1, keepdim=True)
        neg = h.float() @ e_neg.float().t()
        logits = torch.cat([pos, neg], dim=1)
        return (torch.logsumexp(logits, dim=1) - pos.squeeze(1)).sum() * scale
    return _SampledSoftmaxFn.apply(h.contiguous(), e_pos.contiguous(), e_neg.contiguous(), scale)


# ----------------------------------------------------------------------------- DCN v2 cross combine
class _CrossCombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x0, xw, xl):
        y = torch.empty_like(xl)
        rc = _lib.lib().rb_dcn_cross_fwd(x0.data_ptr(), xw.data_ptr(), xl.data_ptr(), y.data_ptr(), y.numel(),
                                         _lib.dtype_code(y.dtype), _lib.stream_ptr(y.device))
        _lib.check(rc, "rb_dcn_cross_fwd")
        ctx.save_for_backward(x0, xw)
        return y

    @staticmethod
    def backward(ctx, dy):
        x0, xw = ctx.saved_tensors
        dy = dy.contiguous()
        dxw = torch.empty_like(xw)
        dx0 = torch.empty(x0.shape, dtype=torch.float32, device=x0.device)
        rc = _lib.lib().rb_dcn_cross_bwd(dy.data_ptr(), x0.data_ptr(), xw.data_ptr(), dxw.data_ptr(), dx0.data_ptr(), 0,
                                         dy.numel(), _lib.dtype_code(dy.dtype), _lib.stream_ptr(dy.device))
        _lib.check(rc, "rb_dcn_cross_bwd")
        return dx0.to(x0.dtype), dxw, dy


def dcn_cross_combine(x0: torch.Tensor, xw: torch.Tensor, xl: torch.Tensor) -> torch.Tensor:
    """``x0 * xw + xl`` (one cross layer of DCN v2 after its projection ``xw = W x_l + b``), fused forward and backward."""
    if not (x0.is_cuda and x0.dtype in (torch.bfloat16, torch.float16, torch.float32) and x0.numel() % 8 == 0
            and x0.dtype == xw.dtype == xl.dtype and x0.shape == xw.shape == xl.shape):
        return x0 * xw + xl
    return _CrossCombineFn.apply(x0.contiguous(), xw.contiguous(), xl.contiguous())


# ----------------------------------------------------------------------------- multislice concat
def multislice_concat(x: torch.Tensor, slices: Sequence[Tuple[int, int]]) -> torch.Tensor:
    """``torch.cat([x[:, a:b] for a, b in slices], dim=1)`` for a 2-D row-major ``x`` in one launch (<= 32 slices)."""
    starts = [int(a) for a, _ in slices]
    lens = [int(b) - int(a) for a, b in slices]
    if any(l < 0 for l in lens) or any(a < 0 or a + l > x.shape[1] for a, l in zip(starts, lens)):
        raise ValueError("slice outside the tensor")
    if not x.is_cuda or len(slices) > 32 or x.dim() != 2 or x.stride(1) != 1:
        return torch.cat([x[:, a:a + l] for a, l in zip(starts, lens)], dim=1)
    out = torch.empty(x.shape[0], sum(lens), dtype=x.dtype, device=x.device)
    s_arr, l_arr = np.asarray(starts, dtype=np.int32), np.asarray(lens, dtype=np.int32)
    rc = _lib.lib().rb_multislice_concat(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), x.shape[0],
                                         s_arr.ctypes.data, l_arr.ctypes.data, len(lens), x.element_size(),
                                         _lib.stream_ptr(x.device))
    _lib.check(rc, "rb_multislice_concat")
    return out

"""16-bit GEMM with fused epilogues on the tcgen05 kernel (``csrc/cuda/gemm_tcgen05.cu``).

``gemm16`` computes ``out[M,N] = epi(alpha * A @ B^T)`` where each operand may be stored
contraction-major (``[M,K]`` / ``[N,K]``) or "MN-major" (``[K,M]`` / ``[K,N]``).  On CPU tensors the
same contract is evaluated with fp32 PyTorch ops (this is also the numerical reference of the GPU tests).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

EPI_NONE = 0        # 16-bit out = acc (+bias)
EPI_RELU = 1        # 16-bit out = relu(acc + bias)
EPI_RELU_MASK = 2   # 16-bit out = acc * (aux > 0)
EPI_F32_ATOMIC = 3  # fp32 out += acc (split-K capable)
EPI_SILU = 4        # 16-bit out = silu(acc + bias)
EPI_F32 = 5         # fp32 out = acc (+bias)
EPI_DSILU = 6       # 16-bit out = acc * silu'(aux)


def _ref(a, b, a_mn, b_mn, bias, aux, epi, alpha, out, out_dtype):
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    acc = (af @ bf) * alpha
    if bias is not None:
        acc = acc + bias.float()
    if epi == EPI_RELU:
        acc = torch.relu(acc)
    elif epi == EPI_SILU:
        acc = torch.nn.functional.silu(acc)
    elif epi == EPI_RELU_MASK:
        acc = acc * (aux.float() > 0)
    elif epi == EPI_DSILU:
        x = aux.float()
        s = torch.sigmoid(x)
        acc = acc * (s * (1 + x * (1 - s)))
    if epi == EPI_F32_ATOMIC:
        out += acc
        return out
    res = acc.to(out_dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def gemm16(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
           out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
           aux: Optional[torch.Tensor] = None, epi: int = EPI_NONE, alpha: float = 1.0,
           splits: int = 1, colsum_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = epi(alpha * A @ B^T)``; ``a``/``b`` are bf16 or fp16 2-D tensors with unit inner stride.

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``), ``b`` is ``[N,K]`` (or ``[K,N]`` when ``b_mn``).
    ``out`` may be a strided row view (e.g. a column slice of a wider buffer).  fp32 epilogues
    (``EPI_F32``, ``EPI_F32_ATOMIC``) need an fp32 ``out``; ``EPI_F32_ATOMIC`` accumulates into it.
    ``colsum_out`` (fp32 ``[N]``, 16-bit epilogues only) accumulates the column sums of the output values - the bias
    gradient when the output is a layer's ``dZ`` - inside the same epilogue.
    """
    assert a.dim() == 2 and b.dim() == 2 and a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16)
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, "contraction mismatch %d vs %d" % (K, Kb)
    f32_out = epi in (EPI_F32, EPI_F32_ATOMIC)
    out_dtype = torch.float32 if f32_out else a.dtype
    if epi == EPI_F32_ATOMIC:
        assert out is not None, "EPI_F32_ATOMIC accumulates into a caller-provided fp32 buffer"
    if not a.is_cuda:
        return _ref(a, b, a_mn, b_mn, bias, aux, epi, alpha, out, out_dtype)

    assert a.stride(1) == 1 and b.stride(1) == 1
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() >= N
    ld_aux = 0
    if epi in (EPI_RELU_MASK, EPI_DSILU):
        assert aux is not None and aux.dtype == a.dtype and aux.shape == (M, N) and aux.stride(1) == 1
        ld_aux = aux.stride(0)
    rc = _lib.lib().rb_gemm16(
        a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(), b.stride(0), int(b_mn),
        out.data_ptr(), out.stride(0), M, N, K, _lib.ptr(bias), _lib.ptr(aux), ld_aux, epi, float(alpha),
        int(splits), int(a.dtype == torch.bfloat16), _lib.num_sms(a.device), _lib.ptr(colsum_out),
        _lib.status_tensor(a.device).data_ptr(), _lib.stream_ptr(a.device))
    _lib.check(rc, "rb_gemm16")
    return out


def pick_splits(M: int, N: int, K: int, num_sms: int = 148) -> int:
    """Split-K factor for a weight-gradient GEMM (small M x N, long contraction) on the persistent kernel: work items
    (tiles x splits) run in rounds of ``num_sms``; an item costs its k-blocks plus a fixed epilogue (the fp32 vector
    reductions of a 128 x BN tile, about eight k-blocks' worth).  Pick the split count with the shortest schedule."""
    bn = 256 if N > 128 else (128 if N > 64 else 64)
    tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
    kb = (K + 63) // 64
    if tiles >= num_sms or kb <= 8:
        return 1
    best, best_cost = 1, None
    for s in range(1, min(kb, 64) + 1):
        rounds = (tiles * s + num_sms - 1) // num_sms
        cost = rounds * ((kb + s - 1) // s + 8)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best

"""Row-wise HSTU helper ops on ``csrc/cuda/hstu_misc.cu`` with PyTorch fallbacks for CPU tensors:
``ln_mul`` (LayerNorm(x) * u, optional dropout = ``norm_multiply_dropout``), relative attention bias
(time / position, dense form for API parity), jagged <-> padded, 2-D jagged concat / split, reverse_sequence,
1-D gather with scatter-add gradient, ``matmul_nt`` (differentiable ``a @ b^T`` on the tcgen05 GEMM)."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import _lib, gemm


# ----------------------------------------------------------------------------- ln_mul
class _LnMulFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, u, gamma, beta, eps: float, drop: float, seed: int):
        rows, C = x.shape
        out = torch.empty_like(x)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = _lib.lib().rb_ln_mul_fwd(x.data_ptr(), _lib.ptr(u), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(),
                                      mean.data_ptr(), rstd.data_ptr(), rows, C, eps, drop, seed, _lib.dtype_code(x.dtype),
                                      _lib.stream_ptr(x.device))
        _lib.check(rc, "rb_ln_mul_fwd")
        ctx.save_for_backward(x, u if u is not None else x.new_zeros(0), gamma, beta, mean, rstd)
        ctx.has_u, ctx.drop, ctx.seed = u is not None, drop, seed
        return out

    @staticmethod
    def backward(ctx, dy):
        x, u, gamma, beta, mean, rstd = ctx.saved_tensors
        u = u if ctx.has_u else None
        rows, C = x.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        du = torch.empty_like(x) if u is not None else None
        dg = torch.zeros(C, dtype=torch.float32, device=x.device)
        db = torch.zeros(C, dtype=torch.float32, device=x.device)
        rc = _lib.lib().rb_ln_mul_bwd(dy.data_ptr(), x.data_ptr(), _lib.ptr(u), gamma.data_ptr(), beta.data_ptr(),
                                      mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), _lib.ptr(du), dg.data_ptr(),
                                      db.data_ptr(), rows, C, ctx.drop, ctx.seed, _lib.dtype_code(x.dtype),
                                      _lib.num_sms(x.device), _lib.stream_ptr(x.device))
        _lib.check(rc, "rb_ln_mul_bwd")
        return dx, du, dg, db, None, None, None


def ln_mul(x: torch.Tensor, u: Optional[torch.Tensor], gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5,
           dropout_ratio: float = 0.0, seed: int = 0) -> torch.Tensor:
    """``Dropout(LayerNorm(x; gamma, beta) * u)`` over the last dim of a 2-D tensor (fp32 or bf16; gamma/beta fp32)."""
    if not x.is_cuda or x.dtype not in (torch.float32, torch.bfloat16) or x.shape[1] > 2048:
        y = torch.nn.functional.layer_norm(x.float(), (x.shape[1],), gamma.float(), beta.float(), eps)
        if u is not None:
            y = y * u.float()
        if dropout_ratio > 0:
            y = torch.nn.functional.dropout(y, dropout_ratio, True)
        return y.to(x.dtype)
    return _LnMulFn.apply(x.contiguous(), None if u is None else u.contiguous(), gamma.float().contiguous(),
                          beta.float().contiguous(), eps, dropout_ratio, seed)


# ----------------------------------------------------------------------------- matmul on the tcgen05 GEMM
class _MatmulNT(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return gemm.gemm16(a, b)

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        dy = dy.contiguous()
        da = gemm.gemm16(dy, b, b_mn=True) if ctx.needs_input_grad[0] else None
        db = None
        if ctx.needs_input_grad[1]:
            db32 = torch.zeros(b.shape, dtype=torch.float32, device=b.device)
            gemm.gemm16(dy, a, a_mn=True, b_mn=True, out=db32, epi=gemm.EPI_F32_ATOMIC,
                        splits=gemm.pick_splits(b.shape[0], b.shape[1], a.shape[0]))
            db = db32.to(b.dtype)
        return da, db


def matmul_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a [M,K] @ b[N,K]^T`` (bf16 / fp16, K and N multiples of 8), differentiable, on the tcgen05 GEMM."""
    if not a.is_cuda:
        return (a.float() @ b.float().t()).to(a.dtype)
    return _MatmulNT.apply(a.contiguous(), b.contiguous())


# ----------------------------------------------------------------------------- relative attention bias (dense)
def relative_attn_bias_time(timestamps: torch.Tensor, timestamps_weights: torch.Tensor, bucket_divisor: float,
                            with_index: bool = False):
    """timestamps [B,S], weights [L, num_buckets+1] -> rab [L,B,S,S] (and the bucket index [B,S,S])."""
    B, S = timestamps.shape
    L, nb1 = timestamps_weights.shape
    if not timestamps.is_cuda:
        dt = timestamps.float()[:, :, None] - timestamps.float()[:, None, :]
        bk = torch.clamp(torch.floor(torch.log(dt.abs().clamp(1.0, 7.0e16)) / bucket_divisor), 0, nb1 - 1).long()
        out = timestamps_weights.float()[:, bk]
        return (out, bk.int()) if with_index else out
    out = torch.empty(L, B, S, S, dtype=torch.float32, device=timestamps.device)
    bk = torch.empty(B, S, S, dtype=torch.int32, device=timestamps.device) if with_index else None
    rc = _lib.lib().rb_rab_time_fwd(timestamps.float().contiguous().data_ptr(), timestamps_weights.float().contiguous().data_ptr(),
                                    L, B, S, nb1 - 1, float(bucket_divisor), out.data_ptr(), _lib.ptr(bk),
                                    _lib.num_sms(out.device), _lib.stream_ptr(out.device))
    _lib.check(rc, "rb_rab_time_fwd")
    return (out, bk) if with_index else out


def relative_attn_bias_time_backward(rab_time_grad: torch.Tensor, bucket_timestamps: torch.Tensor, num_buckets: int):
    """grad [L,B,S,S], buckets [B,S,S] -> d weights [L, num_buckets+1] (scatter-add by bucket)."""
    L = rab_time_grad.shape[0]
    per = bucket_timestamps.numel()
    if not rab_time_grad.is_cuda:
        dw = torch.zeros(L, num_buckets + 1)
        dw.index_add_(1, bucket_timestamps.reshape(-1).long(), rab_time_grad.float().reshape(L, -1))
        return dw
    dw = torch.zeros(L, num_buckets + 1, dtype=torch.float32, device=rab_time_grad.device)
    rc = _lib.lib().rb_rab_time_bwd(rab_time_grad.float().contiguous().data_ptr(), bucket_timestamps.int().contiguous().data_ptr(),
                                    L, per, num_buckets, dw.data_ptr(), _lib.num_sms(dw.device), _lib.stream_ptr(dw.device))
    _lib.check(rc, "rb_rab_time_bwd")
    return dw


def relative_attn_bias_pos(rel_pos_bias: torch.Tensor, identity: torch.Tensor, past_valid_lens: List[int]) -> torch.Tensor:
    """bias [S,S] repeated per batch; rows >= valid length take row ``valid``; identity positions take ``bias[0,0]``;
    cropped to ``identity.shape``."""
    S, s, B = rel_pos_bias.shape[0], identity.shape[0], len(past_valid_lens)
    if not rel_pos_bias.is_cuda:
        out = rel_pos_bias.float()[None].repeat(B, 1, 1)
        for b, v in enumerate(past_valid_lens):
            out[b, v:] = out[b, min(v, S - 1)].clone()
        out = out[:, :s, :s]
        return out * (1 - identity.float()) + identity.float() * rel_pos_bias.float()[0, 0]
    out = torch.empty(B, s, s, dtype=torch.float32, device=rel_pos_bias.device)
    vl = torch.tensor(past_valid_lens, dtype=torch.int32, device=out.device)
    rc = _lib.lib().rb_rab_pos(rel_pos_bias.float().contiguous().data_ptr(), S, identity.float().contiguous().data_ptr(), s,
                               vl.data_ptr(), B, out.data_ptr(), _lib.num_sms(out.device), _lib.stream_ptr(out.device))
    _lib.check(rc, "rb_rab_pos")
    return out


# ----------------------------------------------------------------------------- jagged data movement
def jagged_to_padded(values: torch.Tensor, offsets: torch.Tensor, max_len: int, pad: float = 0.0) -> torch.Tensor:
    B, D = offsets.numel() - 1, values.shape[1]
    out = torch.empty(B, max_len, D, dtype=values.dtype, device=values.device)
    if not values.is_cuda:
        out.fill_(pad)
        o = offsets.tolist()
        for b in range(B):
            n = min(o[b + 1] - o[b], max_len)
            out[b, :n] = values[o[b]:o[b] + n]
        return out
    rc = _lib.lib().rb_jagged_to_padded(values.contiguous().data_ptr(), offsets.long().contiguous().data_ptr(), B, max_len, D,
                                        out.data_ptr(), pad, _lib.dtype_code(values.dtype), _lib.num_sms(out.device),
                                        _lib.stream_ptr(out.device))
    _lib.check(rc, "rb_jagged_to_padded")
    return out


def padded_to_jagged(padded: torch.Tensor, offsets: torch.Tensor, total: int) -> torch.Tensor:
    B, S, D = padded.shape
    out = torch.empty(total, D, dtype=padded.dtype, device=padded.device)
    if not padded.is_cuda:
        o = offsets.tolist()
        for b in range(B):
            out[o[b]:o[b + 1]] = padded[b, : o[b + 1] - o[b]]
        return out
    rc = _lib.lib().rb_padded_to_jagged(padded.contiguous().data_ptr(), offsets.long().contiguous().data_ptr(), B, S, D,
                                        out.data_ptr(), _lib.dtype_code(padded.dtype), _lib.num_sms(out.device),
                                        _lib.stream_ptr(out.device))
    _lib.check(rc, "rb_padded_to_jagged")
    return out


def concat_2d_jagged(values_a: torch.Tensor, values_b: torch.Tensor, offsets_a: torch.Tensor, offsets_b: torch.Tensor):
    """Per sample: rows of A followed by rows of B -> (values, offsets)."""
    off = offsets_a + offsets_b
    D = values_a.shape[1]
    out = torch.empty(values_a.shape[0] + values_b.shape[0], D, dtype=values_a.dtype, device=values_a.device)
    if not values_a.is_cuda:
        oa, ob, oo = offsets_a.tolist(), offsets_b.tolist(), off.tolist()
        for b in range(len(oa) - 1):
            la = oa[b + 1] - oa[b]
            out[oo[b]:oo[b] + la] = values_a[oa[b]:oa[b + 1]]
            out[oo[b] + la:oo[b + 1]] = values_b[ob[b]:ob[b + 1]]
        return out, off
    a, b = values_a.contiguous(), values_b.contiguous()
    rc = _lib.lib().rb_concat_2d_jagged(a.data_ptr(), b.data_ptr(), offsets_a.long().contiguous().data_ptr(),
                                        offsets_b.long().contiguous().data_ptr(), offsets_a.numel() - 1, D, out.data_ptr(), 0,
                                        _lib.dtype_code(a.dtype), _lib.stream_ptr(a.device))
    _lib.check(rc, "rb_concat_2d_jagged")
    return out, off


def split_2d_jagged(values: torch.Tensor, offsets_a: torch.Tensor, offsets_b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    D = values.shape[1]
    na, nb = int(offsets_a[-1].item()), int(offsets_b[-1].item())
    a = torch.empty(na, D, dtype=values.dtype, device=values.device)
    b = torch.empty(nb, D, dtype=values.dtype, device=values.device)
    if not values.is_cuda:
        oa, ob = offsets_a.tolist(), offsets_b.tolist()
        for i in range(len(oa) - 1):
            o0, la = oa[i] + ob[i], oa[i + 1] - oa[i]
            a[oa[i]:oa[i + 1]] = values[o0:o0 + la]
            b[ob[i]:ob[i + 1]] = values[o0 + la:o0 + la + ob[i + 1] - ob[i]]
        return a, b
    rc = _lib.lib().rb_concat_2d_jagged(a.data_ptr(), b.data_ptr(), offsets_a.long().contiguous().data_ptr(),
                                        offsets_b.long().contiguous().data_ptr(), offsets_a.numel() - 1, D,
                                        values.contiguous().data_ptr(), 1, _lib.dtype_code(values.dtype),
                                        _lib.stream_ptr(values.device))
    _lib.check(rc, "rb_concat_2d_jagged")
    return a, b


def reverse_sequence(x: torch.Tensor, seq_lengths: torch.Tensor) -> torch.Tensor:
    """x [B,S,D]: reverse the first ``len_b`` positions of every sample."""
    B, S = x.shape[0], x.shape[1]
    xc = x.contiguous().view(B, S, -1)
    if not x.is_cuda:
        out = xc.clone()
        for b, n in enumerate(seq_lengths.tolist()):
            out[b, :n] = xc[b, :n].flip(0)
        return out.view_as(x)
    out = torch.empty_like(xc)
    rc = _lib.lib().rb_reverse_sequence(xc.data_ptr(), seq_lengths.long().contiguous().data_ptr(), B, S, xc.shape[2],
                                        out.data_ptr(), _lib.dtype_code(x.dtype), _lib.num_sms(x.device), _lib.stream_ptr(x.device))
    _lib.check(rc, "rb_reverse_sequence")
    return out.view_as(x)


class _Gather1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, index):
        ctx.save_for_backward(index)
        ctx.n = x.numel()
        out = torch.empty(index.numel(), dtype=torch.float32, device=x.device)
        rc = _lib.lib().rb_gather1d(x.data_ptr(), index.data_ptr(), index.numel(), out.data_ptr(), _lib.num_sms(x.device),
                                    _lib.stream_ptr(x.device))
        _lib.check(rc, "rb_gather1d")
        return out

    @staticmethod
    def backward(ctx, g):
        (index,) = ctx.saved_tensors
        dx = torch.zeros(ctx.n, dtype=torch.float32, device=g.device)
        rc = _lib.lib().rb_scatter_add1d(g.contiguous().data_ptr(), index.data_ptr(), index.numel(), dx.data_ptr(),
                                         _lib.num_sms(g.device), _lib.stream_ptr(g.device))
        _lib.check(rc, "rb_scatter_add1d")
        return dx, None


def gather_for_rank1(x: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """1-D ``index_select`` (fp32) whose gradient is a scatter-add."""
    if not x.is_cuda:
        return x.index_select(0, index.long())
    return _Gather1d.apply(x.float().contiguous(), index.long().contiguous())


def multislice_concat(x: torch.Tensor, slice_begin: List[int], slice_size: List[int]) -> torch.Tensor:
    """Concatenate column slices ``x[:, b:b+n]`` of a 2-D tensor (one kernel launch on the GPU)."""
    from .model_ops import multislice_concat as _msc

    return _msc(x, [(int(b), int(b) + int(n)) for b, n in zip(slice_begin, slice_size)])


def token_mixing(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, epsilon: float = 1e-7) -> torch.Tensor:
    """``LayerNorm(x + x^T)`` on ``[B,S,S]``."""
    B, S, _ = x.shape
    y = (x + x.transpose(1, 2)).reshape(B * S, S)
    return ln_mul(y.contiguous(), None, gamma, beta, epsilon).view(B, S, S)

"""HSTU jagged / paged SiLU attention.

``hstu_attention`` (autograd-capable) and ``hstu_attention_paged`` run the tcgen05 forward kernel
(``csrc/cuda/hstu_attention_fwd.cu``); ``hstu_attention_ref`` is the fp32 PyTorch statement of the same
math (mask generator and operation order of the reference golden, ``build/presmoke/hstu/hstu_common.py:
108-153,286-345``) and serves CPU tensors, the tests and the gradient of the fused forward.

The relative bias is ``ts_w[bucket(ts_i - ts_j)] + pos_w[clamp(i - j, 0, len(pos_w) - 1)]`` with
``bucket = clamp(floor(log(clamp(|dt|, 1, e^38.8)) / divisor), 0, num_buckets)``
(``relative_attn_bias_time/v220/README.md:34-68``), evaluated inside the kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib


def hstu_mask(len_q: int, len_k: int, causal: bool, num_context: int, num_target: int, group_size: int,
              device=None) -> torch.Tensor:
    if not causal:
        return torch.ones(len_q, len_k, device=device)
    m = torch.tril(torch.ones(len_q, len_k, device=device), diagonal=len_k - len_q)
    if num_context > 0:
        m[:num_context, : len_k - num_target] = 1
    if group_size > 0 and num_target > 0:
        idx = torch.arange(num_target, device=device)
        tm = (idx[:, None] >= idx[None, :]) & ((idx[:, None] // group_size) == (idx[None, :] // group_size))
        nq = min(num_target, len_q)
        m[len_q - nq:, len_k - num_target:] = tm[num_target - nq:].to(m.dtype)
    return m


def time_buckets(dt: torch.Tensor, divisor: float, num_buckets: int) -> torch.Tensor:
    a = dt.abs().clamp(min=1.0, max=7.0e16)
    return torch.clamp(torch.floor(torch.log(a) / divisor), 0, num_buckets).long()


def hstu_attention_ref(q, k, v, q_offsets, k_offsets, alpha: float, scale: float, causal: bool = True,
                       num_context=None, num_target=None, target_group_size: int = 0, ts=None, ts_w=None,
                       ts_divisor: float = 0.301, pos_w=None) -> torch.Tensor:
    """q [Tq,H,D], k/v [Tk,H,D] jagged by the offsets; fp32 math, P is cast to the input dtype before P V."""
    H, D = q.shape[1], q.shape[2]
    out = torch.zeros(q.shape[0], H, v.shape[2], dtype=torch.float32, device=q.device)
    qo, ko = q_offsets.tolist(), k_offsets.tolist()
    for b in range(len(qo) - 1):
        lq, lk = qo[b + 1] - qo[b], ko[b + 1] - ko[b]
        if lq == 0:
            continue
        qq = q[qo[b]:qo[b + 1]].float().transpose(0, 1)
        kk = k[ko[b]:ko[b + 1]].float().transpose(0, 1)
        vv = v[ko[b]:ko[b + 1]].float().transpose(0, 1)
        s = qq @ kk.transpose(1, 2)                                  # [H, lq, lk]
        pi = torch.arange(lq, device=q.device) + (lk - lq)
        j = torch.arange(lk, device=q.device)
        if ts is not None and ts_w is not None:
            t = ts[ko[b]:ko[b + 1]].float()
            bk = time_buckets(t[pi][:, None] - t[None, :], ts_divisor, ts_w.numel() - 1)
            s = s + ts_w.float()[bk][None]
        if pos_w is not None:
            d = (pi[:, None] - j[None, :]).clamp(0, pos_w.numel() - 1)
            s = s + pos_w.float()[d][None]
        p = torch.nn.functional.silu(s * alpha) * scale
        nc = int(num_context[b]) if num_context is not None else 0
        nt = int(num_target[b]) if num_target is not None else 0
        p = p * hstu_mask(lq, lk, causal, nc, nt, target_group_size, q.device)[None]
        p = p.to(q.dtype).float()
        out[qo[b]:qo[b + 1]] = (p @ vv).transpose(0, 1)
    return out.to(q.dtype)


def _i32(t: Optional[torch.Tensor], device) -> Optional[torch.Tensor]:
    if t is None:
        return None
    return t.to(device=device, dtype=torch.int32).contiguous()


def hstu_attn_fwd(q, k, v, q_offsets, k_offsets, max_len_q: int, alpha: float, scale: float, causal: bool = True,
                  num_context=None, num_target=None, target_group_size: int = 0, ts=None, ts_w=None,
                  ts_divisor: float = 0.301, pos_w=None, out: Optional[torch.Tensor] = None,
                  page_ids=None, page_indptr=None, page_size: int = 0, attn_bias: Optional[torch.Tensor] = None,
                  attn_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Forward kernel launch.  ``attn_bias`` / ``attn_mask``: dense ``[B, H or 1, S, S]`` operands indexed by (query
    position, key position) - the bias (bf16 / fp32) is added to ``Q K^T`` before the activation, the 0/1 mask (bool /
    uint8 / bf16 / fp32) multiplies the result; they replace the in-kernel time / position bias and are not paged.  ``q`` [Tq,H,D] (row stride may exceed H*D, e.g. a slice of a fused projection);
    ``k``/``v`` likewise, or - paged - both the cache tensor ``[pages, 2, page, H, D]``."""
    assert q.is_cuda and q.dtype == torch.bfloat16
    Tq, H, D = q.shape
    assert q.stride(2) == 1 and q.stride(1) == D
    dev = q.device
    qo, ko = _i32(q_offsets, dev), _i32(k_offsets, dev)
    if out is None:
        out = torch.empty(Tq, H, D, dtype=q.dtype, device=dev)
    paged = page_ids is not None
    if paged:
        cache = k
        assert cache.dim() == 5 and cache.is_contiguous()
        num_pages, ld_k, Tk = cache.shape[0], H * D, 0
        kp = vp = cache.data_ptr()
    else:
        assert k.stride(2) == 1 and k.stride(1) == D and v.stride(2) == 1 and v.stride(1) == D and k.stride(0) == v.stride(0)
        num_pages, ld_k, Tk = 0, k.stride(0), k.shape[0]
        kp, vp = k.data_ptr(), v.data_ptr()
    B = qo.numel() - 1
    nb = (ts_w.numel() - 1) if ts_w is not None else 0
    f32 = lambda t: None if t is None else t.to(device=dev, dtype=torch.float32).contiguous()  # noqa: E731
    ts_, tsw_, pw_ = f32(ts), f32(ts_w), f32(pos_w)
    nc, nt = _i32(num_context, dev), _i32(num_target, dev)
    pid, pip = _i32(page_ids, dev), _i32(page_indptr, dev)
    if attn_bias is not None or attn_mask is not None:
        if paged or ts_ is not None or pw_ is not None:
            raise ValueError("dense attn_bias / attn_mask cannot be combined with paged K/V or the in-kernel relative bias")

        def dense(t, kinds):
            if t is None:
                return None, 0, 0, 0, 0
            if t.dim() != 4 or t.shape[0] != B or t.shape[1] not in (1, H):
                raise ValueError("dense operand must be [B, H or 1, S, S], got %s" % (tuple(t.shape),))
            if t.dtype == torch.bool:
                t = t.to(torch.uint8)
            if t.dtype not in kinds:
                t = t.to(torch.float32)
            if t.stride(3) != 1:
                t = t.contiguous()
            keep.append(t)
            return t.data_ptr(), kinds[t.dtype], t.stride(0), (t.stride(1) if t.shape[1] == H else 0), t.stride(2)

        keep: list = []
        bp_, bk_, bsb, bsh, bld = dense(attn_bias, {torch.bfloat16: 1, torch.float32: 2})
        mp_, mk_, msb, msh, mld = dense(attn_mask, {torch.uint8: 1, torch.bfloat16: 2, torch.float32: 3})
        rc = _lib.lib().rb_hstu_attn_fwd_dense(
            q.data_ptr(), q.stride(0), Tq, kp, vp, ld_k, Tk, qo.data_ptr(), ko.data_ptr(), B, H, D, int(max_len_q),
            out.data_ptr(), out.stride(0), float(alpha), float(scale), int(causal), _lib.ptr(nc), _lib.ptr(nt),
            int(target_group_size), bp_, bk_, bsb, bsh, bld, mp_, mk_, msb, msh, mld,
            min(t.shape[2] for t in keep), min(t.shape[3] for t in keep),
            _lib.status_tensor(dev).data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc, "rb_hstu_attn_fwd_dense")
        return out
    rc = _lib.lib().rb_hstu_attn_fwd(
        q.data_ptr(), q.stride(0), Tq, kp, vp, ld_k, Tk, qo.data_ptr(), ko.data_ptr(), B, H, D, int(max_len_q),
        out.data_ptr(), out.stride(0), float(alpha), float(scale), int(causal), _lib.ptr(nc), _lib.ptr(nt),
        int(target_group_size), _lib.ptr(ts_), _lib.ptr(tsw_), nb, float(ts_divisor), _lib.ptr(pw_),
        pw_.numel() if pw_ is not None else 0, _lib.ptr(pid), _lib.ptr(pip), int(page_size), num_pages,
        _lib.status_tensor(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "rb_hstu_attn_fwd")
    return out


class _HstuAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, ts_w, pos_w, q_offsets, k_offsets, max_len_q, alpha, scale, causal, num_context,
                num_target, gs, ts, divisor):
        out = hstu_attn_fwd(q, k, v, q_offsets, k_offsets, max_len_q, alpha, scale, causal, num_context, num_target, gs,
                            ts, ts_w, divisor, pos_w)
        ctx.save_for_backward(q, k, v, ts_w if ts_w is not None else q.new_zeros(0),
                              pos_w if pos_w is not None else q.new_zeros(0))
        ctx.meta = (q_offsets, k_offsets, alpha, scale, causal, num_context, num_target, gs, ts, divisor,
                    ts_w is not None, pos_w is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, ts_w, pos_w = ctx.saved_tensors
        qo, ko, alpha, scale, causal, nc, nt, gs, ts, divisor, has_t, has_p = ctx.meta
        from .hstu_attention_bwd import hstu_attn_bwd

        dq, dk, dv, dtw, dpw = hstu_attn_bwd(dout, q, k, v, qo, ko, alpha, scale, causal, nc, nt, gs, ts,
                                             ts_w if has_t else None, divisor, pos_w if has_p else None)
        return (dq, dk, dv, dtw, dpw) + (None,) * 11


def hstu_attention(q, k, v, q_offsets, k_offsets=None, max_len_q: Optional[int] = None, alpha: float = 1.0,
                   scale: float = 0.0, causal: bool = True, num_context=None, num_target=None,
                   target_group_size: int = 0, ts=None, ts_w=None, ts_divisor: float = 0.301, pos_w=None) -> torch.Tensor:
    """Differentiable HSTU attention over jagged ``[T, H, D]`` tensors.  ``scale == 0`` means ``1 / max_len_q``."""
    k_offsets = q_offsets if k_offsets is None else k_offsets
    if max_len_q is None:
        max_len_q = int((q_offsets[1:] - q_offsets[:-1]).max().item())
    if scale == 0.0:
        scale = 1.0 / max(max_len_q, 1)
    if not q.is_cuda or q.dtype != torch.bfloat16 or q.shape[2] not in (64, 128) or v.shape[2] != q.shape[2] \
            or k.shape[1] != q.shape[1]:
        return hstu_attention_ref(q, k, v, q_offsets, k_offsets, alpha, scale, causal, num_context, num_target,
                                  target_group_size, ts, ts_w, ts_divisor, pos_w)
    return _HstuAttnFn.apply(q, k, v, ts_w, pos_w, q_offsets, k_offsets, max_len_q, alpha, scale, causal, num_context,
                             num_target, target_group_size, ts, ts_divisor)


def hstu_attention_paged(q, kv_cache, q_offsets, k_offsets, page_ids, page_indptr, page_size: int, max_len_q: int,
                         alpha: float, scale: float, num_target=None, target_group_size: int = 0, ts=None, ts_w=None,
                         ts_divisor: float = 0.301, pos_w=None) -> torch.Tensor:
    """Inference: queries (the new tokens and candidates, a suffix of every user's key positions) against K/V held
    in the paged cache ``[pages, 2, page, H, D]``; the new tokens' K/V must already be appended to their pages."""
    return hstu_attn_fwd(q, kv_cache, kv_cache, q_offsets, k_offsets, max_len_q, alpha, scale, True, None, num_target,
                         target_group_size, ts, ts_w, ts_divisor, pos_w, page_ids=page_ids, page_indptr=page_indptr,
                         page_size=page_size)

"""Backward of HSTU attention.

``hstu_attn_bwd`` returns (dQ, dK, dV, d ts_w, d pos_w).  Math (``build/presmoke/hstu/hstu_common.py:387-477``):
with ``x = alpha (Q K^T + bias)``, ``P = SiLU(x) scale mask``: ``dV = P^T dO``, ``dP = dO V^T``,
``dS = dP scale mask alpha sigma(x) (1 + x (1 - sigma(x)))``, ``dQ = dS K``, ``dK = dS^T Q``, ``dBias = dS``
(scatter-added into the time-bucket and position tables).

``hstu_attn_bwd`` runs the tcgen05 kernel (``csrc/cuda/hstu_attention_bwd.cu``: head dim 64, bf16, CUDA);
``hstu_attn_bwd_ref`` evaluates the same formulas per sequence with batched PyTorch matmuls in fp32 (chunked
over query rows so the [H, chunk, len] score block stays small) and serves every other case and the tests.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .hstu_attention import hstu_mask, time_buckets


def hstu_attn_bwd(dout, q, k, v, q_offsets, k_offsets, alpha: float, scale: float, causal: bool, num_context,
                  num_target, gs: int, ts, ts_w, ts_divisor: float, pos_w, max_len_k: Optional[int] = None,
                  want_dts: bool = True, want_dpos: bool = True):
    """-> (dq, dk, dv, d_ts_w, d_pos_w); the bias gradients are None when not wanted (or when there is no such bias)."""
    ok = (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[2] == 64 and v.shape[2] == 64 and k.shape[1] == q.shape[1]
          and (pos_w is None or pos_w.numel() <= 4096) and (ts_w is None or ts_w.numel() <= 192))
    if not ok:
        return hstu_attn_bwd_ref(dout, q, k, v, q_offsets, k_offsets, alpha, scale, causal, num_context, num_target, gs,
                                 ts, ts_w, ts_divisor, pos_w)
    dev = q.device
    Tq, H, D = q.shape
    Tk = k.shape[0]
    i32 = lambda t: None if t is None else t.to(device=dev, dtype=torch.int32).contiguous()  # noqa: E731
    f32 = lambda t: None if t is None else t.to(device=dev, dtype=torch.float32).contiguous()  # noqa: E731
    qo, ko = i32(q_offsets), i32(k_offsets)
    if max_len_k is None:
        max_len_k = int((ko[1:] - ko[:-1]).max().item())
    dout = dout if (dout.stride(2) == 1 and dout.stride(1) == D) else dout.contiguous()
    assert q.stride(2) == 1 and q.stride(1) == D and k.stride(1) == D and v.stride(1) == D and k.stride(0) == v.stride(0)
    dq32 = torch.zeros(Tq, H * D, dtype=torch.float32, device=dev)
    dk = torch.empty(Tk, H, D, dtype=q.dtype, device=dev)
    dv = torch.empty(Tk, H, D, dtype=q.dtype, device=dev)
    ts_, tsw_, pw_ = f32(ts), f32(ts_w), f32(pos_w)
    dtw = torch.zeros_like(tsw_) if (want_dts and tsw_ is not None and ts_ is not None) else None
    dpw = torch.zeros_like(pw_) if (want_dpos and pw_ is not None) else None
    nc, nt = i32(num_context), i32(num_target)
    rc = _lib.lib().rb_hstu_attn_bwd(
        q.data_ptr(), q.stride(0), dout.data_ptr(), dout.stride(0), Tq, k.data_ptr(), v.data_ptr(), k.stride(0), Tk,
        qo.data_ptr(), ko.data_ptr(), qo.numel() - 1, H, D, max_len_k, float(alpha), float(scale), int(causal),
        _lib.ptr(nc), _lib.ptr(nt), int(gs), _lib.ptr(ts_), _lib.ptr(tsw_), (tsw_.numel() - 1) if tsw_ is not None else 0,
        float(ts_divisor), _lib.ptr(pw_), pw_.numel() if pw_ is not None else 0, dq32.data_ptr(), dq32.stride(0),
        dk.data_ptr(), dv.data_ptr(), dk.stride(0), _lib.ptr(dtw), _lib.ptr(dpw), _lib.status_tensor(dev).data_ptr(),
        _lib.stream_ptr(dev))
    _lib.check(rc, "rb_hstu_attn_bwd")
    return dq32.view(Tq, H, D).to(q.dtype), dk, dv, dtw, dpw


def hstu_attn_bwd_ref(dout, q, k, v, q_offsets, k_offsets, alpha: float, scale: float, causal: bool, num_context,
                      num_target, gs: int, ts, ts_w, ts_divisor: float, pos_w, chunk: int = 1024):
    H, D = q.shape[1], q.shape[2]
    dq = torch.zeros_like(q, dtype=torch.float32)
    dk = torch.zeros_like(k, dtype=torch.float32)
    dv = torch.zeros_like(v, dtype=torch.float32)
    dtw = torch.zeros_like(ts_w, dtype=torch.float32) if ts_w is not None else None
    dpw = torch.zeros_like(pos_w, dtype=torch.float32) if pos_w is not None else None
    qo, ko = q_offsets.tolist(), k_offsets.tolist()
    for b in range(len(qo) - 1):
        lq, lk = qo[b + 1] - qo[b], ko[b + 1] - ko[b]
        if lq == 0:
            continue
        kk = k[ko[b]:ko[b + 1]].float().transpose(0, 1)             # [H, lk, D]
        vv = v[ko[b]:ko[b + 1]].float().transpose(0, 1)
        nc = int(num_context[b]) if num_context is not None else 0
        nt = int(num_target[b]) if num_target is not None else 0
        mask_full = hstu_mask(lq, lk, causal, nc, nt, gs, q.device)
        t = ts[ko[b]:ko[b + 1]].float() if (ts is not None and ts_w is not None) else None
        j = torch.arange(lk, device=q.device)
        for r0 in range(0, lq, chunk):
            r1 = min(lq, r0 + chunk)
            qq = q[qo[b] + r0:qo[b] + r1].float().transpose(0, 1)     # [H, c, D]
            go = dout[qo[b] + r0:qo[b] + r1].float().transpose(0, 1)
            pi = torch.arange(r0, r1, device=q.device) + (lk - lq)
            s = qq @ kk.transpose(1, 2)
            bk = dd = None
            if t is not None:
                bk = time_buckets(t[pi][:, None] - t[None, :], ts_divisor, ts_w.numel() - 1)
                s = s + ts_w.float()[bk][None]
            if pos_w is not None:
                dd = (pi[:, None] - j[None, :]).clamp(0, pos_w.numel() - 1)
                s = s + pos_w.float()[dd][None]
            x = s * alpha
            sig = torch.sigmoid(x)
            m = mask_full[r0:r1][None]
            p = (x * sig * scale * m).to(q.dtype).float()
            dv[ko[b]:ko[b + 1]] += (p.transpose(1, 2) @ go).transpose(0, 1)
            dp = go @ vv.transpose(1, 2)
            ds = (dp * scale * m * alpha * sig * (1 + x * (1 - sig))).to(q.dtype).float()
            dq[qo[b] + r0:qo[b] + r1] = (ds @ kk).transpose(0, 1)
            dk[ko[b]:ko[b + 1]] += (ds.transpose(1, 2) @ qq).transpose(0, 1)
            if dtw is not None or dpw is not None:
                dsum = ds.sum(0) / alpha * alpha                      # dBias = dS (already includes alpha)
                if dtw is not None:
                    dtw.index_add_(0, bk.reshape(-1), dsum.reshape(-1))
                if dpw is not None:
                    dpw.index_add_(0, dd.reshape(-1), dsum.reshape(-1))
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dtw, dpw

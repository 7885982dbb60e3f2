"""Backward of HSTU attention.

``hstu_attn_bwd`` returns (dQ, dK, dV, d ts_w, d pos_w).  Math (``build/presmoke/hstu/hstu_common.py:387-477``):
with ``x = alpha (Q K^T + bias)``, ``P = SiLU(x) scale mask``: ``dV = P^T dO``, ``dP = dO V^T``,
``dS = dP scale mask alpha sigma(x) (1 + x (1 - sigma(x)))``, ``dQ = dS K``, ``dK = dS^T Q``, ``dBias = dS``
(scatter-added into the time-bucket and position tables).

This module evaluates those formulas per sequence with batched PyTorch matmuls in fp32 (chunked over query
rows so the [H, chunk, len] score block stays small).
"""
from __future__ import annotations

from typing import Optional

import torch

from .hstu_attention import hstu_mask, time_buckets


def hstu_attn_bwd(dout, q, k, v, q_offsets, k_offsets, alpha: float, scale: float, causal: bool, num_context,
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

"""HSTU generative recommender: jagged sequences of item ids -> stacked HSTU layers -> sampled-softmax
next-item loss.

Layer (the doc-level HSTU layer of the reference, ``docs/en/torch/torch_rec_v2/04_migration_and_training/
migration_and_training.md:234-282``):

    uvqk = SiLU(Linear(LayerNorm(x)));  u, v, q, k = split(uvqk)
    a    = hstu_attention(q, k, v; causal, alpha = 1/sqrt(d_head), scale = 1/max_len, rel pos + time bias)
    x    = x + Linear(LayerNorm(a) * u)

Projections run on the tcgen05 GEMM (``FusedMLP``), attention on the tcgen05 HSTU kernels with the bias
evaluated inside the kernel, the norm-gate on the fused row kernel.  Item embeddings come from a dynamic
hash-table collection (row-wise sharded); the loss scores the true next item against shared sampled
negatives.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional

import torch
from torch import nn

from ..modules.mlp import FusedMLP
from ..ops import hstu_ops, model_ops
from ..ops.hstu_attention import hstu_attention
from ..sparse.jagged_tensor import KeyedJaggedTensor


@dataclasses.dataclass
class HSTUConfig:
    num_layers: int = 8
    d_model: int = 512
    num_heads: int = 8
    head_dim: int = 64
    max_seq_len: int = 4096
    num_time_buckets: int = 128
    time_bucket_divisor: float = 0.301
    num_negatives: int = 512
    dropout: float = 0.0


class HSTULayer(nn.Module):
    def __init__(self, cfg: HSTUConfig, device, dtype=torch.bfloat16) -> None:
        super().__init__()
        self.cfg = cfg
        hd = cfg.num_heads * cfg.head_dim
        self.uvqk = FusedMLP(cfg.d_model, [4 * hd], final_activation=False, device=device, dtype=dtype)
        self.out = FusedMLP(hd, [cfg.d_model], final_activation=False, device=device, dtype=dtype)
        self.norm_in_w = nn.Parameter(torch.ones(cfg.d_model, device=device))
        self.norm_in_b = nn.Parameter(torch.zeros(cfg.d_model, device=device))
        self.norm_attn_w = nn.Parameter(torch.ones(hd, device=device))
        self.norm_attn_b = nn.Parameter(torch.zeros(hd, device=device))
        self.ts_w = nn.Parameter(torch.zeros(cfg.num_time_buckets + 1, device=device).normal_(0, 0.02))
        self.pos_w = nn.Parameter(torch.zeros(cfg.max_seq_len, device=device).normal_(0, 0.02))

    def forward(self, x: torch.Tensor, offsets: torch.Tensor, max_len: int, timestamps: Optional[torch.Tensor]) -> torch.Tensor:
        c = self.cfg
        H, Dh = c.num_heads, c.head_dim
        hd = H * Dh
        xn = hstu_ops.ln_mul(x, None, self.norm_in_w, self.norm_in_b)
        uvqk = torch.nn.functional.silu(self.uvqk(xn))
        u, v, q, k = uvqk.split(hd, dim=1)                 # one split: its backward is a single concatenation
        T = x.shape[0]
        a = hstu_attention(q.unflatten(1, (H, Dh)), k.unflatten(1, (H, Dh)), v.unflatten(1, (H, Dh)), offsets,
                           max_len_q=max_len, alpha=1.0 / math.sqrt(Dh), scale=1.0 / max_len, causal=True,
                           ts=timestamps, ts_w=self.ts_w if timestamps is not None else None,
                           ts_divisor=c.time_bucket_divisor, pos_w=self.pos_w)
        y = hstu_ops.ln_mul(a.reshape(T, hd), u.contiguous(), self.norm_attn_w, self.norm_attn_b,
                            dropout_ratio=c.dropout if self.training else 0.0)
        return x + self.out(y)


class HSTU(nn.Module):
    """``forward(items KJT (features "item" and "neg"), offsets, max_len, timestamps) -> loss``."""

    def __init__(self, cfg: HSTUConfig, embedding: nn.Module, device, dtype=torch.bfloat16) -> None:
        super().__init__()
        self.cfg, self.embedding, self.dtype = cfg, embedding, dtype
        self.layers = nn.ModuleList([HSTULayer(cfg, device, dtype) for _ in range(cfg.num_layers)])
        self.norm_out_w = nn.Parameter(torch.ones(cfg.d_model, device=device))
        self.norm_out_b = nn.Parameter(torch.zeros(cfg.d_model, device=device))

    def encode(self, x: torch.Tensor, offsets, max_len: int, timestamps) -> torch.Tensor:
        for layer in self.layers:
            x = layer(x, offsets, max_len, timestamps)
        return hstu_ops.ln_mul(x, None, self.norm_out_w, self.norm_out_b)

    def forward(self, features: KeyedJaggedTensor, offsets: torch.Tensor, max_len: int,
                timestamps: Optional[torch.Tensor] = None, global_tokens: Optional[int] = None,
                predict_positions: Optional[torch.Tensor] = None):
        """``predict_positions``: optional int64 indices of every token that is not the last of its sequence (the
        positions that have a next item to predict); passing them from the host side of the input pipeline keeps
        the step free of a device-to-host synchronisation."""
        emb = self.embedding(features)
        x0 = emb["item"].values().to(self.dtype)                      # [T, d]
        neg = emb["neg"].values().to(self.dtype)                      # [num_negatives, d]
        h = self.encode(x0, offsets, max_len, timestamps)
        # position t predicts the item at t + 1 of the same sequence
        if predict_positions is not None:
            keep = predict_positions
        else:
            T = x0.shape[0]
            last = torch.zeros(T, dtype=torch.bool, device=x0.device)
            last[offsets[1:] - 1] = True
            keep = (~last).nonzero(as_tuple=True)[0]
        hq = h[keep]
        pos = x0[keep + 1]
        denom = global_tokens if global_tokens else max(keep.numel(), 1)
        # one GEMM for the negative logits, then one fused pass: positive logit, log-sum-exp, loss and all gradients
        return model_ops.sampled_softmax_loss(hq, pos, neg, 1.0 / denom)

"""DCN v2: embedding bags + bottom MLP -> cross network (full-rank or low-rank) -> deep MLP -> logit, BCE loss.

    x0 = concat(bottom_mlp(dense), pooled embeddings)            [B, (F + 1) D]
    x_{l+1} = x0 * (W_l x_l + b_l) + x_l                         (low rank: W_l = U_l V_l^T)
    logit = head(deep_mlp(x_L))

On CUDA the linear maps run on the tcgen05 GEMM (bf16 operands, fp32 accumulation; bias in the epilogue), the
Hadamard-and-add is one fused elementwise kernel, and the gradient GEMMs read their operands in place
(MN-major).  The embedding collection may be any KJT -> KeyedTensor module (plain, hash, sharded, dynamic).
The reference ships no model code; this is the model of its dynamic-embedding benchmark configuration.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
from torch import nn

from ..ops import gemm
from ..ops import model_ops
from ..sparse.jagged_tensor import KeyedTensor


class _Linear16(torch.autograd.Function):
    """``y = x W^T + b`` on the 16-bit GEMM with fp32 master weights (``w16`` is their 16-bit shadow)."""

    @staticmethod
    def forward(ctx, x, w32, b32, w16):
        ctx.save_for_backward(x, w16)
        ctx.has_bias = b32 is not None
        return gemm.gemm16(x, w16, bias=b32)

    @staticmethod
    def backward(ctx, dy):
        x, w16 = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm.gemm16(dy, w16, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = torch.zeros(w16.shape, dtype=torch.float32, device=x.device)
        gemm.gemm16(dy, x, a_mn=True, b_mn=True, out=dw, epi=gemm.EPI_F32_ATOMIC, splits=gemm.pick_splits(w16.shape[0], w16.shape[1], x.shape[0]))
        db = dy.float().sum(0) if ctx.has_bias else None
        return dx, dw, db, None


class Linear16(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=torch.bfloat16) -> None:
        super().__init__()
        if in_features % 8 or out_features % 8:
            raise ValueError("Linear16 needs feature counts that are multiples of 8")
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device).uniform_(-1, 1) / in_features ** 0.5)
        self.bias = nn.Parameter(torch.zeros(out_features, device=device)) if bias else None
        self.dtype = dtype

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            return torch.nn.functional.linear(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))
        return _Linear16.apply(x, self.weight, self.bias, self.weight.detach().to(self.dtype))


class CrossNet(nn.Module):
    def __init__(self, width: int, num_layers: int, low_rank: int = 0, device=None, dtype=torch.bfloat16) -> None:
        super().__init__()
        self.low_rank = low_rank
        if low_rank:
            self.v = nn.ModuleList([Linear16(width, low_rank, bias=False, device=device, dtype=dtype) for _ in range(num_layers)])
            self.u = nn.ModuleList([Linear16(low_rank, width, bias=True, device=device, dtype=dtype) for _ in range(num_layers)])
        else:
            self.w = nn.ModuleList([Linear16(width, width, bias=True, device=device, dtype=dtype) for _ in range(num_layers)])

    def forward(self, x0: torch.Tensor) -> torch.Tensor:
        x = x0
        n = len(self.u) if self.low_rank else len(self.w)
        for l in range(n):
            y = self.u[l](self.v[l](x)) if self.low_rank else self.w[l](x)
            x = model_ops.dcn_cross_combine(x0, y, x)        # x0 * y + x: fused forward, one fused pass for all three gradients
        return x


class DCNv2(nn.Module):
    """``forward(dense [B, F_dense], sparse KJT) -> logits [B]``."""

    def __init__(self, embedding_bag_collection: nn.Module, dense_in_features: int, dense_arch_layer_sizes: Sequence[int],
                 cross_layers: int = 3, low_rank: int = 0, deep_layer_sizes: Sequence[int] = (1024, 512),
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16) -> None:
        super().__init__()
        dev = torch.device(device) if device is not None else torch.device("cpu")
        self.sparse_arch = embedding_bag_collection
        cfgs = embedding_bag_collection.embedding_bag_configs()
        self.sparse_width = sum(c.embedding_dim * len(c.feature_names) for c in cfgs)
        self.compute_dtype = dtype if dev.type == "cuda" else torch.float32
        dims = [(dense_in_features + 7) // 8 * 8] + list(dense_arch_layer_sizes)
        self.dense_pad = dims[0] - dense_in_features
        self.dense_arch = nn.ModuleList([Linear16(a, b, device=dev, dtype=dtype) for a, b in zip(dims[:-1], dims[1:])])
        width = self.sparse_width + dims[-1]
        if width % 8:
            raise ValueError("cross width must be a multiple of 8")
        self.cross = CrossNet(width, cross_layers, low_rank, dev, dtype)
        ddims = [width] + list(deep_layer_sizes)
        self.deep = nn.ModuleList([Linear16(a, b, device=dev, dtype=dtype) for a, b in zip(ddims[:-1], ddims[1:])])
        self.head = nn.Linear(ddims[-1], 1, device=dev)

    def forward(self, dense_features: torch.Tensor, sparse_features) -> torch.Tensor:
        x = dense_features.to(self.compute_dtype)
        if self.dense_pad:
            x = torch.nn.functional.pad(x, (0, self.dense_pad))
        for lin in self.dense_arch:
            x = torch.relu(lin(x))
        kt = self.sparse_arch(sparse_features)
        pooled = kt.values() if isinstance(kt, KeyedTensor) else kt
        x0 = torch.cat([x, pooled.to(self.compute_dtype)], dim=1)
        h = self.cross(x0)
        for lin in self.deep:
            h = torch.relu(lin(h))
        return self.head(h.float()).squeeze(1)


class DCNv2Train(nn.Module):
    """``forward(batch) -> (loss, (loss, logits, labels))`` with the BCE loss averaged over ``global_batch_size``."""

    def __init__(self, model: DCNv2, global_batch_size: Optional[int] = None) -> None:
        super().__init__()
        self.model = model
        self.global_batch_size = global_batch_size

    def forward(self, batch):
        logits = self.model(batch.dense_features, batch.sparse_features)
        labels = batch.labels.float()
        n = self.global_batch_size or labels.numel()
        loss = torch.nn.functional.binary_cross_entropy_with_logits(logits, labels, reduction="sum") / n
        return loss, (loss.detach(), logits.detach(), labels)

"""DLRM: bottom MLP over dense features, embedding bags over sparse features, pairwise dot
interaction, top MLP, BCE loss.

Two execution modes share one module tree:

* **fused** (CUDA, bf16): ``FusedMLP`` on the tcgen05 GEMM, the embedding collection's fused lookup,
  the ``dot_interaction`` kernel reading the bottom-MLP output and the pooled embeddings in place,
  and a single kernel for the last ``K -> 1`` layer + loss + its backward.
* **reference** (any device, fp32): plain PyTorch modules; used on CPU and as the numerical oracle.

The reference SDK ships no model code (its DLRM example lives outside the tree,
``README_en.md:78-85``); the architecture follows the standard DLRM used by its benchmarks configs.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
from torch import nn

from ..modules.mlp import MLP, FusedMLP
from ..ops import dense_ops
from ..ops.interaction import dot_interaction, dot_interaction_ref, interaction_out_cols
from ..sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor


class _BCEHeadFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h: torch.Tensor, head: "LogitHead", labels: torch.Tensor, inv_batch: float, relu_mask: bool,
                _anchor: torch.Tensor):
        B, K = h.shape
        loss = torch.zeros(1, dtype=torch.float32, device=h.device)
        logits = torch.empty(B, dtype=torch.float32, device=h.device)
        dh = torch.empty(B, K, dtype=h.dtype, device=h.device)
        dense_ops.bce_head(h, head.w32, head.b32, labels, inv_batch, logits, loss, dh, head.wgrad, head.bgrad,
                           relu_mask)
        ctx.save_for_backward(dh)
        ctx.mark_non_differentiable(logits)
        return loss.squeeze(0), logits

    @staticmethod
    def backward(ctx, gloss: torch.Tensor, _glogits):
        (dh,) = ctx.saved_tensors
        # the loss is the root of the backward pass; its incoming gradient is 1
        return dh, None, None, None, None, None


class LogitHead(nn.Module):
    """Final ``K -> 1`` linear layer fused with BCE-with-logits (fp32 master weights in a flat buffer)."""

    def __init__(self, in_features: int, device=None) -> None:
        super().__init__()
        self.in_features = in_features
        n = (in_features + 1 + 63) // 64 * 64
        self.flat_param = nn.Parameter(torch.zeros(n, dtype=torch.float32, device=device))
        self.register_buffer("flat_grad", torch.zeros(n, dtype=torch.float32, device=device), persistent=False)
        self._views()
        bound = 1.0 / in_features ** 0.5
        with torch.no_grad():
            self.w32.uniform_(-bound, bound)
            self.b32.uniform_(-bound, bound)

    def _views(self) -> None:
        K = self.in_features
        self.w32 = self.flat_param.data[:K]
        self.b32 = self.flat_param.data[K:K + 1]
        self.wgrad = self.flat_grad[:K]
        self.bgrad = self.flat_grad[K:K + 1]

    def _apply(self, fn, *a, **k):
        out = super()._apply(fn, *a, **k)
        if self.flat_grad.dtype != torch.float32:
            self.flat_grad = self.flat_grad.float()
        self._views()
        return out

    def set_grad_buffer(self, buf: torch.Tensor) -> None:
        buf.copy_(self.flat_grad)
        self.flat_grad = buf
        self._views()

    def forward(self, h: torch.Tensor, labels: torch.Tensor, inv_batch: float, relu_mask: bool = True):
        return _BCEHeadFn.apply(h, self, labels, inv_batch, relu_mask, self.flat_param)


class DLRM(nn.Module):
    """``forward(dense_features [B, F_dense], sparse_features: KJT) -> logits [B, 1]``.

    ``embedding_bag_collection`` is any module mapping a KJT to a ``KeyedTensor`` of pooled embeddings
    (plain, hash-mapped, sharded or dynamic).  All tables must share ``embedding_dim``, equal to the last
    bottom-MLP width.  ``over_arch_layer_sizes`` ends with 1 (the logit).
    """

    def __init__(self, embedding_bag_collection: nn.Module, dense_in_features: int,
                 dense_arch_layer_sizes: Sequence[int], over_arch_layer_sizes: Sequence[int],
                 dense_device: Optional[torch.device] = None, fused: Optional[bool] = None,
                 dtype: torch.dtype = torch.bfloat16) -> None:
        super().__init__()
        self.sparse_arch = embedding_bag_collection
        cfgs = embedding_bag_collection.embedding_bag_configs()
        self.num_sparse_features = sum(len(c.feature_names) for c in cfgs)
        self.D = cfgs[0].embedding_dim
        if any(c.embedding_dim != self.D for c in cfgs):
            raise ValueError("DLRM needs one embedding_dim for all tables")
        if dense_arch_layer_sizes[-1] != self.D:
            raise ValueError("last bottom-MLP width must equal embedding_dim")
        if over_arch_layer_sizes[-1] != 1:
            raise ValueError("over_arch_layer_sizes must end with 1")
        dev = torch.device(dense_device) if dense_device is not None else torch.device("cpu")
        self.fused = (dev.type == "cuda") if fused is None else fused
        self.F = self.num_sparse_features + 1
        self.n_tri = self.F * (self.F - 1) // 2
        self.dense_in_features = dense_in_features
        self.compute_dtype = dtype
        if self.fused:
            self.inter_cols = interaction_out_cols(self.F, self.D)
            self.dense_arch = FusedMLP(dense_in_features, dense_arch_layer_sizes, final_activation=True, device=dev,
                                       dtype=dtype)
            self.over_arch = FusedMLP(self.D + self.n_tri, over_arch_layer_sizes[:-1], final_activation=True,
                                      device=dev, dtype=dtype)
            assert self.over_arch.in_padded == self.inter_cols
            self.head = LogitHead(over_arch_layer_sizes[-2], device=dev)
        else:
            self.inter_cols = self.D + self.n_tri
            self.dense_arch = MLP(dense_in_features, dense_arch_layer_sizes, final_activation=True, device=dev)
            self.over_arch = MLP(self.inter_cols, over_arch_layer_sizes[:-1], final_activation=True, device=dev)
            self.head = nn.Linear(over_arch_layer_sizes[-2], 1, device=dev)

    # -- shared pieces -----------------------------------------------------------------
    def _pooled(self, sparse_features) -> torch.Tensor:
        kt = self.sparse_arch(sparse_features)
        return kt.values() if isinstance(kt, KeyedTensor) else kt

    def hidden(self, dense_features: torch.Tensor, sparse_features) -> torch.Tensor:
        """Everything up to (excluding) the logit layer."""
        if self.fused:
            # a sharded collection starts its exchange first (own stream), so the bottom MLP runs while ids and rows travel
            dist_ctx = self.sparse_arch.input_dist(sparse_features) if getattr(self.sparse_arch, "split_dist", False) else None
            x = dense_ops.cast_pad(dense_features, self.dense_arch.in_padded, self.compute_dtype)
            d = self.dense_arch(x, grad_premasked=True)     # the interaction backward applies the ReLU mask
            if dist_ctx is not None:
                kt = self.sparse_arch.compute_and_output_dist(dist_ctx)
                pooled = kt.values() if isinstance(kt, KeyedTensor) else kt
            else:
                pooled = self._pooled(sparse_features)
            if pooled.dtype != self.compute_dtype:
                pooled = pooled.to(self.compute_dtype)
            r = dot_interaction(d, pooled, self.F, self.inter_cols, mask_x0=True)
            return self.over_arch(r, grad_premasked=True)
        d = self.dense_arch(dense_features.float())
        pooled = self._pooled(sparse_features).float()
        B = d.shape[0]
        X = torch.cat([d.unsqueeze(1), pooled.reshape(B, self.F - 1, self.D)], dim=1)
        Z = torch.bmm(X, X.transpose(1, 2))
        i, j = torch.tril_indices(self.F, self.F, offset=-1, device=d.device)
        r = torch.cat([d, Z[:, i, j]], dim=1)
        return self.over_arch(r)

    def forward(self, dense_features: torch.Tensor, sparse_features) -> torch.Tensor:
        h = self.hidden(dense_features, sparse_features)
        if self.fused:
            return (h.float() @ self.head.w32 + self.head.b32).unsqueeze(1)
        return self.head(h)


class DLRMTrain(nn.Module):
    """Wraps a ``DLRM`` with the BCE-with-logits loss.  ``forward(batch)`` returns
    ``(loss, (loss.detach(), logits.detach(), labels))`` where ``batch`` has ``dense_features``,
    ``sparse_features`` and ``labels``.  ``global_batch_size`` sets the mean's denominator when the
    batch is split over data-parallel ranks (so summed gradients equal the global-mean gradient)."""

    def __init__(self, dlrm: DLRM, global_batch_size: Optional[int] = None) -> None:
        super().__init__()
        self.model = dlrm
        self.global_batch_size = global_batch_size

    def forward(self, batch) -> Tuple[torch.Tensor, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
        m = self.model
        labels = batch.labels
        h = m.hidden(batch.dense_features, batch.sparse_features)
        B = h.shape[0]
        denom = self.global_batch_size or B
        if m.fused:
            loss, logits = m.head(h, labels.float(), 1.0 / denom, relu_mask=True)
        else:
            logits = m.head(h).squeeze(1)
            loss = torch.nn.functional.binary_cross_entropy_with_logits(logits, labels.float(), reduction="sum") / denom
        return loss, (loss.detach(), logits.detach(), labels)

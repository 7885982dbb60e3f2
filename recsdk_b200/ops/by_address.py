"""Row IO by raw address and the sparse optimizers built on it (``csrc/cuda/by_address.cu``).

    rows = embedding_lookup_by_address(address, embedding_dim, region)          # address 0 -> zeros
    embedding_update_by_address(address, values, update_type, region)           # 0: add (atomic), else: assign
    lazy_adam(gradient, indices, m, v, var, lr, beta1, beta2, epsilon)           # listed rows only, in place
    sgd(gradient, indices, var, lr, weight_decay=0.0)

``address`` holds byte addresses of fp32 rows, e.g. what ``HKVTable.find_pointers`` returns; ``region`` is the tensor (or
``(first_byte, end_byte)`` pair) those rows live in: every address is checked against it before it is dereferenced, a
stray one is skipped and reported through the status word.  Reference ops: ``EmbeddingLookupByAddress``,
``EmbeddingUpdateByAddress``, ``LazyAdam``, ``Sgd`` (``cust_op/framework/tf_plugin/src``) and the by-address optimizers of
``training/tf_rec_v1/python/optimizers``.
"""
from __future__ import annotations

import ctypes
from typing import Tuple, Union

import numpy as np
import torch

from . import _lib

Region = Union[torch.Tensor, Tuple[int, int]]


def _region(region: Region) -> Tuple[int, int]:
    if isinstance(region, torch.Tensor):
        lo = region.data_ptr()
        return lo, lo + region.numel() * region.element_size()
    lo, hi = int(region[0]), int(region[1])
    if hi <= lo:
        raise ValueError("empty address region")
    return lo, hi


def _host_row(addr: int, dim: int) -> np.ndarray:
    return np.ctypeslib.as_array((ctypes.c_float * dim).from_address(addr))


def embedding_lookup_by_address(address: torch.Tensor, embedding_dim: int, region: Region) -> torch.Tensor:
    lo, hi = _region(region)
    a = address.contiguous().long()
    n = a.numel()
    if not a.is_cuda:
        out = torch.zeros(n, embedding_dim)
        for i, p in enumerate(a.tolist()):
            if p == 0:
                continue
            if not (lo <= p and p + 4 * embedding_dim <= hi and p % 4 == 0):
                raise IndexError("address %#x outside the region" % p)
            out[i] = torch.from_numpy(_host_row(p, embedding_dim).copy())
        return out
    out = torch.empty(n, embedding_dim, dtype=torch.float32, device=a.device)
    rc = _lib.lib().rb_rows_gather_by_address(a.data_ptr(), n, embedding_dim, out.data_ptr(), lo, hi, _lib.num_sms(a.device),
                                              _lib.status_tensor(a.device).data_ptr(), _lib.stream_ptr(a.device))
    _lib.check(rc, "rb_rows_gather_by_address")
    return out


def embedding_update_by_address(address: torch.Tensor, embedding: torch.Tensor, update_type: int, region: Region) -> None:
    lo, hi = _region(region)
    a = address.contiguous().long()
    vals = embedding.float().contiguous()
    n, D = vals.shape
    assert a.numel() == n
    if not a.is_cuda:
        for i, p in enumerate(a.tolist()):
            if p == 0:
                continue
            if not (lo <= p and p + 4 * D <= hi and p % 4 == 0):
                raise IndexError("address %#x outside the region" % p)
            row = _host_row(p, D)
            if update_type == 0:
                row += vals[i].numpy()
            else:
                row[:] = vals[i].numpy()
        return
    rc = _lib.lib().rb_rows_update_by_address(a.data_ptr(), n, D, vals.data_ptr(), int(update_type), lo, hi, _lib.num_sms(a.device),
                                              _lib.status_tensor(a.device).data_ptr(), _lib.stream_ptr(a.device))
    _lib.check(rc, "rb_rows_update_by_address")


def _dedup(indices: torch.Tensor, gradient: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sum the gradients of repeated indices (the moment updates below want every row once)."""
    u, inv = torch.unique(indices, return_inverse=True)
    if u.numel() == indices.numel():
        return indices, gradient
    g = torch.zeros(u.numel(), gradient.shape[1], dtype=gradient.dtype, device=gradient.device).index_add_(0, inv, gradient)
    return u, g


def sgd(gradient: torch.Tensor, indices: torch.Tensor, var: torch.Tensor, lr: float, weight_decay: float = 0.0) -> torch.Tensor:
    """``var[indices] -= lr * (gradient + weight_decay * var[indices])`` in place (repeated indices accumulate)."""
    idx, g = indices.long().contiguous(), gradient.float().contiguous()
    if weight_decay != 0.0:
        idx, g = _dedup(idx, g)
    assert var.dtype == torch.float32 and var.dim() == 2 and var.is_contiguous() and g.shape[1] == var.shape[1]
    if not var.is_cuda:
        upd = g + weight_decay * var[idx] if weight_decay != 0.0 else g
        var.index_add_(0, idx, upd, alpha=-float(lr))
        return var
    rc = _lib.lib().rb_rows_sgd(var.data_ptr(), var.shape[0], var.shape[1], idx.data_ptr(), g.data_ptr(), idx.numel(), float(lr),
                                float(weight_decay), _lib.num_sms(var.device), _lib.status_tensor(var.device).data_ptr(),
                                _lib.stream_ptr(var.device))
    _lib.check(rc, "rb_rows_sgd")
    return var


def lazy_adam(gradient: torch.Tensor, indices: torch.Tensor, m: torch.Tensor, v: torch.Tensor, var: torch.Tensor, lr: float,
              beta1: float = 0.9, beta2: float = 0.999, epsilon: float = 1e-8):
    """Adam on the listed rows only (moments of untouched rows do not decay); ``lr`` is the step's effective rate (bias
    correction folded in by the caller, as the reference optimizer does).  In place; returns ``(m, v, var)``."""
    idx, g = _dedup(indices.long().contiguous(), gradient.float().contiguous())
    for t in (m, v, var):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.shape == var.shape
    if not var.is_cuda:
        mr = beta1 * m[idx] + (1 - beta1) * g
        vr = beta2 * v[idx] + (1 - beta2) * g * g
        m[idx], v[idx] = mr, vr
        var[idx] = var[idx] - lr * mr / (vr.sqrt() + epsilon)
        return m, v, var
    rc = _lib.lib().rb_rows_lazy_adam(var.data_ptr(), m.data_ptr(), v.data_ptr(), var.shape[0], var.shape[1], idx.data_ptr(),
                                      g.data_ptr(), idx.numel(), float(lr), float(beta1), float(beta2), float(epsilon),
                                      _lib.num_sms(var.device), _lib.status_tensor(var.device).data_ptr(), _lib.stream_ptr(var.device))
    _lib.check(rc, "rb_rows_lazy_adam")
    return m, v, var

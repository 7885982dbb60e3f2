"""Stand-alone forms of the reference's three in-kernel collectives, for code that called them directly.

The reference ships them as operators of its TensorFlow plug-in (``cust_op/framework/tf_plugin/src/lccl.cpp:20-85``; kernels
``ascendc_op/ai_core_op/lccl/v220/op_kernel/{all2all,all2all_uss,gather_all}.h``):

* ``lccl_all_to_all(send_data, send_count_matrix, ...)``: rows grouped by destination rank travel to their destinations;
  ``send_count_matrix[s][d]`` is the number of rows rank ``s`` sends to rank ``d`` (every rank holds the whole matrix, so
  no size exchange precedes the data).
* ``lccl_all_uss(..., restore)``: the same exchange followed by an unsorted segment sum of the received rows,
  ``out[restore[i]] += recv[i]`` - the exchange of embedding gradients with the sum over duplicate ids.
* ``lccl_gather_all(emb_table, lookup, ...)``: ``emb_table[lookup]`` followed by the exchange - lookup plus distribution
  of the rows.

Inside the sharded collections of this package these operations do not exist as separate steps: the push exchange
(``parallel/push_exchange.py``) looks rows up on their owner and stores them straight into the requester's memory, and
sums pushed gradient rows per distinct row before the optimizer, over NVLink peer memory.  The functions here keep the
reference's argument lists (``shape_vec`` and ``peer_mem`` are accepted and may be ``None``: the output size follows
from the count matrix and there is no caller-managed buffer) and run on any ``torch.distributed`` backend, which is what
host-side and CPU code needs.  ``LCCL_DETERMINISTIC=1`` makes the segment sum independent of the arrival order, like the
reference's deterministic kernel (``all_uss_deterministic.h``).
"""
from __future__ import annotations

import os
from typing import Optional, Sequence, Union

import torch

from ..ops import embedding_ops as E

_Matrix = Union[torch.Tensor, Sequence[Sequence[int]]]


def _splits(send_count_matrix: _Matrix, rank: int, rank_size: int):
    m = torch.as_tensor(send_count_matrix, dtype=torch.int64).cpu().reshape(-1)
    if m.numel() != rank_size * rank_size:
        raise ValueError("send_count_matrix must hold rank_size x rank_size = %d counts, got %d" % (rank_size * rank_size, m.numel()))
    if not 0 <= rank < rank_size:
        raise ValueError("rank %d is outside [0, %d)" % (rank, rank_size))
    m = m.view(rank_size, rank_size)
    if bool((m < 0).any()):
        raise ValueError("send_count_matrix holds a negative count")
    return m[rank].tolist(), m[:, rank].tolist()


def _check_rows(t: torch.Tensor, dim: int, what: str) -> torch.Tensor:
    if t.dim() == 1:
        if dim <= 0 or t.numel() % dim:
            raise ValueError("%s: %d elements are not rows of %d" % (what, t.numel(), dim))
        t = t.view(-1, dim)
    if t.dim() != 2 or (dim > 0 and t.shape[1] != dim):
        raise ValueError("%s must be [rows, %d], got %s" % (what, dim, tuple(t.shape)))
    return t.contiguous()


def lccl_all_to_all(send_data: torch.Tensor, send_count_matrix: _Matrix, shape_vec=None, peer_mem=None, *, rank: int,
                    rank_size: int, dim: int, group=None) -> torch.Tensor:
    """-> ``[sum_s send_count_matrix[s][rank], dim]``: the rows every rank addressed to this one, ordered by source."""
    rows = _check_rows(send_data, dim, "send_data")
    in_splits, out_splits = _splits(send_count_matrix, rank, rank_size)
    if rows.shape[0] != sum(in_splits):
        raise ValueError("send_data has %d rows, the count matrix says this rank sends %d" % (rows.shape[0], sum(in_splits)))
    if shape_vec is not None:
        want = int(torch.as_tensor(shape_vec).reshape(-1)[0])
        if want != sum(out_splits):
            raise ValueError("shape_vec says %d received rows, the count matrix says %d" % (want, sum(out_splits)))
    out = rows.new_empty(sum(out_splits), rows.shape[1])
    if rank_size == 1:
        out.copy_(rows)
        return out
    import torch.distributed as dist

    dist.all_to_all_single(out, rows, out_splits, in_splits, group=group)
    return out


def unsorted_segment_sum(rows: torch.Tensor, restore: torch.Tensor, num_segments: int, deterministic: Optional[bool] = None) -> torch.Tensor:
    """``out[restore[i]] += rows[i]``.  The deterministic form sorts by segment (stable) and sums every segment in row
    order, so the result does not depend on how the hardware schedules the additions."""
    if deterministic is None:
        deterministic = os.environ.get("LCCL_DETERMINISTIC", "0") == "1"
    restore = restore.to(device=rows.device, dtype=torch.int64).reshape(-1)
    if restore.numel() != rows.shape[0]:
        raise ValueError("restore has %d entries for %d rows" % (restore.numel(), rows.shape[0]))
    if restore.numel() and (int(restore.min()) < 0 or int(restore.max()) >= num_segments):
        raise ValueError("restore index outside [0, %d)" % num_segments)
    out = rows.new_zeros(num_segments, rows.shape[1])
    if not restore.numel():
        return out
    if not deterministic:
        return out.index_add_(0, restore, rows)
    order = torch.argsort(restore, stable=True)
    lengths = torch.bincount(restore, minlength=num_segments)
    return torch.segment_reduce(rows[order], "sum", lengths=lengths, axis=0, unsafe=True).to(rows.dtype)


def lccl_all_uss(send_data: torch.Tensor, send_count_matrix: _Matrix, shape_vec, peer_mem, restore: torch.Tensor, *, rank: int,
                 rank_size: int, dim: int, group=None) -> torch.Tensor:
    """All-to-all, then the unsorted segment sum of the received rows by ``restore``; ``shape_vec[0]`` is the number of
    segments (rows of the result)."""
    if shape_vec is None:
        raise ValueError("lccl_all_uss needs shape_vec: its first entry is the number of output rows")
    recv = lccl_all_to_all(send_data, send_count_matrix, None, peer_mem, rank=rank, rank_size=rank_size, dim=dim, group=group)
    return unsorted_segment_sum(recv, restore, int(torch.as_tensor(shape_vec).reshape(-1)[0]))


def lccl_gather_all(emb_table: torch.Tensor, lookup: torch.Tensor, send_count_matrix: _Matrix, shape_vec=None, peer_mem=None, *,
                    rank: int, rank_size: int, dim: int, group=None) -> torch.Tensor:
    """``emb_table[lookup]`` (rows in destination order), then the all-to-all."""
    table = _check_rows(emb_table, dim, "emb_table")
    idx = lookup.to(device=table.device, dtype=torch.int64).reshape(-1)
    if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= table.shape[0]):
        raise ValueError("lookup index outside [0, %d)" % table.shape[0])
    rows = E.gather_rows(table, idx)
    return lccl_all_to_all(rows, send_count_matrix, shape_vec, peer_mem, rank=rank, rank_size=rank_size, dim=dim, group=group)

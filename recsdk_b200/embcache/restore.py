"""``restore`` / ``restore_async``: rebuild the per-id cache offsets from the planner's per-unique-key offsets.

After the swap planner has given every unique key of a batch its device-cache offset, the lookup needs one offset per id:
``hash_indices[r] = unique_indices[unique_inverse[r] + unique_offset[t]]`` for the ids ``r`` of table ``t``.  The native
implementation walks the tables in parallel and writes into the caller's tensor (``torchrec_embcache`` of the reference:
``csrc/ops/restore.cpp:17-70``, asynchronous form ``:72-80``).
"""
from __future__ import annotations

from typing import Sequence

import torch
from torch.autograd.profiler import record_function

from ..host import host


def _np(t: torch.Tensor, name: str):
    if t.device.type != "cpu" or t.dtype != torch.int64 or t.dim() != 1 or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous 1-D int64 CPU tensor")
    return t.numpy()


def restore(unique_indices: torch.Tensor, unique_inverse: torch.Tensor, unique_offset: torch.Tensor,
            offsets_per_table: Sequence[int], hash_indices: torch.Tensor) -> torch.Tensor:
    """Fills ``hash_indices`` in place and returns it."""
    with record_function("## restore ##"):
        host().restore(_np(unique_indices, "unique_indices"), _np(unique_inverse, "unique_inverse"), _np(unique_offset, "unique_offset"),
                       [int(x) for x in offsets_per_table], _np(hash_indices, "hash_indices"))
    return hash_indices


class RestoreTask:
    """Handle of a restore running on the host helper pool; ``get()`` waits and re-raises a range error."""

    def __init__(self, fut, out: torch.Tensor) -> None:
        self._fut, self._out = fut, out

    def ready(self) -> bool:
        return self._fut.ready()

    def get(self) -> torch.Tensor:
        self._fut.get()
        return self._out


def restore_async(unique_indices: torch.Tensor, unique_inverse: torch.Tensor, unique_offset: torch.Tensor,
                  offsets_per_table: Sequence[int], hash_indices: torch.Tensor) -> RestoreTask:
    fut = host().restore_async(_np(unique_indices, "unique_indices"), _np(unique_inverse, "unique_inverse"),
                               _np(unique_offset, "unique_offset"), [int(x) for x in offsets_per_table],
                               _np(hash_indices, "hash_indices"))
    return RestoreTask(fut, hash_indices)

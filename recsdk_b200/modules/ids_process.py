"""Host-side id processing under the reference's Python names (``hybrid_torchrec/modules/ids_process.py:21-111``):
``IdsMapper`` (raw id -> row slot, with fused unique) as an ``nn.Module`` over the native mapper, ``BucketParams`` and
``block_bucketize_sparse_features_cpu`` (row-wise bucketisation by ``id % bucket_size`` with optional de-duplication per
(bucket, feature) and occurrence / click counts; native kernel: ``csrc/host/ids_process.h``).
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Tuple

import numpy as np
import torch
from torch.autograd.profiler import record_function

from ..host import host


@dataclasses.dataclass
class BucketParams:
    lengths: torch.Tensor
    indices: torch.Tensor
    bucketize_pos: bool
    sequence: bool
    block_sizes: torch.Tensor
    bucket_size: int
    total_num_blocks: Optional[torch.Tensor] = None
    weights: Optional[torch.Tensor] = None
    batch_size_per_feature: Optional[torch.Tensor] = None
    max_b: int = 0
    block_bucketize_pos: Optional[torch.Tensor] = None
    return_bucket_mapping: bool = False
    keep_orig_idx: bool = False
    do_unique: bool = False
    return_count: bool = False
    labels: Optional[torch.Tensor] = None


class HashMapBase(torch.nn.Module):
    def forward(self, ids: torch.Tensor):
        raise NotImplementedError


class IdsMapper(HashMapBase):
    """Global ids -> row indices of a table that lives on the device (slots are handed out in order of first sight);
    ``forward`` also returns the distinct slots and the inverse map, so a lookup can gather every row once."""

    def __init__(self, embedding_num: int, only_device_memory: bool = True) -> None:
        super().__init__()
        self.ids_mapper = host().IdsMapper(int(embedding_num))
        self.embedding_num = int(embedding_num)
        self.only_device_memory = bool(only_device_memory)
        self._cache_mgr = None

    def set_cache_mgr(self, cache_mgr) -> None:
        self._cache_mgr = cache_mgr

    def statistic_key_count(self, ids: torch.Tensor, offset: Optional[torch.Tensor], counts: torch.Tensor, table_i: int) -> None:
        """Hand the occurrence counts of ``ids`` to the cache manager (which keeps them only for tables with admission on)."""
        if self._cache_mgr is None:
            raise RuntimeError("no cache manager set: call set_cache_mgr first")
        self._cache_mgr.statistics_key_count(int(table_i), np.ascontiguousarray(ids.cpu().numpy().astype(np.int64)),
                                             np.ascontiguousarray(counts.cpu().numpy().astype(np.int64)), None)

    def forward(self, ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        with record_function("## ids2indices ##"):
            hi, uniq, _uids, inv = self.ids_mapper.ids2indices_unique_out(np.ascontiguousarray(ids.cpu().numpy().astype(np.int64)))
            dev = ids.device
            return torch.from_numpy(hi).to(dev), torch.from_numpy(uniq).to(dev), torch.from_numpy(inv).to(dev)

    def ids2indices_unique_out(self, ids: torch.Tensor, hash_indices: torch.Tensor, offset: torch.Tensor, unique: torch.Tensor,
                               unique_ids: torch.Tensor, unique_inverse: torch.Tensor, unique_offset: List[int], table_id: int) -> None:
        """Out-variant for one table of a batch: ``ids`` is the whole value list, ``offset[table_id] .. offset[table_id + 1]``
        this table's part; slots go to the same range of ``hash_indices``, the distinct slots / ids are appended at
        ``unique_offset[table_id]`` of ``unique`` / ``unique_ids``, ``unique_inverse`` gets positions in that unique list, and
        ``unique_offset[table_id + 1]`` is set to the end of this table's distinct entries."""
        lo, hi_ = int(offset[table_id]), int(offset[table_id + 1])
        hi, uniq, uids, inv = self.ids_mapper.ids2indices_unique_out(np.ascontiguousarray(ids[lo:hi_].cpu().numpy().astype(np.int64)))
        u0 = int(unique_offset[table_id])
        hash_indices[lo:hi_] = torch.from_numpy(hi).to(hash_indices.dtype)
        unique[u0:u0 + len(uniq)] = torch.from_numpy(uniq).to(unique.dtype)
        unique_ids[u0:u0 + len(uids)] = torch.from_numpy(uids).to(unique_ids.dtype)
        unique_inverse[lo:hi_] = torch.from_numpy(inv).to(unique_inverse.dtype) + u0
        unique_offset[table_id + 1] = u0 + len(uniq)

    def size(self) -> int:
        return int(self.ids_mapper.size())


def block_bucketize_sparse_features_cpu(bucket_params: BucketParams):
    """-> ``(new_lengths, new_indices, new_weights | None, new_pos | None, unbucketize_permute | None[, counts])``.

    Bucket-major output (``new_lengths[(bucket * F + f) * B + b]``), bucket of an id = ``id % bucket_size``.
    ``do_unique``: inside every (bucket, feature) group an id is kept once, in the bag where it first appears; later
    occurrences shorten their bags; ``unbucketize_permute[i]`` is then the position of the kept copy of element ``i``.
    ``return_count``: occurrences of every kept id (``[n, 1]``; with ``labels`` ``[n, 2]``: occurrences and the sum of the
    per-sample labels, the "click" count)."""
    p = bucket_params
    lengths = np.ascontiguousarray(p.lengths.cpu().numpy().astype(np.int64))
    indices = np.ascontiguousarray(p.indices.cpu().numpy().astype(np.int64))
    W = int(p.bucket_size)
    if p.batch_size_per_feature is not None:
        raise NotImplementedError("variable batch sizes per feature are not supported")
    B = int(p.max_b) if p.max_b else 0
    if B <= 0:
        nblocks = int(p.block_sizes.numel()) if p.block_sizes is not None else 1
        B = lengths.size // max(nblocks, 1)
    F = lengths.size // max(B, 1)
    w = None if p.weights is None else np.ascontiguousarray(p.weights.cpu().numpy().astype(np.float32))
    # ids keep their value (they are raw keys that the owner's mapper translates), whatever ``keep_orig_idx`` says
    nl, ni, nw, perm = host().block_bucketize_sparse_features(lengths, indices, w, F, B, W, None, False)
    counts = None
    if p.do_unique:
        n = ni.size
        group = np.repeat(np.arange(nl.size) // B, nl)               # (bucket * F + f) of every bucketized element
        pairs = np.stack([group, ni], axis=1)
        _u, first, inv, cnt = np.unique(pairs, axis=0, return_index=True, return_inverse=True, return_counts=True)
        inv = inv.reshape(-1)
        rank = np.empty(first.size, dtype=np.int64)
        rank[np.argsort(first, kind="stable")] = np.arange(first.size)          # kept ids in order of first appearance
        keep = np.zeros(n, dtype=bool)
        keep[first] = True
        bag = np.repeat(np.arange(nl.size), nl)
        nl = nl - np.bincount(bag[~keep], minlength=nl.size)
        kept_idx = np.empty(first.size, dtype=np.int64)
        kept_idx[rank] = ni[first]
        if p.return_count:
            counts = np.zeros((first.size, 2 if p.labels is not None else 1), dtype=np.int64)
            counts[rank, 0] = cnt
            if p.labels is not None:
                lab = p.labels.cpu().numpy().astype(np.int64)
                np.add.at(counts[:, 1], rank[inv], lab[bag % B])
        if nw is not None and w is not None:
            kw = np.empty(first.size, dtype=np.float32)
            kw[rank] = nw[first]
            nw = kw
        perm = rank[inv][perm]
        ni = kept_idx
    out = (torch.from_numpy(nl), torch.from_numpy(ni), None if w is None else torch.from_numpy(nw), None,
           torch.from_numpy(perm) if (p.sequence or p.do_unique) else None)
    return out + ((torch.from_numpy(counts),) if counts is not None else ())


# ----------------------------------------------------------------------------------------------------------------------
# ``torch.ops.hybrid.block_bucketize_sparse_features_cpu``: the operator form, with the reference's argument list
# (``hybrid_torchrec/src/bind_torch_lib.cpp:11-19``, ``src/ids_process/bucketize.h:14-27``)
# ----------------------------------------------------------------------------------------------------------------------
_HYBRID_LIB = torch.library.Library("hybrid", "DEF")
_HYBRID_LIB.define(
    "block_bucketize_sparse_features_cpu(Tensor lengths, Tensor indices, bool bucketize_pos, bool sequence, Tensor block_sizes, "
    "int bucket_size, Tensor? total_num_blocks=None, Tensor? weights=None, Tensor? batch_size_per_feature=None, int max_B=-1, "
    "Tensor[]? block_bucketize_pos=None, bool return_bucket_mapping=False, bool keep_orig_idx=False, bool do_unique=False, "
    "bool return_count=False, Tensor? labels=None) -> (Tensor, Tensor, Tensor?, Tensor?, Tensor?, Tensor?, Tensor)")


def _block_bucketize_op(lengths, indices, bucketize_pos, sequence, block_sizes, bucket_size, total_num_blocks=None, weights=None,
                        batch_size_per_feature=None, max_B=-1, block_bucketize_pos=None, return_bucket_mapping=False,
                        keep_orig_idx=False, do_unique=False, return_count=False, labels=None):
    """-> (new_lengths, new_indices, new_weights?, new_pos?, unbucketize_permute?, bucket_mapping?, counts); ``counts`` is
    empty unless ``do_unique`` and ``return_count`` are set; ``bucket_mapping[i]`` is the bucket of input element ``i``."""
    if block_bucketize_pos is not None:
        raise NotImplementedError("explicit bucket boundaries are not supported: buckets are id % bucket_size")
    out = block_bucketize_sparse_features_cpu(BucketParams(
        lengths, indices, bool(bucketize_pos), bool(sequence), block_sizes, int(bucket_size), total_num_blocks, weights,
        batch_size_per_feature, max(int(max_B), 0), None, bool(return_bucket_mapping), bool(keep_orig_idx), bool(do_unique),
        bool(return_count), labels))
    counts = out[5] if len(out) > 5 else torch.empty(0, dtype=torch.int64)
    mapping = (indices.to(torch.int64) % int(bucket_size)) if return_bucket_mapping else None
    return out[0], out[1], out[2], out[3], out[4], mapping, counts


_HYBRID_LIB.impl("block_bucketize_sparse_features_cpu", _block_bucketize_op, "CPU")

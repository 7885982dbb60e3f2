"""Device-side id preprocessing: segmented unique, row-wise bucketisation, compaction, table ranges.

CUDA tensors run the kernels of ``csrc/cuda/sparse_ops.cu``; CPU tensors take an equivalent PyTorch path (the
oracle of the GPU tests).  Semantics follow the reference's dynamic_emb extension ops
(``csrc/dynamic_emb_op.cpp:748-830`` unique, ``:1001-1124`` segmented unique / dedup,
``csrc/ops/block_bucketsize_sparse_features``, ``csrc/ops/maskselect_op``, ``csrc/ops/get_table_range_op``,
``csrc/ops/get_new_length_and_offsets_op``).  The order of the unique keys inside a table is unspecified on the
GPU (hash order), as in the reference; ``inverse`` is consistent with it.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from . import _lib

_WS = {}      # scratch buffers per (device, purpose): reused by consecutive calls on ONE stream; callers that run these
              # ops on several streams of a device at once must serialise them


def _ws(device, name: str, n: int, dtype) -> torch.Tensor:
    key = (device, name, dtype)
    t = _WS.get(key)
    if t is None or t.numel() < n:
        t = torch.empty(max(n, 1024), dtype=dtype, device=device)
        _WS[key] = t
    return t


def segmented_unique(keys: torch.Tensor, table_offsets: torch.Tensor, with_counts: bool = False
                     ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Per-table unique of ``keys`` (int64 [n]); table t owns ``keys[table_offsets[t]:table_offsets[t+1]]``.

    Returns ``(unique_buf, inverse, unique_offsets, counts)``: ``unique_buf[unique_offsets[t]:unique_offsets[t+1]]``
    are table t's distinct keys (the buffer has n entries; only the first ``unique_offsets[-1]`` are defined),
    ``unique_buf[inverse[i]] == keys[i]``, ``counts[j]`` the multiplicity of ``unique_buf[j]``.  No host sync."""
    n, T = keys.numel(), table_offsets.numel() - 1
    dev = keys.device
    if not keys.is_cuda:
        uo = [0]
        us, inv, cs = [], torch.empty(n, dtype=torch.int64), []
        offs = table_offsets.tolist()
        for t in range(T):
            u, i, c = torch.unique(keys[offs[t]:offs[t + 1]], return_inverse=True, return_counts=True)
            inv[offs[t]:offs[t + 1]] = i + uo[-1]
            us.append(u)
            cs.append(c)
            uo.append(uo[-1] + u.numel())
        ub = torch.zeros(n, dtype=torch.int64)
        ub[: uo[-1]] = torch.cat(us) if us else ub[:0]
        cb = torch.zeros(n, dtype=torch.int32)
        cb[: uo[-1]] = torch.cat(cs).int() if cs else cb[:0]
        return ub, inv, torch.tensor(uo, dtype=torch.int64), cb if with_counts else None
    keys = keys.contiguous()
    offs = table_offsets.to(device=dev, dtype=torch.int64).contiguous()
    table = _ws(dev, "uniq_table", 2 * n + T, torch.int64)
    slots = _ws(dev, "uniq_slots", 2 * n + T, torch.int32)
    small = _ws(dev, "uniq_small", 2 * T, torch.int32)
    pos = _ws(dev, "uniq_pos", n, torch.int32)
    unique = torch.empty(n, dtype=torch.int64, device=dev)
    inverse = torch.empty(n, dtype=torch.int64, device=dev)
    counts = torch.empty(n, dtype=torch.int32, device=dev) if with_counts else None
    uoffs = torch.empty(T + 1, dtype=torch.int64, device=dev)
    rc = _lib.lib().rb_segmented_unique(keys.data_ptr(), n, offs.data_ptr(), T, table.data_ptr(), slots.data_ptr(),
                                        small.data_ptr(), small[T:].data_ptr(), pos.data_ptr(), unique.data_ptr(),
                                        inverse.data_ptr(), _lib.ptr(counts), uoffs.data_ptr(),
                                        _lib.status_tensor(dev).data_ptr(), _lib.num_sms(dev), _lib.stream_ptr(dev))
    _lib.check(rc, "rb_segmented_unique")
    return unique, inverse, uoffs, counts


def unique(keys: torch.Tensor, with_counts: bool = False):
    """``(unique keys, inverse[, counts])``; trims the buffer, which costs one host sync on CUDA."""
    offs = torch.tensor([0, keys.numel()], dtype=torch.int64)
    ub, inv, uo, c = segmented_unique(keys, offs, with_counts)
    k = int(uo[-1].item())
    return (ub[:k], inv, c[:k]) if with_counts else (ub[:k], inv)


def block_bucketize_sparse_features(lengths: torch.Tensor, indices: torch.Tensor, world: int, F: int, B: int,
                                    block_sizes: Optional[torch.Tensor] = None, weights: Optional[torch.Tensor] = None,
                                    local_rows: bool = False, want_permute: bool = True):
    """Row-wise bucketisation (bucket-major output, like FBGEMM's op of the same name).  Round robin ``id % world``
    when ``block_sizes`` is None, else contiguous blocks ``min(id // block_sizes[f], world - 1)``.
    Returns ``(new_lengths [world*F*B], new_indices, new_weights | None, unbucketize_permute | None)``."""
    dev = indices.device
    if not indices.is_cuda:
        from ..host import host
        import numpy as np

        bs = None if block_sizes is None else block_sizes.numpy().astype(np.int64)
        w = None if weights is None else weights.numpy().astype(np.float32)
        nl, ni, nw, perm = host().block_bucketize_sparse_features(lengths.numpy().astype(np.int64), indices.numpy().astype(np.int64),
                                                                  w, F, B, world, bs, local_rows)
        return (torch.from_numpy(nl), torch.from_numpy(ni), None if weights is None else torch.from_numpy(nw),
                torch.from_numpy(perm) if want_permute else None)
    FB = F * B
    offsets = torch.zeros(FB + 1, dtype=torch.int64, device=dev)
    torch.cumsum(lengths.to(torch.int64), 0, out=offsets[1:])
    indices = indices.contiguous()
    bs = None if block_sizes is None else block_sizes.to(device=dev, dtype=torch.int64).contiguous()
    new_lengths = torch.empty(world * FB, dtype=torch.int64, device=dev)
    st = _lib.stream_ptr(dev)
    rc = _lib.lib().rb_block_bucketize_count(offsets.data_ptr(), indices.data_ptr(), F, B, world, _lib.ptr(bs),
                                             new_lengths.data_ptr(), st)
    _lib.check(rc, "rb_block_bucketize_count")
    new_offsets = torch.zeros(world * FB + 1, dtype=torch.int64, device=dev)
    torch.cumsum(new_lengths, 0, out=new_offsets[1:])
    new_indices = torch.empty_like(indices)
    new_weights = None if weights is None else torch.empty_like(weights, dtype=torch.float32)
    w32 = None if weights is None else weights.float().contiguous()
    perm = torch.empty_like(indices) if want_permute else None
    rc = _lib.lib().rb_block_bucketize_fill(offsets.data_ptr(), indices.data_ptr(), _lib.ptr(w32), F, B, world, _lib.ptr(bs),
                                            int(local_rows), new_offsets.data_ptr(), new_indices.data_ptr(),
                                            _lib.ptr(new_weights), _lib.ptr(perm), st)
    _lib.check(rc, "rb_block_bucketize_fill")
    return new_lengths, new_indices, new_weights, perm


def select(values: Optional[torch.Tensor], flags: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Order-preserving compaction ``values[flags]`` (``values`` None: the selected positions).  Returns a buffer
    of ``flags.numel()`` entries and the device count; no host sync."""
    n = flags.numel()
    dev = flags.device
    if not flags.is_cuda:
        src = torch.arange(n, dtype=torch.int64) if values is None else values
        sel = src[flags.bool()]
        out = torch.zeros(n, dtype=torch.int64)
        out[: sel.numel()] = sel
        return out, torch.tensor([sel.numel()], dtype=torch.int64)
    f8 = flags.to(torch.uint8).contiguous()
    out = torch.empty(n, dtype=torch.int64, device=dev)
    cnt = torch.zeros(1, dtype=torch.int64, device=dev)
    if n == 0:
        return out, cnt
    nbytes = int(_lib.lib().rb_compact_select_temp_bytes(n))
    temp = _ws(dev, "select_temp", nbytes, torch.uint8)
    v = None if values is None else values.to(torch.int64).contiguous()
    rc = _lib.lib().rb_compact_select(_lib.ptr(v), f8.data_ptr(), n, out.data_ptr(), cnt.data_ptr(), temp.data_ptr(), nbytes,
                                      _lib.stream_ptr(dev))
    _lib.check(rc, "rb_compact_select")
    return out, cnt


def select_index(flags: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return select(None, flags)


def get_table_range(offsets: torch.Tensor, feature_offsets: Sequence[int], B: int) -> torch.Tensor:
    """``out[t] = offsets[feature_offsets[t] * B]``: table t's range of ids in the KJT values
    (``feature_offsets`` [T+1]: first feature of every table)."""
    fo = torch.as_tensor(feature_offsets, dtype=torch.int32)
    if not offsets.is_cuda:
        return offsets.to(torch.int64)[fo.long() * B]
    T = fo.numel() - 1
    fo = fo.to(offsets.device)
    out = torch.empty(T + 1, dtype=torch.int64, device=offsets.device)
    offsets = offsets.to(torch.int64).contiguous()
    rc = _lib.lib().rb_table_range(offsets.data_ptr(), fo.data_ptr(), T, B, out.data_ptr(), _lib.stream_ptr(offsets.device))
    _lib.check(rc, "rb_table_range")
    return out


def get_new_length_and_offsets(unique_offsets: torch.Tensor, feature_offsets: Sequence[int], B: int
                               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Lengths / offsets of the deduplicated KJT: table t's ``u_t`` distinct keys are spread evenly over its
    ``(features of t) * B`` bags, the first ``u_t mod bags`` bags holding one more."""
    fo = torch.as_tensor(feature_offsets, dtype=torch.int32)
    T = fo.numel() - 1
    FB = int(fo[-1]) * B
    if not unique_offsets.is_cuda:
        nl = torch.zeros(FB, dtype=torch.int64)
        uo = unique_offsets.tolist()
        for t in range(T):
            first, last = int(fo[t]) * B, int(fo[t + 1]) * B
            bags, u = last - first, uo[t + 1] - uo[t]
            if bags:
                nl[first:last] = u // bags
                nl[first:first + u % bags] += 1
        no = torch.zeros(FB + 1, dtype=torch.int64)
        torch.cumsum(nl, 0, out=no[1:])
        return nl, no
    dev = unique_offsets.device
    nl = torch.empty(FB, dtype=torch.int64, device=dev)
    no = torch.empty(FB + 1, dtype=torch.int64, device=dev)
    fo = fo.to(dev)
    rc = _lib.lib().rb_new_lengths_offsets(unique_offsets.contiguous().data_ptr(), fo.data_ptr(), T, B, FB, nl.data_ptr(),
                                           no.data_ptr(), _lib.num_sms(dev), _lib.stream_ptr(dev))
    _lib.check(rc, "rb_new_lengths_offsets")
    return nl, no


def dedup_input_indices(values: torch.Tensor, offsets: torch.Tensor, feature_offsets: Sequence[int], B: int):
    """Per-table dedup of a KJT's ids before the id exchange (reference ``dedup_input_indices_op``):
    returns ``(unique_buf, inverse, new_lengths, new_offsets, unique_offsets)``; after the lookup of the unique
    ids, ``rows[inverse]`` restores the per-id rows."""
    trange = get_table_range(offsets, feature_offsets, B)
    ub, inv, uo, _ = segmented_unique(values, trange)
    nl, no = get_new_length_and_offsets(uo, feature_offsets, B)
    return ub, inv, nl, no, uo

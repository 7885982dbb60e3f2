"""KeyedJaggedTensor variants that carry side tensors through the input pipeline (pinning, device copies, stream
recording, key splits and permutations):

* ``KeyedJaggedTensorWithLookHelper`` - the id-mapping results of the host stage: ``hash_indices`` (slot per id),
  ``unique_indices`` / ``unique_offset`` / ``unique_inverse`` (per-table de-duplication) so the lookup can gather
  unique rows once (``hybrid_torchrec/sparse/jagged_tensor_with_looup_helper.py:20-462`` of the reference);
* ``KeyedJaggedTensorWithCount`` - per-id occurrence counts for admission statistics
  (``sparse/jagged_tensor_with_count.py:24-387``);
* ``KeyedJaggedTensorWithTimestamp`` - per-id timestamps for time-based eviction
  (``torchrec_embcache/sparse/jagged_tensor_with_timestamp.py:31-157``);
* ``ExtendedJaggedTensor`` - a JaggedTensor with named extra per-value tensors
  (``sparse/extended_jagged_tensor.py:37-633``).

Per-value side tensors are sliced together with the values; whole-batch side tensors travel unchanged.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .jagged_tensor import JaggedTensor, KeyedJaggedTensor


class _SideTensorKJT(KeyedJaggedTensor):
    PER_VALUE: tuple = ()        # names of side tensors aligned with values()
    WHOLE: tuple = ()            # names of side tensors that describe the whole batch

    def _init_side(self, **side: Optional[torch.Tensor]) -> None:
        for n in self.PER_VALUE + self.WHOLE:
            t = side.get(n)
            if t is not None and n in self.PER_VALUE and t.shape[0] != self._values.shape[0]:
                raise ValueError("%s must have one entry per id (%d), got %d" % (n, self._values.shape[0], t.shape[0]))
            setattr(self, "_" + n, t)

    def _side(self) -> Dict[str, Optional[torch.Tensor]]:
        return {n: getattr(self, "_" + n) for n in self.PER_VALUE + self.WHOLE}

    def _wrap(self, base: KeyedJaggedTensor, side: Dict[str, Optional[torch.Tensor]]) -> "_SideTensorKJT":
        out = self.__class__.__new__(self.__class__)
        out.__dict__.update(base.__dict__)
        out._init_side(**side)
        return out

    def to(self, device: torch.device, non_blocking: bool = False):
        side = {n: None if t is None else t.to(device, non_blocking=non_blocking) for n, t in self._side().items()}
        return self._wrap(KeyedJaggedTensor.to(self, device, non_blocking), side)

    def pin_memory(self):
        side = {n: None if t is None else (t if t.is_pinned() else t.pin_memory()) for n, t in self._side().items()}
        return self._wrap(KeyedJaggedTensor.pin_memory(self), side)

    def record_stream(self, stream) -> None:
        KeyedJaggedTensor.record_stream(self, stream)
        for t in self._side().values():
            if t is not None and t.is_cuda:
                t.record_stream(stream)

    def split(self, segments: List[int]):
        parts = KeyedJaggedTensor.split(self, segments)
        opk, start, out = self.offset_per_key(), 0, []
        for seg, p in zip(segments, parts):
            v0, v1 = opk[start], opk[start + seg]
            side = {n: (None if t is None else (t[v0:v1] if n in self.PER_VALUE else t)) for n, t in self._side().items()}
            out.append(self._wrap(p, side))
            start += seg
        return out

    def permute(self, indices: List[int], indices_tensor: Optional[torch.Tensor] = None):
        base = KeyedJaggedTensor.permute(self, indices, indices_tensor)
        opk = self.offset_per_key()
        side = {}
        for n, t in self._side().items():
            if t is None or n in self.WHOLE:
                side[n] = t
            else:
                side[n] = torch.cat([t[opk[i]:opk[i + 1]] for i in indices]) if indices else t[:0]
        return self._wrap(base, side)


class KeyedJaggedTensorWithLookHelper(_SideTensorKJT):
    PER_VALUE = ("hash_indices", "unique_inverse")
    WHOLE = ("unique_indices", "unique_offset")

    def __init__(self, keys, values, weights=None, lengths=None, offsets=None, stride=None, length_per_key=None, offset_per_key=None,
                 hash_indices=None, unique_indices=None, unique_offset=None, unique_inverse=None) -> None:
        super().__init__(keys, values, weights, lengths, offsets, stride, length_per_key, offset_per_key)
        self._init_side(hash_indices=hash_indices, unique_indices=unique_indices, unique_offset=unique_offset, unique_inverse=unique_inverse)

    @staticmethod
    def from_kjt(kjt: KeyedJaggedTensor, hash_indices=None, unique_indices=None, unique_offset=None, unique_inverse=None):
        return KeyedJaggedTensorWithLookHelper(kjt.keys(), kjt.values(), kjt.weights_or_none(), kjt.lengths_or_none(), kjt.offsets_or_none(),
                                               kjt.stride(), hash_indices=hash_indices, unique_indices=unique_indices,
                                               unique_offset=unique_offset, unique_inverse=unique_inverse)

    hash_indices = property(lambda self: self._hash_indices)
    unique_indices = property(lambda self: self._unique_indices)
    unique_offset = property(lambda self: self._unique_offset)
    unique_inverse = property(lambda self: self._unique_inverse)


class KeyedJaggedTensorWithCount(_SideTensorKJT):
    PER_VALUE = ("counts",)

    def __init__(self, keys, values, weights=None, lengths=None, offsets=None, stride=None, length_per_key=None, offset_per_key=None,
                 counts=None) -> None:
        super().__init__(keys, values, weights, lengths, offsets, stride, length_per_key, offset_per_key)
        self._init_side(counts=counts)

    counts = property(lambda self: self._counts)

    @staticmethod
    def dedup(kjt: KeyedJaggedTensor) -> "KeyedJaggedTensorWithCount":
        """Per (feature, sample) bag: distinct ids with their multiplicities (bags keep their order)."""
        lens, vals, B = kjt.lengths().tolist(), kjt.values(), kjt.stride()
        new_vals, new_cnt, new_len, pos = [], [], [], 0
        for n in lens:
            u, c = torch.unique(vals[pos:pos + n], return_counts=True)
            new_vals.append(u)
            new_cnt.append(c)
            new_len.append(u.numel())
            pos += n
        cat = lambda xs, like: torch.cat(xs) if xs else like[:0]  # noqa: E731
        return KeyedJaggedTensorWithCount(kjt.keys(), cat(new_vals, vals), None, torch.tensor(new_len, dtype=torch.int64), None, B,
                                          counts=cat(new_cnt, vals))


class KeyedJaggedTensorWithTimestamp(_SideTensorKJT):
    PER_VALUE = ("timestamps",)

    def __init__(self, keys, values, weights=None, lengths=None, offsets=None, stride=None, length_per_key=None, offset_per_key=None,
                 timestamps=None) -> None:
        super().__init__(keys, values, weights, lengths, offsets, stride, length_per_key, offset_per_key)
        self._init_side(timestamps=timestamps)

    timestamps = property(lambda self: self._timestamps)


class ExtendedJaggedTensor(JaggedTensor):
    """JaggedTensor with named per-value side tensors (``extras``) that move and pin with it."""

    def __init__(self, values, weights=None, lengths=None, offsets=None, extras: Optional[Dict[str, torch.Tensor]] = None) -> None:
        super().__init__(values, weights, lengths, offsets)
        self.extras = dict(extras or {})
        for n, t in self.extras.items():
            if t.shape[0] != values.shape[0]:
                raise ValueError("extra %r must have one entry per value" % n)

    def to(self, device: torch.device, non_blocking: bool = False) -> "ExtendedJaggedTensor":
        b = JaggedTensor.to(self, device, non_blocking)
        return ExtendedJaggedTensor(b.values(), b.weights_or_none(), b._lengths, b._offsets,
                                    {n: t.to(device, non_blocking=non_blocking) for n, t in self.extras.items()})

    def record_stream(self, stream) -> None:
        JaggedTensor.record_stream(self, stream)
        for t in self.extras.values():
            if t.is_cuda:
                t.record_stream(stream)

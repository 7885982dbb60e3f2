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
        if hasattr(self, "_unique_offset_host"):          # a host-side copy that travels with whole-batch side tensors
            out._unique_offset_host = self._unique_offset_host
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


    # -- the reference's generic forms (``extended_jagged_tensor.py:288-580``): the caller names the class to build ----------
    def _as(self, constructor, kjt: "_SideTensorKJT"):
        if constructor is None or constructor is type(kjt):
            return kjt
        side = {n: t for n, t in kjt._side().items() if t is not None}
        return constructor(keys=kjt.keys(), values=kjt.values(), weights=kjt.weights_or_none(), lengths=kjt.lengths_or_none(),
                           offsets=kjt.offsets_or_none(), stride=kjt.stride(), **side)

    def split_extend(self, segments: List[int], constructor=None):
        if len(segments) > len(self.keys()):
            raise ValueError("len of segments should be <= len(keys)")
        return [self._as(constructor, p) for p in self.split(segments)]

    def permute_extend(self, indices: List[int], indices_tensor: Optional[torch.Tensor] = None, constructor=None,
                       extra_permute_func=None):
        out = self.permute(indices, indices_tensor)
        if extra_permute_func is not None:
            side = {n: (extra_permute_func(t) if t is not None and n in self.PER_VALUE else t) for n, t in out._side().items()}
            out = self._wrap(out, side)
        return self._as(constructor, out)

    def pin_memory_extend(self, constructor=None):
        return self._as(constructor, self.pin_memory())

    # -- constructors / conversions that keep the side tensors ------------------------------------------------------
    @classmethod
    def from_lengths_sync(cls, keys: List[str], values: torch.Tensor, lengths: torch.Tensor, weights: Optional[torch.Tensor] = None,
                          stride: Optional[int] = None, **side: Optional[torch.Tensor]):
        return cls(keys, values, weights, lengths, None, stride, **side)

    @classmethod
    def from_offsets_sync(cls, keys: List[str], values: torch.Tensor, offsets: torch.Tensor, weights: Optional[torch.Tensor] = None,
                          stride: Optional[int] = None, **side: Optional[torch.Tensor]):
        return cls(keys, values, weights, None, offsets, stride, **side)

    @classmethod
    def empty_like(cls, kjt: KeyedJaggedTensor):
        """No ids, same keys / stride / device; every side tensor empty."""
        v = kjt.values()
        z = torch.zeros(len(kjt.keys()) * kjt.stride(), dtype=torch.int64, device=v.device)
        side = {n: v.new_zeros(0, dtype=torch.int64) for n in cls.PER_VALUE + cls.WHOLE}
        return cls(kjt.keys(), v[:0], None, z, None, kjt.stride(), **side)

    @classmethod
    def concat(cls, kjts: List["_SideTensorKJT"]):
        """Feature-wise concatenation (all inputs share the stride); per-id side tensors follow their ids, whole-batch side
        tensors must be absent (they describe one batch and cannot be merged)."""
        if not kjts:
            raise ValueError("concat of an empty list")
        base = KeyedJaggedTensor.concat(list(kjts))
        side: Dict[str, Optional[torch.Tensor]] = {}
        for n in cls.PER_VALUE:
            ts = [getattr(k, "_" + n) for k in kjts]
            if any(t is None for t in ts):
                if any(t is not None for t in ts):
                    raise ValueError("%s is set on some inputs only" % n)
                side[n] = None
            else:
                side[n] = torch.cat(ts)
        for n in cls.WHOLE:
            if any(getattr(k, "_" + n) is not None for k in kjts):
                raise ValueError("%s describes one batch and cannot be concatenated" % n)
            side[n] = None
        out = cls.__new__(cls)
        out.__dict__.update(base.__dict__)
        out._init_side(**side)
        return out

    def to_dict(self) -> Dict[str, "ExtendedJaggedTensor"]:
        """Per key: an ``ExtendedJaggedTensor`` whose extras are this key's slice of every per-id side tensor."""
        base = KeyedJaggedTensor.to_dict(self)
        opk = self.offset_per_key()
        out = {}
        for i, k in enumerate(self.keys()):
            jt = base[k]
            extras = {n: t[opk[i]:opk[i + 1]] for n, t in self._side().items() if t is not None and n in self.PER_VALUE}
            out[k] = self._jt_class()._rebuild(jt.values(), jt.weights_or_none(), jt._lengths, jt._offsets, extras)
        return out

    @classmethod
    def _jt_class(cls):
        return {"KeyedJaggedTensorWithCount": JaggedTensorWithCount,
                "KeyedJaggedTensorWithTimestamp": JaggedTensorWithTimestamp}.get(cls.__name__, ExtendedJaggedTensor)

    @classmethod
    def from_jt_dict(cls, jt_dict: Dict[str, JaggedTensor]):
        """Key-major concatenation of per-key jagged tensors; per-id side tensors are taken from each tensor's ``extras``
        (all keys must carry the same ones)."""
        keys = list(jt_dict.keys())
        base = KeyedJaggedTensor.from_jt_dict(jt_dict)
        side: Dict[str, Optional[torch.Tensor]] = {}
        for n in cls.PER_VALUE:
            ts = [getattr(jt_dict[k], "extras", {}).get(n) for k in keys]
            if all(t is None for t in ts):
                side[n] = None
            elif any(t is None for t in ts):
                raise ValueError("%s is set on some keys only" % n)
            else:
                side[n] = torch.cat(ts)
        return cls(keys, base.values(), base.weights_or_none(), base.lengths(), None, base.stride(), **side)

    # -- what an all-to-all of this batch has to carry (labels and tensors in matching order) --------------------------
    def dist_labels(self) -> List[str]:
        return KeyedJaggedTensor.dist_labels(self) + [n for n in self.PER_VALUE if getattr(self, "_" + n) is not None]

    def dist_tensors(self) -> List[torch.Tensor]:
        return KeyedJaggedTensor.dist_tensors(self) + [getattr(self, "_" + n) for n in self.PER_VALUE
                                                       if getattr(self, "_" + n) is not None]

    def dist_splits(self, key_splits: List[int]) -> List[List[int]]:
        """Send splits of every distributed tensor when the keys are dealt to ranks as ``key_splits`` (keys per rank):
        lengths travel as ``keys * stride`` entries, values and every per-id side tensor as the ids of those keys."""
        lpk, stride, start = self.length_per_key(), self.stride(), 0
        len_splits, val_splits = [], []
        for n in key_splits:
            len_splits.append(n * stride)
            val_splits.append(sum(lpk[start:start + n]))
            start += n
        return [len_splits] + [list(val_splits) for _ in range(len(self.dist_labels()) - 1)]

    @classmethod
    def dist_init(cls, keys: List[str], tensors: List[torch.Tensor], labels: List[str], stride: int):
        """Rebuild a batch from the tensors an all-to-all delivered (``labels`` as produced by ``dist_labels``)."""
        got = dict(zip(labels, tensors))
        side = {n: got.get(n) for n in cls.PER_VALUE}
        return cls(keys, got["values"], got.get("weights"), got["lengths"], None, stride, **side)

    def __str__(self) -> str:
        parts = ["%s(keys=%s, stride=%d, nnz=%d" % (type(self).__name__, self.keys(), self.stride(), self.values().numel())]
        for n, t in self._side().items():
            parts.append("%s=%s" % (n, "None" if t is None else tuple(t.shape)))
        return ", ".join(parts) + ")"


class KeyedJaggedTensorWithLookHelper(_SideTensorKJT):
    PER_VALUE = ("hash_indices", "unique_inverse")
    WHOLE = ("unique_indices", "unique_offset", "unique_ids")

    def __init__(self, keys, values, weights=None, lengths=None, offsets=None, stride=None, length_per_key=None, offset_per_key=None,
                 hash_indices=None, unique_indices=None, unique_offset=None, unique_inverse=None, unique_ids=None,
                 unique_offset_host=None) -> None:
        super().__init__(keys, values, weights, lengths, offsets, stride, length_per_key, offset_per_key)
        self._init_side(hash_indices=hash_indices, unique_indices=unique_indices, unique_offset=unique_offset, unique_inverse=unique_inverse,
                        unique_ids=unique_ids)
        self._unique_offset_host = None if unique_offset_host is None else list(unique_offset_host)

    @staticmethod
    def from_kjt(kjt: KeyedJaggedTensor, hash_indices=None, unique_indices=None, unique_offset=None, unique_inverse=None, unique_ids=None,
                 unique_offset_host=None):
        return KeyedJaggedTensorWithLookHelper(kjt.keys(), kjt.values(), kjt.weights_or_none(), kjt.lengths_or_none(), kjt.offsets_or_none(),
                                               kjt.stride(), hash_indices=hash_indices, unique_indices=unique_indices,
                                               unique_offset=unique_offset, unique_inverse=unique_inverse, unique_ids=unique_ids,
                                               unique_offset_host=unique_offset_host)

    unique_ids = property(lambda self: self._unique_ids)

    @property
    def unique_offset_host(self):
        """Per-table offsets of the unique list as a host list: the copy given at construction, else read from the tensor
        (a device-to-host copy when it lives on the GPU)."""
        host_copy = getattr(self, "_unique_offset_host", None)
        if host_copy is not None:
            return host_copy
        return None if self._unique_offset is None else self._unique_offset.cpu().tolist()

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

    @classmethod
    def _rebuild(cls, values, weights, lengths, offsets, extras: Dict[str, torch.Tensor]):
        return cls(values, weights, lengths, offsets, extras)

    def to(self, device: torch.device, non_blocking: bool = False) -> "ExtendedJaggedTensor":
        b = JaggedTensor.to(self, device, non_blocking)
        return self._rebuild(b.values(), b.weights_or_none(), b._lengths, b._offsets,
                             {n: t.to(device, non_blocking=non_blocking) for n, t in self.extras.items()})

    def record_stream(self, stream) -> None:
        JaggedTensor.record_stream(self, stream)
        for t in self.extras.values():
            if t.is_cuda:
                t.record_stream(stream)

    @property
    def extra(self) -> Optional[torch.Tensor]:
        """The side tensor when there is exactly one (the reference's classes carry a single ``extra``); else None."""
        return next(iter(self.extras.values())) if len(self.extras) == 1 else None


class JaggedTensorWithCount(ExtendedJaggedTensor):
    """JaggedTensor whose ids carry their number of occurrences (``hybrid_torchrec/sparse/jagged_tensor_with_count.py:24-49``)."""

    def __init__(self, values, weights=None, lengths=None, offsets=None, counts=None) -> None:
        super().__init__(values, weights, lengths, offsets, {} if counts is None else {"counts": counts})

    @classmethod
    def _rebuild(cls, values, weights, lengths, offsets, extras):
        return cls(values, weights, lengths, offsets, extras.get("counts"))

    counts = property(lambda self: self.extras.get("counts"))


class JaggedTensorWithTimestamp(ExtendedJaggedTensor):
    """JaggedTensor whose ids carry a timestamp (``torchrec_embcache/sparse/jagged_tensor_with_timestamp.py:31-59``)."""

    def __init__(self, values, weights=None, lengths=None, offsets=None, timestamps=None) -> None:
        super().__init__(values, weights, lengths, offsets, {} if timestamps is None else {"timestamps": timestamps})

    @classmethod
    def _rebuild(cls, values, weights, lengths, offsets, extras):
        return cls(values, weights, lengths, offsets, extras.get("timestamps"))

    timestamps = property(lambda self: self.extras.get("timestamps"))


class KeyedExtendedJaggedTensor(_SideTensorKJT):
    """KJT with one generic per-id side tensor ``extra`` (any dtype; e.g. labels or timestamps) and the argument checks
    of the reference's class (``hybrid_torchrec/sparse/extended_jagged_tensor.py:69-235``): distinct keys, a positive
    stride, per-key list arguments that are integer lists of the right length, ``extra`` aligned with the ids."""
    PER_VALUE = ("extra",)

    def __init__(self, keys, values, weights=None, lengths=None, offsets=None, stride=None, length_per_key=None, offset_per_key=None,
                 extra=None) -> None:
        self._validate_keys(keys)
        self._validate_stride(stride)
        self._validate_int_list(length_per_key, "length_per_key", len(keys))
        self._validate_int_list(offset_per_key, "offset_per_key", len(keys) + 1)
        if lengths is None and offsets is None:
            raise ValueError("either lengths or offsets is required")
        super().__init__(keys, values, weights, lengths, offsets, stride, length_per_key, offset_per_key)
        self._init_side(extra=extra)

    extra = property(lambda self: self._extra)

    @staticmethod
    def _validate_keys(keys) -> None:
        if not isinstance(keys, (list, tuple)) or not all(isinstance(k, str) for k in keys):
            raise TypeError("keys must be a list of strings")
        if len(set(keys)) != len(keys):
            raise ValueError("duplicate keys: %s" % sorted(k for k in set(keys) if list(keys).count(k) > 1))

    @staticmethod
    def _validate_stride(stride) -> None:
        if stride is not None and (not isinstance(stride, int) or isinstance(stride, bool) or stride < 0):
            raise ValueError("stride must be a non-negative int, got %r" % (stride,))

    @staticmethod
    def _validate_int_list(v, name: str, want_len: int) -> None:
        if v is None:
            return
        if not isinstance(v, (list, tuple)) or not all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            raise TypeError("%s must be a list of ints" % name)
        if len(v) != want_len:
            raise ValueError("%s needs %d entries, got %d" % (name, want_len, len(v)))

    def to_base(self) -> KeyedJaggedTensor:
        """The plain KJT (side tensor dropped)."""
        return KeyedJaggedTensor(self.keys(), self.values(), self.weights_or_none(), self.lengths_or_none(), self.offsets_or_none(),
                                 self.stride())

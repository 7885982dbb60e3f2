"""Jagged sparse-feature containers: ``JaggedTensor``, ``KeyedJaggedTensor``, ``KeyedTensor``.

API-compatible subset of the TorchRec types that every module of the reference consumes
(``hybrid_torchrec/sparse/*`` subclasses them; TorchRec itself is not part of the reference tree).
Layout: for keys ``k_0..k_{F-1}`` and batch size ``B`` (``stride``), ``lengths`` has ``F*B`` entries in
key-major order and ``values`` holds the concatenated ids of bag ``(k, b)`` in that order.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch


def _cumsum0(lengths: torch.Tensor) -> torch.Tensor:
    out = torch.zeros(lengths.numel() + 1, dtype=torch.int64, device=lengths.device)
    torch.cumsum(lengths.reshape(-1), 0, out=out[1:])
    return out


class JaggedTensor:
    """``values`` [nnz(, D)] with per-row ``lengths`` / ``offsets`` (one of the two is enough)."""

    def __init__(self, values: torch.Tensor, weights: Optional[torch.Tensor] = None,
                 lengths: Optional[torch.Tensor] = None, offsets: Optional[torch.Tensor] = None) -> None:
        if lengths is None and offsets is None:
            raise ValueError("JaggedTensor needs lengths or offsets")
        self._values = values
        self._weights = weights
        self._lengths = lengths
        self._offsets = offsets

    @staticmethod
    def empty(is_weighted: bool = False, device: Optional[torch.device] = None,
              values_dtype: torch.dtype = torch.int64) -> "JaggedTensor":
        w = torch.empty(0, device=device) if is_weighted else None
        return JaggedTensor(torch.empty(0, dtype=values_dtype, device=device), w,
                            lengths=torch.empty(0, dtype=torch.int64, device=device))

    @staticmethod
    def from_dense(values: Sequence[torch.Tensor], weights: Optional[Sequence[torch.Tensor]] = None) -> "JaggedTensor":
        lengths = torch.tensor([v.shape[0] for v in values], dtype=torch.int64)
        vals = torch.cat(list(values)) if len(values) else torch.empty(0)
        w = torch.cat(list(weights)) if weights is not None else None
        return JaggedTensor(vals, w, lengths=lengths.to(vals.device))

    def values(self) -> torch.Tensor:
        return self._values

    def weights(self) -> torch.Tensor:
        if self._weights is None:
            raise ValueError("JaggedTensor has no weights")
        return self._weights

    def weights_or_none(self) -> Optional[torch.Tensor]:
        return self._weights

    def lengths(self) -> torch.Tensor:
        if self._lengths is None:
            self._lengths = self._offsets[1:] - self._offsets[:-1]
        return self._lengths

    def offsets(self) -> torch.Tensor:
        if self._offsets is None:
            self._offsets = _cumsum0(self._lengths)
        return self._offsets

    def to_dense(self) -> List[torch.Tensor]:
        off = self.offsets().tolist()
        return [self._values[off[i]:off[i + 1]] for i in range(len(off) - 1)]

    def to_padded_dense(self, desired_length: Optional[int] = None, padding_value: float = 0.0) -> torch.Tensor:
        lengths = self.lengths()
        n = lengths.numel()
        max_len = int(lengths.max().item()) if n else 0
        L = desired_length if desired_length is not None else max_len
        tail = self._values.shape[1:]
        out = self._values.new_full((n, L) + tuple(tail), padding_value)
        off = self.offsets()
        pos = torch.arange(self._values.shape[0], device=self._values.device)
        row = torch.repeat_interleave(torch.arange(n, device=pos.device), lengths)
        col = pos - off[:-1][row]
        keep = col < L
        out[row[keep], col[keep]] = self._values[keep]
        return out

    def to(self, device: torch.device, non_blocking: bool = False) -> "JaggedTensor":
        mv = lambda t: None if t is None else t.to(device, non_blocking=non_blocking)  # noqa: E731
        return JaggedTensor(mv(self._values), mv(self._weights), mv(self._lengths), mv(self._offsets))

    def record_stream(self, stream) -> None:
        for t in (self._values, self._weights, self._lengths, self._offsets):
            if t is not None and t.is_cuda:
                t.record_stream(stream)

    def __repr__(self) -> str:
        return "JaggedTensor(values=%s, lengths=%s)" % (self._values, self.lengths())


class KeyedJaggedTensor:
    """Batch of jagged features keyed by feature name (key-major layout)."""

    def __init__(self, keys: List[str], values: torch.Tensor, weights: Optional[torch.Tensor] = None,
                 lengths: Optional[torch.Tensor] = None, offsets: Optional[torch.Tensor] = None,
                 stride: Optional[int] = None, length_per_key: Optional[List[int]] = None,
                 offset_per_key: Optional[List[int]] = None) -> None:
        if lengths is None and offsets is None:
            raise ValueError("KeyedJaggedTensor needs lengths or offsets")
        self._keys = list(keys)
        self._values = values
        self._weights = weights
        self._lengths = lengths
        self._offsets = offsets
        n = lengths.numel() if lengths is not None else offsets.numel() - 1
        if stride is None:
            stride = n // len(self._keys) if self._keys else 0
        self._stride = stride
        self._length_per_key = length_per_key
        self._offset_per_key = offset_per_key
        # True when the producer guarantees every bag holds exactly one id (fast paths skip offsets)
        self.one_hot = False

    def _carry(self, other: "KeyedJaggedTensor") -> "KeyedJaggedTensor":
        other.one_hot = self.one_hot
        return other

    # -- constructors ---------------------------------------------------------
    @staticmethod
    def from_lengths_sync(keys: List[str], values: torch.Tensor, lengths: torch.Tensor,
                          weights: Optional[torch.Tensor] = None, stride: Optional[int] = None) -> "KeyedJaggedTensor":
        kjt = KeyedJaggedTensor(keys, values, weights, lengths=lengths, stride=stride)
        kjt.length_per_key()
        return kjt

    @staticmethod
    def from_offsets_sync(keys: List[str], values: torch.Tensor, offsets: torch.Tensor,
                          weights: Optional[torch.Tensor] = None, stride: Optional[int] = None) -> "KeyedJaggedTensor":
        kjt = KeyedJaggedTensor(keys, values, weights, offsets=offsets, stride=stride)
        kjt.length_per_key()
        return kjt

    @staticmethod
    def from_jt_dict(jt_dict: Dict[str, JaggedTensor]) -> "KeyedJaggedTensor":
        keys = list(jt_dict.keys())
        values = torch.cat([jt_dict[k].values() for k in keys])
        lengths = torch.cat([jt_dict[k].lengths() for k in keys])
        ws = [jt_dict[k].weights_or_none() for k in keys]
        weights = torch.cat(ws) if all(w is not None for w in ws) and ws else None
        return KeyedJaggedTensor(keys, values, weights, lengths=lengths)

    @staticmethod
    def empty(is_weighted: bool = False, device: Optional[torch.device] = None,
              values_dtype: torch.dtype = torch.int64) -> "KeyedJaggedTensor":
        w = torch.empty(0, device=device) if is_weighted else None
        return KeyedJaggedTensor([], torch.empty(0, dtype=values_dtype, device=device), w,
                                 lengths=torch.empty(0, dtype=torch.int64, device=device), stride=0)

    @staticmethod
    def concat(kjts: List["KeyedJaggedTensor"]) -> "KeyedJaggedTensor":
        keys: List[str] = []
        for k in kjts:
            keys += k.keys()
        ws = [k.weights_or_none() for k in kjts]
        out = KeyedJaggedTensor(keys, torch.cat([k.values() for k in kjts]),
                                torch.cat(ws) if all(w is not None for w in ws) else None,
                                lengths=torch.cat([k.lengths() for k in kjts]), stride=kjts[0].stride())
        out.one_hot = all(k.one_hot for k in kjts)
        return out

    # -- accessors ------------------------------------------------------------
    def keys(self) -> List[str]:
        return self._keys

    def values(self) -> torch.Tensor:
        return self._values

    def weights(self) -> torch.Tensor:
        if self._weights is None:
            raise ValueError("KeyedJaggedTensor has no weights")
        return self._weights

    def weights_or_none(self) -> Optional[torch.Tensor]:
        return self._weights

    def lengths(self) -> torch.Tensor:
        if self._lengths is None:
            self._lengths = self._offsets[1:] - self._offsets[:-1]
        return self._lengths

    def offsets(self) -> torch.Tensor:
        if self._offsets is None:
            self._offsets = _cumsum0(self._lengths)
        return self._offsets

    def lengths_or_none(self) -> Optional[torch.Tensor]:
        return self._lengths

    def offsets_or_none(self) -> Optional[torch.Tensor]:
        return self._offsets

    def stride(self) -> int:
        return self._stride

    def device(self) -> torch.device:
        return self._values.device

    def length_per_key(self) -> List[int]:
        if self._length_per_key is None:
            if not self._keys:
                self._length_per_key = []
            else:
                self._length_per_key = self.lengths().reshape(len(self._keys), -1).sum(dim=1).tolist()
        return self._length_per_key

    def offset_per_key(self) -> List[int]:
        if self._offset_per_key is None:
            acc, out = 0, [0]
            for n in self.length_per_key():
                acc += n
                out.append(acc)
            self._offset_per_key = out
        return self._offset_per_key

    # -- small accessors of the TorchRec container that user code commonly calls ---------------------------------------
    def index_per_key(self) -> Dict[str, int]:
        return self._key_indices()

    def variable_stride_per_key(self) -> bool:
        """Every key has the same number of bags here (one per sample)."""
        return False

    def stride_per_key(self) -> List[int]:
        return [self._stride] * len(self._keys)

    def lengths_offset_per_key(self) -> List[int]:
        """Start of every key's bags in ``lengths()`` (``[0, B, 2B, ...]``)."""
        return [i * self._stride for i in range(len(self._keys) + 1)]

    def inverse_indices_or_none(self):
        return None

    def flatten_lengths(self) -> "KeyedJaggedTensor":
        return self._carry(KeyedJaggedTensor(self._keys, self._values, self._weights, self.lengths().reshape(-1), None, self._stride,
                                             self._length_per_key, self._offset_per_key))

    def sync(self) -> "KeyedJaggedTensor":
        """Compute the host-side per-key lengths and offsets now (one device-to-host read for device tensors)."""
        self.length_per_key()
        self.offset_per_key()
        return self

    def unsync(self) -> "KeyedJaggedTensor":
        self._length_per_key = None
        self._offset_per_key = None
        return self

    @staticmethod
    def empty_like(kjt: "KeyedJaggedTensor") -> "KeyedJaggedTensor":
        """No ids, same keys, stride and device."""
        v = kjt.values()
        w = kjt.weights_or_none()
        return KeyedJaggedTensor(kjt.keys(), v[:0], None if w is None else w[:0],
                                 lengths=torch.zeros(len(kjt.keys()) * kjt.stride(), dtype=torch.int64, device=v.device), stride=kjt.stride())

    def __len__(self) -> int:
        return len(self._keys)

    def _key_indices(self) -> Dict[str, int]:
        return {k: i for i, k in enumerate(self._keys)}

    # -- transforms -----------------------------------------------------------
    def split(self, segments: List[int]) -> List["KeyedJaggedTensor"]:
        out, start, opk = [], 0, self.offset_per_key()
        B = self._stride
        for seg in segments:
            end = start + seg
            keys = self._keys[start:end]
            v0, v1 = opk[start], opk[end]
            out.append(self._carry(KeyedJaggedTensor(
                keys, self._values[v0:v1], None if self._weights is None else self._weights[v0:v1],
                lengths=self.lengths()[start * B:end * B], stride=B,
                length_per_key=self.length_per_key()[start:end])))
            start = end
        return out

    def permute(self, indices: List[int], indices_tensor: Optional[torch.Tensor] = None) -> "KeyedJaggedTensor":
        B, opk = self._stride, self.offset_per_key()
        lens = self.lengths().reshape(len(self._keys), B) if self._keys else self.lengths().reshape(0, 0)
        keys = [self._keys[i] for i in indices]
        vals = [self._values[opk[i]:opk[i + 1]] for i in indices]
        ws = None if self._weights is None else [self._weights[opk[i]:opk[i + 1]] for i in indices]
        idx = indices_tensor if indices_tensor is not None else torch.tensor(indices, dtype=torch.int64, device=lens.device)
        return self._carry(KeyedJaggedTensor(
            keys, torch.cat(vals) if vals else self._values[:0],
            None if ws is None else (torch.cat(ws) if ws else self._weights[:0]),
            lengths=lens[idx].reshape(-1), stride=B, length_per_key=[self.length_per_key()[i] for i in indices]))

    def __getitem__(self, key: str) -> JaggedTensor:
        i = self._key_indices()[key]
        opk, B = self.offset_per_key(), self._stride
        return JaggedTensor(self._values[opk[i]:opk[i + 1]],
                            None if self._weights is None else self._weights[opk[i]:opk[i + 1]],
                            lengths=self.lengths()[i * B:(i + 1) * B])

    def to_dict(self) -> Dict[str, JaggedTensor]:
        return {k: self[k] for k in self._keys}

    def to(self, device: torch.device, non_blocking: bool = False) -> "KeyedJaggedTensor":
        mv = lambda t: None if t is None else t.to(device, non_blocking=non_blocking)  # noqa: E731
        return self._carry(KeyedJaggedTensor(self._keys, mv(self._values), mv(self._weights), mv(self._lengths),
                                             mv(self._offsets), self._stride, self._length_per_key,
                                             self._offset_per_key))

    def pin_memory(self) -> "KeyedJaggedTensor":
        pm = lambda t: None if t is None else (t if t.is_pinned() else t.pin_memory())  # noqa: E731
        return self._carry(KeyedJaggedTensor(self._keys, pm(self._values), pm(self._weights), pm(self._lengths),
                                             pm(self._offsets), self._stride, self._length_per_key,
                                             self._offset_per_key))

    def record_stream(self, stream) -> None:
        for t in (self._values, self._weights, self._lengths, self._offsets):
            if t is not None and t.is_cuda:
                t.record_stream(stream)

    def dist_labels(self) -> List[str]:
        labels = ["lengths", "values"]
        if self._weights is not None:
            labels.append("weights")
        return labels

    def dist_tensors(self) -> List[torch.Tensor]:
        out = [self.lengths(), self._values]
        if self._weights is not None:
            out.append(self._weights)
        return out

    def __repr__(self) -> str:
        return "KeyedJaggedTensor(keys=%s, stride=%d, nnz=%d)" % (self._keys, self._stride, self._values.numel())


class KeyedTensor:
    """Dense ``[B, sum(D_k)]`` tensor with per-key column ranges (pooled embedding output)."""

    def __init__(self, keys: List[str], length_per_key: List[int], values: torch.Tensor, key_dim: int = 1) -> None:
        self._keys = list(keys)
        self._length_per_key = list(length_per_key)
        self._values = values
        self._key_dim = key_dim
        acc, off = 0, [0]
        for n in self._length_per_key:
            acc += n
            off.append(acc)
        self._offset_per_key = off

    @staticmethod
    def from_tensor_list(keys: List[str], tensors: List[torch.Tensor], key_dim: int = 1, cat_dim: int = 1) -> "KeyedTensor":
        return KeyedTensor(keys, [t.shape[key_dim] for t in tensors], torch.cat(tensors, dim=cat_dim), key_dim)

    def keys(self) -> List[str]:
        return self._keys

    def values(self) -> torch.Tensor:
        return self._values

    def key_dim(self) -> int:
        return self._key_dim

    def length_per_key(self) -> List[int]:
        return self._length_per_key

    def offset_per_key(self) -> List[int]:
        return self._offset_per_key

    def __getitem__(self, key: str) -> torch.Tensor:
        i = self._keys.index(key)
        return self._values.narrow(self._key_dim, self._offset_per_key[i], self._length_per_key[i])

    def to_dict(self) -> Dict[str, torch.Tensor]:
        return {k: self[k] for k in self._keys}

    def to(self, device: torch.device, non_blocking: bool = False) -> "KeyedTensor":
        return KeyedTensor(self._keys, self._length_per_key, self._values.to(device, non_blocking=non_blocking), self._key_dim)

    def record_stream(self, stream) -> None:
        if self._values.is_cuda:
            self._values.record_stream(stream)

    @staticmethod
    def regroup(keyed_tensors: List["KeyedTensor"], groups: List[List[str]]) -> List[torch.Tensor]:
        lookup: Dict[str, Tuple["KeyedTensor", str]] = {}
        for kt in keyed_tensors:
            for k in kt.keys():
                lookup[k] = (kt, k)
        return [torch.cat([lookup[k][0][k] for k in g], dim=1) for g in groups]

    def __repr__(self) -> str:
        return "KeyedTensor(keys=%s, shape=%s)" % (self._keys, tuple(self._values.shape))


class KJTList:
    """A list of ``KeyedJaggedTensor`` that moves as one unit (one entry per sharding group of a module's input)."""

    def __init__(self, features) -> None:
        self.features = list(features)

    def __len__(self) -> int:
        return len(self.features)

    def __getitem__(self, i: int) -> KeyedJaggedTensor:
        return self.features[i]

    def __iter__(self):
        return iter(self.features)

    def to(self, device: torch.device, non_blocking: bool = False) -> "KJTList":
        return KJTList([f.to(device, non_blocking=non_blocking) for f in self.features])

    def pin_memory(self) -> "KJTList":
        return KJTList([f.pin_memory() for f in self.features])

    def record_stream(self, stream) -> None:
        for f in self.features:
            f.record_stream(stream)


def kjt_list_to_device(batch: KJTList, device: torch.device, non_blocking: bool = False) -> KJTList:
    """Pin every entry and start its copy to ``device`` (reference ``hybrid_torchrec/distributed/embedding_types.py:15-31``)."""
    if not isinstance(batch, KJTList):
        raise ValueError("%s must be KJTList" % type(batch))
    pin = torch.cuda.is_available()
    return KJTList([(f.pin_memory() if pin else f).to(device, non_blocking=non_blocking) for f in batch.features])

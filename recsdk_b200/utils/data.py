"""Batches and synthetic recommendation data.

``Batch`` is the pipelineable container (``to`` / ``record_stream`` / ``pin_memory``) the train pipelines
move across streams (reference user flow: ``docs/en/torch/torch_rec_v1/03_quick_start/quick_start.md:145-170``).
``RandomRecDataset`` draws ids from a bounded power law (Zipf-like, exponent ``alpha``) per table,
scattered over the table with a multiplicative bijection so that hot rows are not neighbours.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Iterator, List, Optional, Sequence

import torch

from ..sparse.jagged_tensor import KeyedJaggedTensor


@dataclasses.dataclass
class Batch:
    dense_features: torch.Tensor
    sparse_features: KeyedJaggedTensor
    labels: torch.Tensor

    def to(self, device: torch.device, non_blocking: bool = False) -> "Batch":
        return Batch(self.dense_features.to(device, non_blocking=non_blocking),
                     self.sparse_features.to(device, non_blocking=non_blocking),
                     self.labels.to(device, non_blocking=non_blocking))

    def record_stream(self, stream) -> None:
        if self.dense_features.is_cuda:
            self.dense_features.record_stream(stream)
            self.labels.record_stream(stream)
        self.sparse_features.record_stream(stream)

    def pin_memory(self) -> "Batch":
        pm = lambda t: t if t.is_pinned() else t.pin_memory()  # noqa: E731
        return Batch(pm(self.dense_features), self.sparse_features.pin_memory(), pm(self.labels))

    def nbytes(self) -> int:
        n = self.dense_features.numel() * self.dense_features.element_size()
        n += self.labels.numel() * self.labels.element_size()
        kjt = self.sparse_features
        for t in (kjt.values(), kjt.lengths_or_none(), kjt.offsets_or_none(), kjt.weights_or_none()):
            if t is not None:
                n += t.numel() * t.element_size()
        return n


def zipf_ids(n: int, num_rows: int, alpha: float, gen: torch.Generator, device=None) -> torch.Tensor:
    """``n`` ids in ``[0, num_rows)`` with P(rank k) ~ k^-alpha (continuous inverse-CDF sampling), then
    scattered by ``id = rank * P mod num_rows`` with ``P`` coprime to ``num_rows``."""
    u = torch.rand(n, generator=gen, device=device, dtype=torch.float64)
    if abs(alpha - 1.0) < 1e-9:
        x = torch.exp(u * math.log(num_rows + 1.0))
    else:
        a = 1.0 - alpha
        x = ((float(num_rows + 1) ** a - 1.0) * u + 1.0) ** (1.0 / a)
    rank = torch.clamp(x.floor().to(torch.int64) - 1, 0, num_rows - 1)
    p = 2654435761 % num_rows
    while math.gcd(p, num_rows) != 1:
        p += 1
    return (rank * p) % num_rows


class RandomRecDataset:
    """Endless iterator of ``Batch`` objects on the host (optionally pinned).

    ``hash_sizes[i]`` rows for feature ``keys[i]``; bag lengths are 1 (``one_hot``) or Uniform
    ``[min_len, max_len]``; dense features ~ N(0,1); labels ~ Bernoulli(``pos_rate``).
    """

    def __init__(self, keys: Sequence[str], hash_sizes: Sequence[int], batch_size: int, num_dense: int = 13,
                 alpha: float = 1.05, one_hot: bool = True, min_len: int = 1, max_len: int = 1,
                 pos_rate: float = 0.25, seed: int = 0, pin: bool = False, num_batches: Optional[int] = None,
                 ids_dtype: torch.dtype = torch.int64) -> None:
        self.keys, self.hash_sizes = list(keys), [int(h) for h in hash_sizes]
        self.B, self.num_dense, self.alpha = batch_size, num_dense, alpha
        self.one_hot, self.min_len, self.max_len = one_hot, min_len, max_len
        self.pos_rate, self.pin, self.num_batches = pos_rate, pin, num_batches
        self.ids_dtype = ids_dtype
        self.gen = torch.Generator().manual_seed(seed)

    def make_batch(self) -> Batch:
        B, g = self.B, self.gen
        vals: List[torch.Tensor] = []
        lens: List[torch.Tensor] = []
        for hs in self.hash_sizes:
            if self.one_hot:
                ln = torch.ones(B, dtype=torch.int64)
            else:
                ln = torch.randint(self.min_len, self.max_len + 1, (B,), generator=g)
            lens.append(ln)
            vals.append(zipf_ids(int(ln.sum()), hs, self.alpha, g))
        values = torch.cat(vals).to(self.ids_dtype)
        lengths = torch.cat(lens)
        kjt = KeyedJaggedTensor(self.keys, values, lengths=lengths, stride=B)
        kjt.one_hot = self.one_hot  # type: ignore[attr-defined]
        dense = torch.randn(B, self.num_dense, generator=g)
        labels = (torch.rand(B, generator=g) < self.pos_rate).float()
        b = Batch(dense, kjt, labels)
        return b.pin_memory() if self.pin else b

    def __iter__(self) -> Iterator[Batch]:
        i = 0
        while self.num_batches is None or i < self.num_batches:
            yield self.make_batch()
            i += 1

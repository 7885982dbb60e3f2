"""Initializer objects of the dynamic-embedding API: ``initializer(buffer, indices, keys)`` fills the rows ``indices`` of
``buffer`` (``[rows, dim]``).  Normal, truncated normal (resampled until inside ``[lower, upper]``... bounded: after a few
rounds the stragglers are clamped), uniform, constant and the debugging one (every element of a row = ``key % 100000``).
The tables draw new rows inside their insert kernel from the same distributions; these objects serve user code that
fills buffers itself.  Reference: ``dynamic_emb/distributed/initializers/dynamicemb_initializers.py:37-123``.
"""
from __future__ import annotations

import abc
from typing import Optional

import torch

from .dynamicemb_config import DynamicEmbInitializerArgs, DynamicEmbInitializerMode


class BaseDynamicEmbInitializer(abc.ABC):
    def __init__(self, args: DynamicEmbInitializerArgs, seed: Optional[int] = None) -> None:
        self._args = args
        if self._args.lower is None:
            self._args.lower = 0.0
        if self._args.upper is None:
            self._args.upper = 1.0
        self._gen: Optional[torch.Generator] = None
        self._seed = seed

    def _generator(self, device: torch.device) -> Optional[torch.Generator]:
        if self._seed is None:
            return None
        if self._gen is None or self._gen.device != device:
            self._gen = torch.Generator(device=device).manual_seed(self._seed)
        return self._gen

    def _rows(self, buffer: torch.Tensor, indices: torch.Tensor):
        if buffer.dim() != 2:
            raise ValueError("buffer must be [rows, dim]")
        return indices.numel(), buffer.shape[1]

    @abc.abstractmethod
    def __call__(self, buffer: torch.Tensor, indices: torch.Tensor, keys: Optional[torch.Tensor] = None) -> None: ...


class NormalInitializer(BaseDynamicEmbInitializer):
    def __call__(self, buffer, indices, keys=None) -> None:
        n, d = self._rows(buffer, indices)
        x = torch.randn(n, d, device=buffer.device, generator=self._generator(buffer.device))
        buffer[indices.long()] = (x * self._args.std_dev + self._args.mean).to(buffer.dtype)


class UniformInitializer(BaseDynamicEmbInitializer):
    def __call__(self, buffer, indices, keys=None) -> None:
        n, d = self._rows(buffer, indices)
        x = torch.rand(n, d, device=buffer.device, generator=self._generator(buffer.device))
        buffer[indices.long()] = (self._args.lower + (self._args.upper - self._args.lower) * x).to(buffer.dtype)


class TruncatedNormalInitializer(BaseDynamicEmbInitializer):
    ROUNDS = 32

    def __call__(self, buffer, indices, keys=None) -> None:
        n, d = self._rows(buffer, indices)
        a = self._args
        g = self._generator(buffer.device)
        x = torch.randn(n, d, device=buffer.device, generator=g) * a.std_dev + a.mean
        for _ in range(self.ROUNDS):
            bad = (x < a.lower) | (x > a.upper)
            if not bool(bad.any()):
                break
            x = torch.where(bad, torch.randn(n, d, device=buffer.device, generator=g) * a.std_dev + a.mean, x)
        buffer[indices.long()] = x.clamp(a.lower, a.upper).to(buffer.dtype)


class ConstantInitializer(BaseDynamicEmbInitializer):
    def __call__(self, buffer, indices, keys=None) -> None:
        buffer[indices.long()] = self._args.value


class DebugInitializer(BaseDynamicEmbInitializer):
    def __call__(self, buffer, indices, keys=None) -> None:
        if keys is None:
            raise ValueError("DebugInitializer requires keys, but got None.")
        buffer[indices.long()] = (keys.long() % 100000).to(buffer.dtype)[:, None].expand(-1, buffer.shape[1])


_BY_MODE = {DynamicEmbInitializerMode.NORMAL: NormalInitializer, DynamicEmbInitializerMode.TRUNCATED_NORMAL: TruncatedNormalInitializer,
            DynamicEmbInitializerMode.UNIFORM: UniformInitializer, DynamicEmbInitializerMode.CONSTANT: ConstantInitializer,
            DynamicEmbInitializerMode.DEBUG: DebugInitializer}


def create_initializer(args: DynamicEmbInitializerArgs, seed: Optional[int] = None) -> BaseDynamicEmbInitializer:
    return _BY_MODE[args.mode](args, seed)

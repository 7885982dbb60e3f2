"""Training pipeline for models with multi-tier (embcache) tables.

While batch i runs forward / backward on the compute stream, batch i+1 is copied to the device, distributed to
its owner ranks, its swap plan is computed on the native thread pool, the victims leave for host memory and the
incoming rows arrive - all on side streams.  Every ``evict_step_interval`` steps the feature filter evicts stale
features from all tiers.  Reference: ``torchrec_embcache/distributed/train_pipeline.py:226-293`` (signature),
``:574-633`` (fill), ``:656-731`` (progress), swap stages ``:424-537``.
"""
from __future__ import annotations

from typing import Any, Callable, Iterator, List, Optional

import torch

from ..parallel.train_pipeline import TrainPipelineBase
from .configs import MIN_EVICT_STEP_INTERVAL
from .embedding_bag import EmbCacheShardedEmbeddingBagCollection


def embcache_modules(model: torch.nn.Module) -> List[EmbCacheShardedEmbeddingBagCollection]:
    return [m for m in model.modules() if isinstance(m, EmbCacheShardedEmbeddingBagCollection)]


class EmbCacheTrainPipelineSparseDist(TrainPipelineBase):
    def __init__(self, model: torch.nn.Module, optimizer, cpu_device=None, npu_device=None, return_loss: bool = False,
                 evict_step_interval: Optional[int] = None, execute_all_batches: bool = True, apply_jit: bool = False,
                 context_type=None, pipeline_postproc: bool = False, custom_model_fwd: Optional[Callable] = None,
                 custom_model_zero_grad: Optional[Callable] = None, custom_model_bwd: Optional[Callable] = None,
                 sparse_features_of: Callable[[Any], Any] = lambda batch: batch.sparse_features) -> None:
        device = torch.device(npu_device) if npu_device is not None else torch.device("cpu")
        super().__init__(model, optimizer, device, return_loss)
        if evict_step_interval is not None and evict_step_interval < MIN_EVICT_STEP_INTERVAL:
            raise ValueError("evict_step_interval must be >= %d" % MIN_EVICT_STEP_INTERVAL)
        self._evict_every = evict_step_interval
        self._execute_all = execute_all_batches
        self._fwd, self._zero, self._bwd = custom_model_fwd, custom_model_zero_grad, custom_model_bwd
        self._features_of = sparse_features_of
        self._mods = embcache_modules(model)
        self._cuda = device.type == "cuda"
        self._copy_stream = torch.cuda.Stream(device) if self._cuda else None
        self._next = None
        self._exhausted = False
        self._steps = 0

    def _fetch(self, it: Iterator):
        """Next batch: H2D copy on the copy stream, then the prefetch (input dist + swap) for every embcache module."""
        try:
            host_batch = next(it)
        except StopIteration:
            self._exhausted = True
            return None
        if self._cuda:
            with torch.cuda.stream(self._copy_stream):
                batch = host_batch.to(self._device, non_blocking=True)
            torch.cuda.current_stream(self._device).wait_stream(self._copy_stream)
            batch.record_stream(torch.cuda.current_stream(self._device))
        else:
            batch = host_batch.to(self._device)
        feats = self._features_of(batch)
        for m in self._mods:
            m.prefetch(feats)
        return batch

    def progress(self, dataloader_iter: Iterator):
        if self._next is None and not self._exhausted:
            self._next = self._fetch(dataloader_iter)
        if self._next is None:
            raise StopIteration
        batch = self._next
        # batch i+1: copy, distribute and swap while batch i computes
        self._next = self._fetch(dataloader_iter) if not self._exhausted else None
        (self._zero or self._optimizer.zero_grad)()
        loss, out = (self._fwd or self._model)(batch)
        (self._bwd(loss) if self._bwd else loss.backward())
        sync = getattr(self._model, "sync_dense_grads", None)
        if sync is not None:
            sync()
        self._optimizer.step()
        self._steps += 1
        if self._evict_every and self._steps % self._evict_every == 0:
            for m in self._mods:
                m.host_embedding_evict()
        loss = loss.detach()
        return (loss, out) if self._return_loss else out

"""Training pipeline for models with multi-tier (embcache) tables.

Stages per call of ``progress`` (CUDA), in the order they are issued:

1. the compute stream waits for the swap of batch i (one event) and gets forward / backward / optimizer of batch i;
2. while the GPU works on that, the host takes batch i+1: pinned host-to-device copy on the copy stream, input
   distribution on the host copy of the ids (native bucketize; gloo exchange with several ranks), per-table batch
   planning on the native thread pool (distinct keys, admission statistics, swap plan);
3. the swap traffic of batch i+1 goes to the memcpy stream, which first waits for the backward of batch i-1 (the last
   step that may have trained a victim): victims gather -> pinned buffer (``cudaMemcpyAsync`` D2H) -> host
   ``embedding_update`` on a worker; host ``embedding_lookup`` -> pinned buffer -> ``cudaMemcpyAsync`` H2D -> scatter.

The slot allocator never hands a batch a slot that the current or the previous batch uses, so the swap of batch i+1
touches rows that batch i does not read or train.  Every ``evict_step_interval`` steps the feature filter evicts stale
features from all tiers.  Without CUDA (or with several ranks and no host process group) the swap runs synchronously
inside ``prefetch``.  ``LOCAL_UNIQUE_PARALLEL_BATCH_NUM`` (1..24, default 2) is validated like the reference does and
bounds how many batches the host stages may run ahead.
Reference: ``torchrec_embcache/distributed/train_pipeline.py:226-293`` (signature, environment check ``:274-290``),
``:574-633`` (fill), ``:656-731`` (progress), swap stages ``:424-537``.
"""
from __future__ import annotations

import os
from typing import Any, Callable, Iterator, List, Optional

import torch
from torch.autograd.profiler import record_function

from ..parallel.train_pipeline import TrainPipelineBase
from .configs import MIN_EVICT_STEP_INTERVAL

MAX_LOCAL_UNIQUE_PARALLEL_BATCH_NUM = 24
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
        raw = os.environ.get("LOCAL_UNIQUE_PARALLEL_BATCH_NUM", "2")
        if not raw.isdigit():
            raise ValueError("Param error, LOCAL_UNIQUE_PARALLEL_BATCH_NUM must be a number, but got %s." % raw)
        self.local_unique_parallel_batch_num = int(raw)
        if not 1 <= self.local_unique_parallel_batch_num <= MAX_LOCAL_UNIQUE_PARALLEL_BATCH_NUM:
            raise ValueError("Param error: LOCAL_UNIQUE_PARALLEL_BATCH_NUM must be in [1, %d], but got %s."
                             % (MAX_LOCAL_UNIQUE_PARALLEL_BATCH_NUM, raw))
        self._async = self._cuda and all(m._async_ready() for m in self._mods)

    def _fetch(self, it: Iterator):
        """Next batch: H2D copy on the copy stream, then input dist + swap for every embcache module.  On the asynchronous
        path nothing here waits for the compute stream, so it is called right after a step has been enqueued."""
        try:
            with record_function("## get_next_batch ##"):
                host_batch = next(it)
        except StopIteration:
            self._exhausted = True
            return None
        with record_function("## copy_batch_to_gpu ##"):
            if self._cuda:
                with torch.cuda.stream(self._copy_stream):
                    batch = host_batch.to(self._device, non_blocking=True)
                    copied = torch.cuda.Event()
                    copied.record()
            else:
                batch, copied = host_batch.to(self._device), None
        feats = self._features_of(batch)
        if self._async:
            host_feats = self._features_of(host_batch)
            with record_function("## start_sparse_data_dist ##"):
                for m in self._mods:
                    m.prefetch_async(feats, host_feats)
        else:
            if copied is not None:
                torch.cuda.current_stream(self._device).wait_event(copied)
                batch.record_stream(torch.cuda.current_stream(self._device))
                copied = None
            for m in self._mods:
                m.prefetch(feats)
        return batch, copied

    def _run_step(self, batch):
        with record_function("## zero_grad ##"):
            (self._zero or self._optimizer.zero_grad)()
        with record_function("## forward ##"):
            loss, out = (self._fwd or self._model)(batch)
        with record_function("## backward ##"):
            (self._bwd(loss) if self._bwd else loss.backward())
            for m in self._mods:
                m.mark_step_done()
            sync = getattr(self._model, "sync_dense_grads", None)
            if sync is not None:
                sync()
        with record_function("## optimizer ##"):
            self._optimizer.step()
        return loss, out

    def attach(self, model: Optional[torch.nn.Module] = None) -> None:
        """(Re-)bind the pipeline to ``model`` (or to the current one) and look its multi-tier modules up again."""
        if model is not None:
            self._model = model
        self._mods = embcache_modules(self._model)
        self._async = self._cuda and all(m._async_ready() for m in self._mods)

    def fill_pipeline(self, dataloader_iter: Iterator) -> None:
        """Stage the first batch (copy, input distribution, swap) without running a step; ``progress`` does this itself
        on its first call."""
        if self._next is None and not self._exhausted:
            self._next = self._fetch(dataloader_iter)

    def wait_pipeline_compute_swapinfo(self) -> None:
        """Bring the staged batch's swap to rest: every pending host update applied, the memcpy stream drained.  Call it
        before a save that happens in the middle of an epoch (while a next batch is staged), as with the reference
        (``distributed/train_pipeline.py:733-735``); the swap plan itself is already complete when ``progress`` returns."""
        for m in self._mods:
            m.drain_host_updates()
            if getattr(m, "_memcpy_stream", None) is not None:
                m._memcpy_stream.synchronize()

    def progress(self, dataloader_iter: Iterator):
        self.fill_pipeline(dataloader_iter)
        if self._next is None:
            raise StopIteration
        batch, copied = self._next
        if self._async:
            if copied is not None:
                with record_function("## wait_for_batch ##"):
                    torch.cuda.current_stream(self._device).wait_event(copied)
                    batch.record_stream(torch.cuda.current_stream(self._device))
            loss, out = self._run_step(batch)                  # batch i is on the GPU's queue ...
            self._next = self._fetch(dataloader_iter) if not self._exhausted else None   # ... the host turns to batch i+1
        else:
            self._next = self._fetch(dataloader_iter) if not self._exhausted else None
            loss, out = self._run_step(batch)
        self._steps += 1
        if self._evict_every and self._steps % self._evict_every == 0:
            for m in self._mods:
                m.host_embedding_evict()
        loss = loss.detach()
        return (loss, out) if self._return_loss else out

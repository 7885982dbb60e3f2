"""Training pipelines.

``TrainPipelineSparseDist.progress(dataloader_iter)`` runs one optimisation step and overlaps it with
the host-to-device copy of the next batch on a dedicated copy stream (pinned host memory ->
``cudaMemcpyAsync``), like the reference's pipelines overlap input distribution and copies with
compute (``hybrid_torchrec/distributed/hybrid_train_pipeline.py:273-335``, ``_copy_to_npu`` ``:450-473``).

With ``cuda_graph=True`` the whole step (input dist, forward, backward with the fused sparse update,
dense gradient all-reduce, dense optimizer) is captured once into a CUDA graph after a few eager
steps and replayed from static input buffers; the step count / learning rate of the dense
optimizer and the barrier epochs live on the device, so replays stay correct.
"""
from __future__ import annotations

from typing import Any, Iterator, Optional, Tuple

import torch
from torch.autograd.profiler import record_function

from ..utils.data import Batch


from ..utils import trace  # noqa: E402


class TrainPipelineBase:
    """No overlap: fetch, copy, step.  Works on CPU as well."""

    def __init__(self, model: torch.nn.Module, optimizer, device: torch.device, return_loss: bool = False,
                 status_poll_steps: int = 16) -> None:
        self._model, self._optimizer, self._device = model, optimizer, device
        self._return_loss = return_loss
        # Kernels report dropped entries (a receive list that was too small) and peer timeouts through a device status
        # word; the pipeline watches it without synchronising and raises (CapacityError / PeerTimeoutError) instead of
        # training on with incomplete gradients.
        from ..ops import _lib

        self._status = _lib.StatusPoller(device, status_poll_steps) if device.type == "cuda" else None

    def _step(self, batch) -> Tuple[torch.Tensor, Any]:
        # profiler ranges carry the reference pipelines' names (hybrid_train_pipeline.py:282-319)
        trace.mark("step.zero_grad")
        with record_function("## zero_grad ##"):
            self._optimizer.zero_grad()
        trace.mark("step.input_dist")
        with record_function("## forward ##"):
            loss, out = self._model(batch)
        trace.mark("dense.backward")
        with record_function("## backward ##"):
            loss.backward()
            sync = getattr(self._model, "sync_dense_grads", None)
            if sync is not None:
                sync()
        trace.mark("step.optimizer")
        with record_function("## optimizer ##"):
            self._optimizer.step()
        trace.mark("step.end")
        # hand back a graph-free loss: a live autograd graph would pin its AccumulateGrad nodes (and
        # the stream they were created on) across steps, which breaks a later CUDA-graph capture
        return loss.detach(), out

    def progress(self, dataloader_iter: Iterator[Batch]):
        batch = next(dataloader_iter).to(self._device)
        loss, out = self._step(batch)
        if self._status is not None:
            self._status.poll()
        return (loss, out) if self._return_loss else out


class TrainPipelineSparseDist(TrainPipelineBase):
    def __init__(self, model: torch.nn.Module, optimizer, device: torch.device, execute_all_batches: bool = True,
                 apply_jit: bool = False, return_loss: bool = False, cuda_graph: bool = False,
                 graph_warmup_steps: int = 3, status_poll_steps: int = 16) -> None:
        super().__init__(model, optimizer, device, return_loss, status_poll_steps)
        self._execute_all_batches = execute_all_batches
        self._cuda = device.type == "cuda"
        self._memcpy_stream = torch.cuda.Stream(device) if self._cuda else None
        self._cur: Optional[Batch] = None
        self._cur_event: Optional[torch.cuda.Event] = None
        self._exhausted = False
        self._use_graph = cuda_graph and self._cuda
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._graph_warmup = graph_warmup_steps
        self._steps_done = 0
        self._static: Optional[Batch] = None
        self._static_out: Any = None
        self.h2d_bytes_last = 0

    # -- copy stage -------------------------------------------------------------
    def _start_copy(self, dataloader_iter: Iterator[Batch]):
        try:
            with record_function("## get_next_batch ##"):
                host = next(dataloader_iter)
        except StopIteration:
            self._exhausted = True
            return None, None
        if not self._cuda:
            return host, None
        with record_function("## copy_batch_to_gpu ##"):
            with torch.cuda.stream(self._memcpy_stream):
                if hasattr(host, "nbytes"):
                    self.h2d_bytes_last = host.nbytes()
                dev = host.to(self._device, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._memcpy_stream)
        return dev, ev

    def _wait_batch(self, batch, ev) -> None:
        if ev is not None:
            with record_function("## wait_for_batch ##"):
                torch.cuda.current_stream(self._device).wait_event(ev)
                batch.record_stream(torch.cuda.current_stream(self._device))

    # -- graph ------------------------------------------------------------------
    def _copy_into_static(self, batch: Batch) -> None:
        s = self._static
        s.dense_features.copy_(batch.dense_features, non_blocking=True)
        s.labels.copy_(batch.labels, non_blocking=True)
        s.sparse_features.values().copy_(batch.sparse_features.values(), non_blocking=True)
        sl, bl = s.sparse_features.lengths_or_none(), batch.sparse_features.lengths_or_none()
        if sl is not None and bl is not None:
            sl.copy_(bl, non_blocking=True)
        so, bo = s.sparse_features.offsets_or_none(), batch.sparse_features.offsets_or_none()
        if so is not None and bo is not None:
            so.copy_(bo, non_blocking=True)

    def _capture(self, batch: Batch) -> None:
        from ..sparse.jagged_tensor import KeyedJaggedTensor

        # Static shapes: graph mode needs the same number of ids every step (one-hot or fixed-length
        # bags).  Offsets are derived from the lengths inside the graph.
        kjt = batch.sparse_features
        has_len = kjt.lengths_or_none() is not None
        skjt = KeyedJaggedTensor(kjt.keys(), kjt.values().clone(),
                                 lengths=kjt.lengths().clone() if has_len else None,
                                 offsets=None if has_len else kjt.offsets().clone(), stride=kjt.stride())
        skjt.one_hot = kjt.one_hot
        self._static = Batch(batch.dense_features.clone(), skjt, batch.labels.clone())
        torch.cuda.synchronize(self._device)
        from ..ops import _lib

        g = torch.cuda.CUDAGraph()
        n0 = _lib.launch_count
        with torch.cuda.graph(g):
            loss, out = self._step(self._static)
        self.launches_per_step = _lib.launch_count - n0   # this library's kernels inside one replay
        self._graph, self._static_out = g, (loss, out)

    def _graph_step(self, batch: Batch):
        if self._graph is None:
            if self._steps_done < self._graph_warmup:
                return self._step(batch)
            self._capture(batch)
        self._copy_into_static(batch)
        self._graph.replay()
        return self._static_out

    # -- public -----------------------------------------------------------------
    def progress(self, dataloader_iter: Iterator[Batch]):
        if self._cur is None and not self._exhausted:
            self._cur, self._cur_event = self._start_copy(dataloader_iter)
        if self._cur is None:
            raise StopIteration
        batch, ev = self._cur, self._cur_event
        self._wait_batch(batch, ev)
        # start the next copy before launching this step's work so the two overlap
        self._cur, self._cur_event = self._start_copy(dataloader_iter)
        with record_function("## forward_backward_step ##"):
            loss, out = self._graph_step(batch) if self._use_graph else self._step(batch)
        self._steps_done += 1
        if self._status is not None:
            self._status.poll()
        return (loss, out) if self._return_loss else out

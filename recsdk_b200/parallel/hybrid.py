"""The "hybrid" flow: id exchange and id mapping on the host (gloo process group, worker thread) several batches
ahead of the device, which only sees ready-to-use lookup inputs.

* ``get_default_hybrid_sharders(host_env)`` -> sharders that put the input distribution of (hash) embedding bag
  collections on ``host_env`` (``hybrid_torchrec/distributed/sharding_plan.py:18-28`` of the reference);
* ``HybridTrainPipelineSparseDist`` keeps up to ``pipe_n_batch`` batches in flight through the stages
  split -> id all-to-all -> id mapping / unique -> host-to-device copy, in order, on one worker thread (so every
  rank issues the host collectives in the same order), while the main thread trains on the oldest ready batch
  (``hybrid_torchrec/distributed/hybrid_train_pipeline.py:191-335`` progress, ``:344-405`` fill, ``:450-473`` copy).
"""
from __future__ import annotations

import queue
import threading
from typing import Any, Callable, Dict, Iterator, List, Optional

import torch

from ..modules.embedding_modules import EmbeddingBagCollection
from ..modules.hash_embeddingbag import HashEmbeddingBagCollection
from .collective_embeddingbag import CollectiveShardedEmbeddingBagCollection
from .comm import ShardingEnv
from .embeddingbag import ParameterSharding
from .train_pipeline import TrainPipelineBase

MAX_PIPE_N_BATCH = 12


class HybridEmbeddingBagCollectionSharder:
    module_type = EmbeddingBagCollection
    hashed = False

    def __init__(self, host_env: Optional[ShardingEnv] = None, fused_params: Optional[dict] = None) -> None:
        if host_env is not None and host_env.process_group is not None:
            import torch.distributed as dist

            if dist.get_backend(host_env.process_group) != "gloo":
                raise ValueError("the host environment must be a gloo process group")
        self.host_env = host_env
        self.fused_params = dict(fused_params or {})

    def sharding_types(self, compute_device_type: str = "cuda") -> List[str]:
        return ["row_wise", "data_parallel"] if self.hashed else ["row_wise", "table_wise", "data_parallel"]

    def handles(self, module, params: Dict[str, ParameterSharding]) -> bool:
        return isinstance(module, HashEmbeddingBagCollection) == self.hashed

    def shard(self, module, params: Dict[str, ParameterSharding], env: ShardingEnv, device=None):
        from .model_parallel import _optimizer_spec_from_params

        sharded = CollectiveShardedEmbeddingBagCollection(
            module.embedding_bag_configs(), params or {}, env, torch.device(device) if device is not None else torch.device("cpu"),
            _optimizer_spec_from_params(module, None), hashed=self.hashed, input_env=self.host_env)
        if not module.is_meta():
            sharded.load_from_unsharded(module)
        return sharded


class HybridHashEmbeddingBagCollectionSharder(HybridEmbeddingBagCollectionSharder):
    module_type = HashEmbeddingBagCollection
    hashed = True


def get_default_hybrid_sharders(host_env: ShardingEnv) -> List[Any]:
    return [HybridHashEmbeddingBagCollectionSharder(host_env), HybridEmbeddingBagCollectionSharder(host_env)]


class HybridTrainPipelineSparseDist(TrainPipelineBase):
    def __init__(self, model: torch.nn.Module, optimizer, device, execute_all_batches: bool = True, apply_jit: bool = False,
                 return_loss: bool = False, pipe_n_batch: int = 6,
                 sparse_features_of: Callable[[Any], Any] = lambda batch: batch.sparse_features) -> None:
        super().__init__(model, optimizer, torch.device(device), return_loss)
        if not (1 <= pipe_n_batch <= MAX_PIPE_N_BATCH):
            raise ValueError("pipe_n_batch must be in [1, %d]" % MAX_PIPE_N_BATCH)
        self._mods = [m for m in model.modules() if isinstance(m, CollectiveShardedEmbeddingBagCollection)]
        self._features_of = sparse_features_of
        self._ready: "queue.Queue" = queue.Queue(maxsize=pipe_n_batch)
        self._worker: Optional[threading.Thread] = None
        self._cuda = self._device.type == "cuda"
        self._copy_stream = torch.cuda.Stream(self._device) if self._cuda else None
        self._execute_all = execute_all_batches

    # worker thread: one batch after the other, so host collectives keep the same order on every rank
    def _produce(self, it: Iterator) -> None:
        try:
            for host_batch in it:
                if self._cuda:
                    torch.cuda.set_device(self._device)
                    with torch.cuda.stream(self._copy_stream):
                        batch = host_batch.to(self._device, non_blocking=True)
                        feats = self._features_of(batch)
                        for m in self._mods:
                            m.prefetch(self._features_of(host_batch) if m.input_pg is not None else feats)
                            if m.input_pg is not None:                      # prepared under the host KJT: re-key to the device one
                                m._prepared[id(feats)] = m._prepared.pop(id(self._features_of(host_batch)))
                        ev = torch.cuda.Event()
                        ev.record(self._copy_stream)
                else:
                    batch, ev = host_batch.to(self._device), None
                    feats = self._features_of(batch)
                    for m in self._mods:
                        m.prefetch(feats)
                self._ready.put((batch, ev))
            self._ready.put(None)
        except BaseException as e:  # noqa: BLE001 - surfaced on the training thread
            self._ready.put(e)

    def progress(self, dataloader_iter: Iterator):
        if self._worker is None:
            self._worker = threading.Thread(target=self._produce, args=(dataloader_iter,), daemon=True)
            self._worker.start()
        item = self._ready.get()
        if item is None:
            self._ready.put(None)
            raise StopIteration
        if isinstance(item, BaseException):
            raise item
        batch, ev = item
        if ev is not None:
            torch.cuda.current_stream(self._device).wait_event(ev)
            batch.record_stream(torch.cuda.current_stream(self._device))
        loss, out = self._step(batch)
        return (loss, out) if self._return_loss else out

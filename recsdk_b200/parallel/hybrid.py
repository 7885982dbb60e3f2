"""The "hybrid" flow: id exchange and id mapping on the host (gloo process group, worker thread) several batches
ahead of the device, which only sees ready-to-use lookup inputs.

* ``get_default_hybrid_sharders(host_env)`` -> sharders that put the input distribution of (hash) embedding bag
  collections on ``host_env`` (``hybrid_torchrec/distributed/sharding_plan.py:18-28`` of the reference);
* ``HybridTrainPipelineSparseDist`` runs ``pipe_n_batch`` pipeline lines; a batch moves through five stages - split
  (bucketize by owner) -> lengths all-to-all (ONE fused exchange per process group for all sharded modules) -> id
  all-to-all -> id mapping / unique -> host-to-device copy - one stage per visit of its line, and the lines take turns,
  so every asynchronous stage (thread-pool future, gloo work handle, copy stream) has ``pipe_n_batch`` training steps
  to finish before anything waits for it.  All ranks issue the host collectives in the same (step-determined) order
  (``hybrid_torchrec/distributed/hybrid_train_pipeline.py:191-335`` progress, ``:344-405`` fill, ``:108-136`` fused
  splits, ``:450-473`` copy).
"""
from __future__ import annotations

import dataclasses
import enum
from collections import deque
from typing import Any, Callable, Deque, Dict, Iterator, List, Optional, Tuple

import torch
from torch.autograd.profiler import record_function

from ..modules.embedding_modules import EmbeddingBagCollection
from ..modules.hash_embeddingbag import HashEmbeddingBagCollection
from .collective_embeddingbag import CollectiveShardedEmbeddingBagCollection, DistState
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

    def shardable_parameters(self, module) -> Dict[str, torch.nn.Parameter]:
        """Table name -> weight of every table of the collection (what a planner may place)."""
        return {c.name: module.embedding_bags[c.name].weight for c in module.embedding_bag_configs()}

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


# names of the reference's sharded modules (``hybrid_torchrec/distributed/embeddingbag.py:93``, ``hash_embeddingbag.py:39``): one
# class serves both here, the hash variant is the same module built with ``hashed=True``
HybridShardedEmbeddingBagCollection = CollectiveShardedEmbeddingBagCollection


class HybridShardedHashEmbeddingBagCollection(CollectiveShardedEmbeddingBagCollection):
    def __init__(self, *args, **kwargs) -> None:
        kwargs["hashed"] = True
        super().__init__(*args, **kwargs)


def get_default_hybrid_sharders(host_env: ShardingEnv) -> List[Any]:
    """The two sharders in the reference's order (``hybrid_torchrec/distributed/sharding_plan.py:18-28``); ``handles`` tells
    the plain and the hash-mapped collection apart, so the order carries no meaning."""
    return [HybridEmbeddingBagCollectionSharder(host_env), HybridHashEmbeddingBagCollectionSharder(host_env)]


class HybridStage(enum.IntEnum):
    """Last stage a batch has entered (``hybrid_train_pipeline.py:58-63`` of the reference names the same five)."""
    SPLIT = 0
    FIRST_ALL2ALL = 1
    SECOND_ALL2ALL = 2
    POST_INPUT = 3
    COPY_TO_DEVICE = 4


@dataclasses.dataclass
class HybridPipelineContext:
    index: int
    host_batch: Any = None
    batch: Any = None                                   # device batch once the copy stage has been issued
    stage: int = int(HybridStage.SPLIT)
    states: List[DistState] = dataclasses.field(default_factory=list)
    # per process group: (work handle or None, received lengths [W, sum F*B], [(state, first column, columns)])
    fused_splits: List[Tuple[Any, torch.Tensor, List[Tuple[DistState, int, int]]]] = dataclasses.field(default_factory=list)
    copy_event: Any = None


def _staged(m: CollectiveShardedEmbeddingBagCollection) -> bool:
    """Host tensors can go through this module's exchange group (a gloo group, or a single rank)."""
    if m.world == 1 or m.input_pg is not None:
        return True
    import torch.distributed as dist

    return m.pg is not None and dist.get_backend(m.pg) == "gloo"


class HybridTrainPipelineSparseDist(TrainPipelineBase):
    def __init__(self, model: torch.nn.Module, optimizer, device, execute_all_batches: bool = True, apply_jit: bool = False,
                 return_loss: bool = False, pipe_n_batch: int = 6,
                 sparse_features_of: Callable[[Any], Any] = lambda batch: batch.sparse_features) -> None:
        self.param_check(model, torch.device(device), pipe_n_batch, apply_jit, execute_all_batches)
        super().__init__(model, optimizer, torch.device(device), return_loss)
        self._mods = [m for m in model.modules() if isinstance(m, CollectiveShardedEmbeddingBagCollection)]
        self._features_of = sparse_features_of
        self._n = pipe_n_batch
        self._lines: List[Deque[HybridPipelineContext]] = [deque() for _ in range(pipe_n_batch)]
        self._line = 0
        self._filled = False
        self._n_read = 0
        self._cuda = self._device.type == "cuda"
        self._memcpy_stream = torch.cuda.Stream(self._device) if self._cuda else None
        self.stage_log: List[Tuple[int, int, str]] = []      # (training step, batch index, stage) when tracing is on
        self.trace_stages = False
        self._step_no = 0

    def param_check(self, model: torch.nn.Module, device: torch.device, pipe_n_batch, apply_jit, execute_all_batches) -> None:
        """Argument checks of the constructor (``hybrid_train_pipeline.py:240-268`` of the reference; the device may be any
        ``torch.device`` here, CPU included, since the pipeline also runs on the gloo / CPU path)."""
        if not isinstance(pipe_n_batch, int) or isinstance(pipe_n_batch, bool):
            raise ValueError("pipe_n_batch must be an int but got %s" % type(pipe_n_batch).__name__)
        if not (1 <= pipe_n_batch <= MAX_PIPE_N_BATCH):
            raise ValueError("pipe_n_batch must be in [1, %d]" % MAX_PIPE_N_BATCH)
        if not isinstance(model, torch.nn.Module):
            raise TypeError("model must be a torch.nn.Module, got %s" % type(model).__name__)
        if not isinstance(device, torch.device):
            raise TypeError("device must be a torch.device, got %s" % type(device).__name__)
        if apply_jit:
            raise ValueError("apply_jit is not supported")
        if not execute_all_batches:
            raise ValueError("execute_all_batches cannot be False: batches already in the lines have had their ids exchanged")

    def enque_context(self, line_id: int, context: HybridPipelineContext) -> None:
        """Append a batch context to pipeline line ``line_id`` (``hybrid_train_pipeline.py:270-271`` of the reference)."""
        self._lines[line_id % self._n].append(context)

    # ------------------------------------------------------------------ stages
    def _log(self, ctx: HybridPipelineContext, stage: HybridStage) -> None:
        ctx.stage = int(stage)
        if self.trace_stages:
            self.stage_log.append((self._step_no, ctx.index, stage.name))

    def _start_split(self, it: Iterator) -> HybridPipelineContext:
        with record_function("## get_next_batch ##"):
            ctx = HybridPipelineContext(index=self._n_read, host_batch=next(it, None))
        self._n_read += 1
        if ctx.host_batch is not None:
            with record_function("## start_sparse_data_dist ##"):
                feats = self._features_of(ctx.host_batch)
                ctx.states = [m.stage_split(feats) for m in self._mods if _staged(m)]
        self._log(ctx, HybridStage.SPLIT)
        return ctx

    def _first_all2all(self, ctx: HybridPipelineContext) -> None:
        """Lengths of all modules that share a process group travel in one all-to-all."""
        if ctx.host_batch is not None:
            import torch.distributed as dist

            by_pg: Dict[int, List[DistState]] = {}
            pgs: Dict[int, Any] = {}
            for st in ctx.states:
                m = st.module
                pg = m.input_pg if m.input_pg is not None else m.pg
                by_pg.setdefault(id(pg), []).append(st)
                pgs[id(pg)] = pg
            for key, sts in by_pg.items():
                parts = [st.module.stage_send_lengths(st) for st in sts]
                send = parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)
                send = send.contiguous()
                cols, c0 = [], 0
                for st, p in zip(sts, parts):
                    cols.append((st, c0, p.shape[1]))
                    c0 += p.shape[1]
                if sts[0].module.world == 1:
                    ctx.fused_splits.append((None, send, cols))
                else:
                    recv = torch.empty_like(send)
                    work = dist.all_to_all_single(recv, send, group=pgs[key], async_op=True)
                    ctx.fused_splits.append((work, recv, cols))
        self._log(ctx, HybridStage.FIRST_ALL2ALL)

    def _second_all2all(self, ctx: HybridPipelineContext) -> None:
        with record_function("## wait_sparse_data_dist ##"):
            for work, recv, cols in ctx.fused_splits:
                if work is not None:
                    work.wait()
                for st, c0, n in cols:
                    st.module.stage_exchange_ids(st, recv[:, c0:c0 + n].contiguous())
        ctx.fused_splits = []
        self._log(ctx, HybridStage.SECOND_ALL2ALL)

    def _post_input(self, ctx: HybridPipelineContext) -> None:
        with record_function("## _post_input_dist ##"):
            for st in ctx.states:
                st.module.stage_post_input(st)
        self._log(ctx, HybridStage.POST_INPUT)

    def _copy_to_device(self, ctx: HybridPipelineContext) -> None:
        if ctx.host_batch is not None and ctx.batch is None:
            assert ctx.stage == int(HybridStage.POST_INPUT), "copy stage reached before the id mapping stage"
            with record_function("## copy_batch_to_gpu ##"):
                self._copy_batch(ctx)
        self._log(ctx, HybridStage.COPY_TO_DEVICE)

    def _copy_batch(self, ctx: HybridPipelineContext) -> None:
        if self._cuda:
            torch.cuda.set_device(self._device)
            with torch.cuda.stream(self._memcpy_stream):
                ctx.batch = ctx.host_batch.to(self._device, non_blocking=True)
                ctx.copy_event = torch.cuda.Event()
                ctx.copy_event.record(self._memcpy_stream)
        else:
            ctx.batch = ctx.host_batch.to(self._device)
        feats = self._features_of(ctx.batch)
        for st in ctx.states:
            st.module.stage_to_device(st, feats, self._memcpy_stream)
        staged = {id(st.module) for st in ctx.states}
        for m in self._mods:                           # device-group modules: their own prefetch on the device batch
            if id(m) not in staged:
                m.prefetch(feats)
        ctx.states = []

    _ADVANCE = {int(HybridStage.SPLIT): "_first_all2all", int(HybridStage.FIRST_ALL2ALL): "_second_all2all",
                int(HybridStage.SECOND_ALL2ALL): "_post_input"}

    def _advance_line(self, line: Deque[HybridPipelineContext]) -> None:
        for ctx in line:                                   # oldest first: collectives keep batch order
            fn = self._ADVANCE.get(ctx.stage)
            if fn is not None:
                getattr(self, fn)(ctx)

    def _fill(self, it: Iterator) -> None:
        """Four rounds over the lines: afterwards every line holds batches at stages POST_INPUT .. SPLIT."""
        for _ in range(int(HybridStage.COPY_TO_DEVICE)):
            for line in self._lines:
                self._advance_line(line)
                line.append(self._start_split(it))
        self._copy_to_device(self._lines[0][0])
        self._filled = True

    # ------------------------------------------------------------------ one training step
    def progress(self, dataloader_iter: Iterator):
        if not self._filled:
            self._fill(dataloader_iter)
        line = self._lines[self._line % self._n]
        nxt = self._lines[(self._line + 1) % self._n]
        head = line[0]
        if head.host_batch is None:
            raise StopIteration
        line.popleft()
        if head.copy_event is not None:
            with record_function("## wait_for_batch ##"):
                cur = torch.cuda.current_stream(self._device)
                cur.wait_event(head.copy_event)
                head.batch.record_stream(cur)
        # the batch the next step trains on starts its copy now, so that it overlaps this step's compute
        if self._n > 1:
            self._copy_to_device(nxt[0])
        loss, out = self._step(head.batch)
        self._advance_line(line)
        line.append(self._start_split(dataloader_iter))
        if self._n == 1:                                   # single line: its new head is next step's batch
            self._copy_to_device(line[0])
        self._line += 1
        self._step_no += 1
        if self._status is not None:
            self._status.poll()
        return (loss, out) if self._return_loss else out

    def in_flight(self) -> int:
        """Batches read from the dataloader and not trained on yet."""
        return sum(1 for line in self._lines for c in line if c.host_batch is not None)


# the reference's names for the stage enumeration and the per-batch context (``hybrid_train_pipeline.py:58-70``, ``:73-120``)
TaskType = HybridStage
HybridTrainPipelineContext = HybridPipelineContext

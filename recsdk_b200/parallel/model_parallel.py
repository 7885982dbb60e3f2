"""``DistributedModelParallel``: shards embedding collections according to a plan and data-parallelises
everything else.

* Unsharded ``EmbeddingBagCollection`` children are replaced by ``ShardedEmbeddingBagCollection``
  (fused peer-memory backend on CUDA) built from the plan entries of that module path.
* Dense parameters that live in flat buffers (``FusedMLP``, ``LogitHead``) get their gradient buffers
  re-homed into ONE peer-mapped allocation; ``sync_dense_grads()`` averages it across ranks with the
  in-kernel all-reduce (multimem through NVSwitch when a multicast mapping exists).  Remaining dense
  parameters fall back to ``torch.distributed.all_reduce``.
* ``fused_optimizer`` is the ``CombinedOptimizer`` of the sparse in-backward optimizers (no-op ``step``).

Mirrors the role of TorchRec's DMP in the reference's user flow
(``docs/en/torch/torch_rec_v1/03_quick_start/quick_start.md:239-262``).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..modules.embedding_modules import EmbeddingBagCollection
from ..modules.hash_embeddingbag import HashEmbeddingBagCollection
from ..ops import embedding_ops as E
from ..optim import CombinedOptimizer
from ..utils import trace
from .comm import PeerGroup, ShardingEnv
from .collective_embeddingbag import CollectiveShardedEmbeddingBagCollection
from .embeddingbag import ParameterSharding, ShardedEmbeddingBagCollection
from .planner import ShardingPlan


def _optimizer_spec_from_params(ebc: nn.Module, default: Optional[E.OptimizerSpec]) -> E.OptimizerSpec:
    """Translate ``apply_optimizer_in_backward`` annotations into a fused sparse optimizer spec."""
    for p in ebc.parameters():
        classes = getattr(p, "_optimizer_classes", None)
        if classes:
            cls, kw = classes[0], dict(getattr(p, "_optimizer_kwargs", [{}])[0])
            acc = int(kw.pop("accumulate_step", 1)) if kw.pop("use_accumulate", False) else 1
            spec = _spec_of(cls, kw)
            if spec is not None:
                spec.accumulate_step = max(acc, 1)
                return spec
    return default or E.OptimizerSpec()


def _spec_of(cls, kw) -> Optional[E.OptimizerSpec]:
    """Optimizer class + keyword arguments -> fused sparse optimizer spec (None for classes the fused update lacks)."""
    if issubclass(cls, torch.optim.Adagrad):
        kind = E.OPT_ROWWISE_ADAGRAD if kw.get("rowwise", True) else E.OPT_ADAGRAD
        return E.OptimizerSpec(kind=kind, lr=kw.get("lr", 0.01), eps=kw.get("eps", 1e-10),
                               weight_decay=kw.get("weight_decay", 0.0),
                               initial_accumulator_value=kw.get("initial_accumulator_value", 0.0))
    if issubclass(cls, torch.optim.Adam):
        b = kw.get("betas", (0.9, 0.999))
        return E.OptimizerSpec(kind=E.OPT_ADAM, lr=kw.get("lr", 1e-3), eps=kw.get("eps", 1e-8), beta1=b[0],
                               beta2=b[1], weight_decay=kw.get("weight_decay", 0.0))
    if issubclass(cls, torch.optim.SGD):
        return E.OptimizerSpec(kind=E.OPT_SGD, lr=kw.get("lr", 0.01), weight_decay=kw.get("weight_decay", 0.0))
    return None


class DistributedModelParallel(nn.Module):
    def __init__(self, module: nn.Module, env: Optional[ShardingEnv] = None, device: Optional[torch.device] = None,
                 plan: Optional[ShardingPlan] = None, sharders=None, peer: Optional[PeerGroup] = None,
                 sparse_optimizer: Optional[E.OptimizerSpec] = None, out_dtype: torch.dtype = torch.bfloat16,
                 max_local_batch: int = 0, one_hot: bool = False, init_seed: Optional[int] = None,
                 backend: Optional[str] = None, overlap_grad_reduce: bool = True) -> None:
        """``backend``: ``"fused"`` (peer-memory kernels; CUDA only, the default there) or ``"collective"``
        (``torch.distributed`` all-to-all flow; any device, the default on CPU; required for hash tables)."""
        super().__init__()
        dev0 = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                          else torch.device("cpu"))
        self.backend = backend or ("fused" if torch.device(dev0).type == "cuda" else "collective")
        self.env = env or ShardingEnv.from_process_group(None)
        self.device = torch.device(dev0)
        self.world, self.rank = self.env.world_size, self.env.rank
        self.peer = peer
        if self.world > 1 and self.device.type == "cuda" and peer is None:
            self.peer = PeerGroup(self.env.process_group, self.device)
        self.plan = plan or ShardingPlan({})
        self.sharders = list(sharders or [])
        self.sharded_modules: List[nn.Module] = []
        self._shard(module, "", sparse_optimizer, out_dtype, max_local_batch, one_hot, init_seed)
        self.module = module
        for m in module.modules():
            if isinstance(m, (ShardedEmbeddingBagCollection, CollectiveShardedEmbeddingBagCollection)) \
                    and m not in self.sharded_modules:
                self.sharded_modules.append(m)
        self._sharded_param_ids = {id(p) for sm in self.sharded_modules for p in sm.parameters()}
        self.overlap_grad_reduce = overlap_grad_reduce
        self._build_grad_reducer()
        self._broadcast_dense()

    # ------------------------------------------------------------------ sharding
    def _shard(self, parent: nn.Module, prefix: str, spec, out_dtype, max_local_batch, one_hot, init_seed) -> None:
        for name, child in list(parent.named_children()):
            path = prefix + name
            custom = self._custom_shard(child, path)
            if custom is not None:
                setattr(parent, name, custom)
                self.sharded_modules.append(custom)
                continue
            if isinstance(child, EmbeddingBagCollection):
                entries: Dict[str, ParameterSharding] = self.plan.get_module_plan(path)
                hashed = isinstance(child, HashEmbeddingBagCollection)
                if hashed or self.backend == "collective":
                    sharded = CollectiveShardedEmbeddingBagCollection(
                        child.embedding_bag_configs(), entries, self.env, self.device,
                        _optimizer_spec_from_params(child, spec), hashed=hashed,
                        out_dtype=out_dtype if self.device.type == "cuda" else torch.float32)
                    if not child.is_meta():
                        sharded.load_from_unsharded(child)
                    setattr(parent, name, sharded)
                    self.sharded_modules.append(sharded)
                    continue
                fspec = _optimizer_spec_from_params(child, spec)
                if fspec.accumulate_step > 1:
                    raise NotImplementedError("gradient accumulation over several steps runs on the collective backend "
                                              "(backend=\"collective\")")
                from .grouped_embeddingbag import GroupedShardedEmbeddingBagCollection, needs_grouping

                # tables of one collection that differ in storage dtype or pooling: one fused collection per group
                cls = GroupedShardedEmbeddingBagCollection if needs_grouping(child.embedding_bag_configs()) \
                    else ShardedEmbeddingBagCollection
                sharded = cls(
                    child.embedding_bag_configs(), entries, self.env, self.device,
                    fspec, peer=self.peer, out_dtype=out_dtype,
                    max_local_batch=max_local_batch, one_hot=one_hot, init_weights=True)
                if init_seed is not None:
                    sharded.reset_parameters(seed=init_seed)
                elif not child.is_meta():
                    sharded.load_from_unsharded(child)
                setattr(parent, name, sharded)
                self.sharded_modules.append(sharded)
            elif isinstance(child, (ShardedEmbeddingBagCollection, CollectiveShardedEmbeddingBagCollection)):
                continue
            else:
                self._shard(child, path + ".", spec, out_dtype, max_local_batch, one_hot, init_seed)

    def _custom_shard(self, child: nn.Module, path: str) -> Optional[nn.Module]:
        """User-supplied sharders (objects with ``module_type`` and ``shard(module, params, env, device)``; an optional
        ``handles(module, params)`` narrows the match) take precedence over the built-in table sharding."""
        for s in self.sharders:
            mt = getattr(s, "module_type", None)
            if mt is None or not isinstance(child, mt):
                continue
            params = self.plan.get_module_plan(path)
            if hasattr(s, "handles") and not s.handles(child, params):
                continue
            return s.shard(child, params, self.env, self.device)
        return None

    # ------------------------------------------------------------- dense grads
    def _build_grad_reducer(self) -> None:
        """Dense gradients are summed over the data-parallel ranks by the bucketed push all-reduce; each flat module's
        bucket starts on a side stream at the end of that module's backward (``overlap_grad_reduce``)."""
        self._reducer = None
        if self.world == 1 or self.device.type != "cuda" or self.peer is None:
            return
        from .grad_reduce import DenseGradReducer

        wire = torch.float32 if os.environ.get("RECSDK_B200_ALLREDUCE_WIRE", "bf16") == "fp32" else torch.bfloat16
        self._reducer = DenseGradReducer(self.peer, self.module, exclude_param_ids=self._sharded_param_ids,
                                         wire_dtype=wire, overlap=self.overlap_grad_reduce, average=False)

    @torch.no_grad()
    def _broadcast_dense(self) -> None:
        if self.world == 1 or self.env.process_group is None:
            return
        for p in self.module.parameters():
            if id(p) in self._sharded_param_ids:
                continue
            dist.broadcast(p.data, src=0, group=self.env.process_group)
        for m in self.module.modules():
            if hasattr(m, "sync_shadow"):
                m.sync_shadow()

    def sync_dense_grads(self) -> None:
        """Average dense gradients over the data-parallel ranks (call between backward and step)."""
        if self.world == 1:
            return
        for m in self.sharded_modules:
            if hasattr(m, "join_exchange"):
                m.join_exchange()
        if self._reducer is not None:
            self._reducer.sync()
            return
        trace.mark("dense.grad_allreduce")
        for p in self.module.parameters():
            if p.grad is not None and id(p) not in self._sharded_param_ids:
                dist.all_reduce(p.grad, group=self.env.process_group)

    # ------------------------------------------------------------------- misc
    @property
    def fused_optimizer(self) -> CombinedOptimizer:
        return CombinedOptimizer([m.fused_optimizer for m in self.sharded_modules if hasattr(m, "fused_optimizer")])

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def dense_named_parameters(self) -> Dict[str, nn.Parameter]:
        return {n: p for n, p in self.module.named_parameters()
                if id(p) not in self._sharded_param_ids and p.requires_grad}

"""Planner and sharders that turn stock ``EmbeddingCollection`` / ``EmbeddingBagCollection`` tables into dynamic
(hash-table backed) ones.

A table becomes dynamic when its constraint says ``use_dynamicemb=True``; such tables are always row-wise
(``key % world_size``, "round robin"), their per-rank capacity is aligned up to a power of two of at least one
bucket, and the planner reserves ``bytes(dim + optimizer state) * capacity`` of device memory per rank for them
before placing the remaining (static) tables.  Reference: ``dynamic_emb/distributed/planner/types.py:30-75``,
``planners.py:63-77`` (alignment), ``:80-222`` (planner), ``:224-290`` (plan rewriting),
``distributed/embedding.py:58-120`` / ``embeddingbag.py:80-119`` (sharders).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import torch
from torch import nn

from ..modules.embedding_configs import BaseEmbeddingConfig
from ..modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from ..parallel.comm import ShardingEnv
from ..parallel.embeddingbag import ParameterSharding
from ..parallel.planner import EmbeddingShardingPlanner, ParameterConstraints, ShardingPlan, Topology
from .dynamicemb_config import DynamicEmbTableOptions, aligned_capacity_per_rank
from .embedding import DynamicEmbeddingBagCollection, DynamicEmbeddingCollection
from .hkv import OptimizerType

DYNAMICEMB_KERNEL = "DynamicEmb"


@dataclasses.dataclass
class DynamicEmbParameterConstraints(ParameterConstraints):
    use_dynamicemb: bool = False
    dynamicemb_options: Optional[DynamicEmbTableOptions] = None

    def __post_init__(self) -> None:
        if self.use_dynamicemb:
            if self.sharding_types not in (None, ["row_wise"]):
                raise ValueError("dynamic tables are row_wise only")
            if self.compute_kernels not in (None, ["fused"], [DYNAMICEMB_KERNEL]):
                raise ValueError("dynamic tables use the fused compute kernel")
            self.sharding_types = ["row_wise"]
            if self.dynamicemb_options is None:
                self.dynamicemb_options = DynamicEmbTableOptions()


@dataclasses.dataclass
class DynamicEmbParameterSharding(ParameterSharding):
    customized_compute_kernel: str = DYNAMICEMB_KERNEL
    dist_type: str = "roundrobin"
    dynamicemb_options: Optional[DynamicEmbTableOptions] = None
    aligned_rows_per_rank: int = 0
    hbm_bytes_per_rank: int = 0

    def get_additional_fused_params(self) -> dict:
        """The fields this class adds to ``ParameterSharding`` (handed to the compute kernel as fused parameters)."""
        base = {f.name for f in dataclasses.fields(ParameterSharding)}
        return {f.name: getattr(self, f.name) for f in dataclasses.fields(self) if f.name not in base}


_OPT_STATE_ELEMS = {OptimizerType.SGD: lambda d: 0, OptimizerType.ADAGRAD: lambda d: d, OptimizerType.ADAM: lambda d: 2 * d,
                    OptimizerType.ROWWISE_ADAGRAD: lambda d: 4}


@dataclasses.dataclass
class ShardingOption:
    """One placement a table may take: what the planner chooses between."""
    name: str
    module_path: str
    sharding_type: str
    compute_kernel: str
    rows: int
    dim: int
    is_dynamic: bool
    rows_per_rank: int
    hbm_bytes_per_rank: int


class DynamicEmbeddingEnumerator:
    """Lists the placements open to every table of a model: a dynamic table has exactly one (row-wise, round robin, the
    ``DynamicEmb`` kernel, capacity aligned up to a power of two); a static table one per sharding type that its sharder and
    its constraint allow.  ``DynamicEmbeddingShardingPlanner(..., enumerator=...)`` takes the optimizer-state size from the
    options listed here.  Reference: ``dynamic_emb/distributed/planner/enumerators.py:92-230``."""

    def __init__(self, topology: Topology, batch_size: Optional[int] = 512, constraints: Optional[Dict[str, ParameterConstraints]] = None,
                 estimator=None, use_exact_enumerate_order: Optional[bool] = False) -> None:
        if not isinstance(topology, Topology):
            raise TypeError("topology must be a Topology")
        if batch_size is not None and (not isinstance(batch_size, int) or isinstance(batch_size, bool) or batch_size < 1):
            raise ValueError("batch_size must be a positive int")
        if constraints is not None and not isinstance(constraints, dict):
            raise TypeError("constraints must be a dict")
        self.topology, self.batch_size = topology, batch_size
        self.constraints = dict(constraints or {})
        self.estimator = estimator
        self.use_exact_enumerate_order = bool(use_exact_enumerate_order)
        self.optimizer_type = OptimizerType.ROWWISE_ADAGRAD

    def _options_of(self, path: str, cfg: BaseEmbeddingConfig, allowed: List[str]) -> List[ShardingOption]:
        W = self.topology.world_size
        cons = self.constraints.get(cfg.name)
        item = {"FP32": 4, "FP16": 2, "BF16": 2}[cfg.data_type.value]
        if cons is not None and getattr(cons, "use_dynamicemb", False):
            o = cons.dynamicemb_options
            rows = aligned_capacity_per_rank(cfg.num_embeddings, W, o.bucket_capacity)
            elems = cfg.embedding_dim + _OPT_STATE_ELEMS[self.optimizer_type](cfg.embedding_dim)
            return [ShardingOption(cfg.name, path, "row_wise", DYNAMICEMB_KERNEL, cfg.num_embeddings, cfg.embedding_dim, True, rows,
                                   rows * elems * 4)]
        types = [t for t in (cons.sharding_types if cons is not None and cons.sharding_types else allowed) if t in allowed]
        out = []
        for t in types:
            per = {"row_wise": (cfg.num_embeddings + W - 1) // W, "table_wise": cfg.num_embeddings,
                   "data_parallel": cfg.num_embeddings}.get(t)
            if per is None:
                continue
            out.append(ShardingOption(cfg.name, path, t, "fused", cfg.num_embeddings, cfg.embedding_dim, False, per,
                                      per * (cfg.embedding_dim * item + 4)))
        return out

    def enumerate(self, module: nn.Module, sharders=None) -> List[ShardingOption]:
        """Every (table, placement) pair, in module order (``use_exact_enumerate_order``) or sorted by module path."""
        found = []
        for path, m in module.named_modules():
            if isinstance(m, EmbeddingBagCollection):
                cfgs = m.embedding_bag_configs()
            elif isinstance(m, EmbeddingCollection):
                cfgs = m.embedding_configs()
            else:
                continue
            allowed = ["row_wise", "table_wise", "data_parallel"]
            for s in sharders or []:
                mt = getattr(s, "module_type", None)
                if mt is not None and isinstance(m, mt) and hasattr(s, "sharding_types"):
                    allowed = list(s.sharding_types(self.topology.compute_device))
                    break
            found.append((path, [o for c in cfgs for o in self._options_of(path, c, allowed)]))
        if not self.use_exact_enumerate_order:
            found.sort(key=lambda x: x[0])
        return [o for _p, opts in found for o in opts]


class DynamicEmbeddingShardingPlanner:
    def __init__(self, eb_configs: List[BaseEmbeddingConfig], constraints: Optional[Dict[str, ParameterConstraints]] = None,
                 topology: Optional[Topology] = None, batch_size: Optional[int] = None, enumerator=None, storage_reservation=None,
                 proposer=None, partitioner=None, performance_model=None, stats=None, debug: bool = True,
                 optimizer_type: OptimizerType = OptimizerType.ROWWISE_ADAGRAD) -> None:
        self.eb_configs = {c.name: c for c in eb_configs}
        self.constraints = dict(constraints or {})
        self.topology = topology or Topology()
        self.optimizer_type = optimizer_type
        self.debug = debug
        self.enumerator = enumerator
        if enumerator is not None and hasattr(enumerator, "optimizer_type"):
            enumerator.optimizer_type = optimizer_type                 # both must size the optimizer state the same way
            if not enumerator.constraints:
                enumerator.constraints = dict(self.constraints)
        static = {k: v for k, v in self.constraints.items() if not getattr(v, "use_dynamicemb", False)}
        self._dynamic = {k: v for k, v in self.constraints.items() if getattr(v, "use_dynamicemb", False)}
        reserved = 0
        self._dyn_plan: Dict[str, DynamicEmbParameterSharding] = {}
        for name, cons in self._dynamic.items():
            cfg = self.eb_configs.get(name)
            if cfg is None:
                raise KeyError("constraint for unknown table %r" % name)
            o = cons.dynamicemb_options
            rows = aligned_capacity_per_rank(cfg.num_embeddings, self.topology.world_size, o.bucket_capacity)
            row_elems = cfg.embedding_dim + _OPT_STATE_ELEMS[self.optimizer_type](cfg.embedding_dim)
            need = rows * row_elems * 4
            hbm = need if not o.global_hbm_for_values else min(need, o.global_hbm_for_values // self.topology.world_size)
            reserved += hbm
            self._dyn_plan[name] = DynamicEmbParameterSharding("row_wise", compute_kernel="fused", row_partition="mod",
                                                               dynamicemb_options=o, aligned_rows_per_rank=rows,
                                                               hbm_bytes_per_rank=int(hbm))
        if reserved > self.topology.hbm_cap:
            raise RuntimeError("dynamic tables need %.1f GB per GPU, budget %.1f GB" % (reserved / 2 ** 30, self.topology.hbm_cap / 2 ** 30))
        topo = dataclasses.replace(self.topology, hbm_cap=self.topology.hbm_cap - reserved)
        self._static_planner = EmbeddingShardingPlanner(topo, static, batch_size)
        self.reserved_hbm_per_rank = reserved

    def plan(self, module: nn.Module, sharders=None) -> ShardingPlan:
        plan: Dict[str, Dict[str, ParameterSharding]] = {}
        for path, m in module.named_modules():
            cfgs = None
            if isinstance(m, EmbeddingBagCollection):
                cfgs = m.embedding_bag_configs()
            elif isinstance(m, EmbeddingCollection):
                cfgs = m.embedding_configs()
            if cfgs is None:
                continue
            stat = [c for c in cfgs if c.name not in self._dyn_plan]
            entries = dict(self._static_planner._plan_tables(stat)) if stat else {}
            for c in cfgs:
                if c.name in self._dyn_plan:
                    entries[c.name] = self._dyn_plan[c.name]
            plan[path] = entries
        return ShardingPlan(plan)

    def collective_plan(self, module: nn.Module, sharders=None, pg=None) -> ShardingPlan:
        return self.plan(module, sharders)          # deterministic on every rank: nothing to exchange


class _DynamicSharderBase:
    module_type = None
    target = None

    def __init__(self, fused_params: Optional[dict] = None, qcomm_codecs_registry=None, use_index_dedup: bool = False) -> None:
        self.fused_params = dict(fused_params or {})
        self.use_index_dedup = use_index_dedup

    def sharding_types(self, compute_device_type: str = "cuda") -> List[str]:
        return ["row_wise"]

    def compute_kernels(self, sharding_type: str = "row_wise", compute_device_type: str = "cuda") -> List[str]:
        return [DYNAMICEMB_KERNEL]

    def handles(self, module: nn.Module, params: Dict[str, ParameterSharding]) -> bool:
        return isinstance(module, self.module_type) and any(isinstance(p, DynamicEmbParameterSharding) for p in params.values())

    def shard(self, module: nn.Module, params: Dict[str, ParameterSharding], env: ShardingEnv, device=None):
        cfgs = module.embedding_bag_configs() if hasattr(module, "embedding_bag_configs") else module.embedding_configs()
        missing = [c.name for c in cfgs if not isinstance(params.get(c.name), DynamicEmbParameterSharding)]
        if missing:
            raise NotImplementedError("tables %s share a collection with dynamic tables but are not dynamic" % missing)
        options = {c.name: params[c.name].dynamicemb_options for c in cfgs}
        fp = self.fused_params
        return self.target(cfgs, options, env, device, optimizer_type=fp.get("optimizer", OptimizerType.ROWWISE_ADAGRAD),
                           learning_rate=fp.get("learning_rate", fp.get("lr", 0.01)), eps=fp.get("eps", 1e-8),
                           betas=(fp.get("beta1", 0.9), fp.get("beta2", 0.999)), weight_decay=fp.get("weight_decay", 0.0),
                           use_index_dedup=self.use_index_dedup,
                           output_dtype=fp.get("output_dtype", torch.float32))


class DynamicEmbeddingCollectionSharder(_DynamicSharderBase):
    module_type = EmbeddingCollection
    target = DynamicEmbeddingCollection


class DynamicEmbeddingBagCollectionSharder(_DynamicSharderBase):
    module_type = EmbeddingBagCollection
    target = DynamicEmbeddingBagCollection

    def __init__(self, fused_params: Optional[dict] = None, qcomm_codecs_registry=None) -> None:
        super().__init__(fused_params, qcomm_codecs_registry, False)

"""Sharding planner: decides, per embedding table, table-wise / row-wise / data-parallel placement
under the per-GPU HBM budget (B200: 180 GB, planner default 160 GB usable).

API shape follows the TorchRec planner the reference drives
(``EmbeddingShardingPlanner(topology, constraints).collective_plan(model, sharders, pg)``;
``dynamic_emb/distributed/planner/planners.py:80-222``); the device model constants replace the
reference's patched ones (``torchrec1.2.0_npu.patch:411-415``: HBM 64 GB, 897 GB/s).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import torch.distributed as dist
from torch import nn

from .embeddingbag import ParameterSharding

HBM_CAP_BYTES = 160 * 1024 ** 3          # usable of 180 GB HBM3e
HBM_BW_BYTES = 6.5e12                    # measured copy bandwidth
NVLINK_BW_BYTES = 770e9                  # measured peer bandwidth per direction
DDR_CAP_BYTES = 512 * 1024 ** 3


@dataclasses.dataclass
class Topology:
    world_size: int = 1
    compute_device: str = "cuda"
    hbm_cap: int = HBM_CAP_BYTES
    ddr_cap: int = DDR_CAP_BYTES
    local_world_size: Optional[int] = None
    intra_host_bw: float = NVLINK_BW_BYTES
    hbm_mem_bw: float = HBM_BW_BYTES


@dataclasses.dataclass
class ParameterConstraints:
    sharding_types: Optional[List[str]] = None
    compute_kernels: Optional[List[str]] = None
    min_partition: Optional[int] = None
    pooling_factors: Optional[List[float]] = None
    row_partition: Optional[str] = None


class ShardingPlan:
    """``plan[module_path][table_name] -> ParameterSharding``."""

    def __init__(self, plan: Dict[str, Dict[str, ParameterSharding]]) -> None:
        self.plan = plan

    def get_module_plan(self, path: str) -> Dict[str, ParameterSharding]:
        if path in self.plan:
            return self.plan[path]
        if len(self.plan) == 1 and "" in self.plan:
            return self.plan[""]
        return {}

    def __repr__(self) -> str:
        rows = []
        for path, tabs in self.plan.items():
            for t, ps in tabs.items():
                rows.append("%s.%s: %s%s" % (path, t, ps.sharding_type, "" if not ps.ranks else " @%s" % ps.ranks))
        return "ShardingPlan(\n  " + "\n  ".join(rows) + "\n)"


def _table_bytes(cfg, opt_elems_per_row: int = 1) -> int:
    item = {"FP32": 4, "FP16": 2, "BF16": 2}[cfg.data_type.value]
    return cfg.num_embeddings * (cfg.embedding_dim * item + 4 * opt_elems_per_row)


class EmbeddingShardingPlanner:
    """Greedy planner.

    * tables whose constraint names a sharding type get it;
    * otherwise tables larger than ``row_wise_threshold_bytes`` (default: 1/8 of a GPU's budget or
      more than a fair share) are row-wise, tiny tables (< ``dp_threshold_bytes``) data-parallel when
      allowed, and the rest table-wise, dealt out so that every rank owns the same number of them
      (lookup / update work is per id, not per row) in snake order of size (bytes stay even too).
    """

    def __init__(self, topology: Optional[Topology] = None, constraints: Optional[Dict[str, ParameterConstraints]] = None,
                 batch_size: Optional[int] = None, row_wise_threshold_bytes: Optional[int] = None,
                 dp_threshold_bytes: int = 0) -> None:
        self.topology = topology or Topology()
        self.constraints = constraints or {}
        self.batch_size = batch_size
        self.rw_threshold = row_wise_threshold_bytes
        self.dp_threshold = dp_threshold_bytes

    def _plan_tables(self, cfgs) -> Dict[str, ParameterSharding]:
        W = self.topology.world_size
        out: Dict[str, ParameterSharding] = {}
        if W == 1:
            return {c.name: ParameterSharding("data_parallel") for c in cfgs}
        total = sum(_table_bytes(c) for c in cfgs)
        fair = total / W
        rw_thr = self.rw_threshold if self.rw_threshold is not None else min(self.topology.hbm_cap // 8, max(fair / 2, 1))
        load = [0.0] * W
        tw: List = []
        for c in cfgs:
            cons = self.constraints.get(c.name)
            st = cons.sharding_types[0] if cons and cons.sharding_types else None
            nb = _table_bytes(c)
            if st is None:
                if nb >= rw_thr:
                    st = "row_wise"
                elif nb <= self.dp_threshold:
                    st = "data_parallel"
                else:
                    st = "table_wise"
            if st == "row_wise":
                out[c.name] = ParameterSharding("row_wise", row_partition=(cons.row_partition if cons and cons.row_partition else "mod"))
                for r in range(W):
                    load[r] += nb / W
            elif st == "data_parallel":
                out[c.name] = ParameterSharding("data_parallel")
                for r in range(W):
                    load[r] += nb
            elif st == "table_wise":
                tw.append((nb, c))
            else:
                raise NotImplementedError("sharding type %r" % st)
        # Table-wise tables concentrate a whole feature's lookups and updates on their owner.  With the pull design a
        # row-wise table costs no extra traffic, so only as many tables stay table-wise as can be dealt out evenly
        # (the same number per rank); the largest left-overs become row-wise.  Dealing in snake order over the size
        # ranking also evens out the bytes.
        tw.sort(key=lambda x: -x[0])
        extra = len(tw) % W
        for nb, c in tw[:extra]:
            out[c.name] = ParameterSharding("row_wise", row_partition="mod")
            for r in range(W):
                load[r] += nb / W
        for i, (nb, c) in enumerate(tw[extra:]):
            rnd, pos = divmod(i, W)
            r = pos if rnd % 2 == 0 else W - 1 - pos
            load[r] += nb
            out[c.name] = ParameterSharding("table_wise", ranks=[r])
        if max(load) > self.topology.hbm_cap:
            raise RuntimeError("plan needs %.1f GB on one GPU, budget %.1f GB" % (max(load) / 2 ** 30, self.topology.hbm_cap / 2 ** 30))
        return out

    def plan(self, module: nn.Module, sharders=None) -> ShardingPlan:
        from ..modules.embedding_modules import EmbeddingBagCollection

        plan: Dict[str, Dict[str, ParameterSharding]] = {}
        for path, m in module.named_modules():
            if isinstance(m, EmbeddingBagCollection):
                plan[path] = self._plan_tables(m.embedding_bag_configs())
        return ShardingPlan(plan)

    def collective_plan(self, module: nn.Module, sharders=None, pg: Optional["dist.ProcessGroup"] = None) -> ShardingPlan:
        """Every rank computes the same deterministic plan; rank 0's is broadcast for safety."""
        plan = self.plan(module, sharders)
        if pg is not None or (dist.is_available() and dist.is_initialized()):
            obj = [plan.plan]
            dist.broadcast_object_list(obj, src=0, group=pg)
            plan = ShardingPlan(obj[0])
        return plan

"""Sharded checkpoints of the static embedding collections, reloadable at another world size.

Every rank writes the rows it holds together with their GLOBAL row ids and a sharding record per table
(``ShardMetadata``: global shape, sharding type, row partition, the writer's rank and world size), i.e. the information a
``ShardedTensor`` carries in the reference flow (``hybrid_torchrec/distributed/embeddingbag.py:695-789`` registers
state-dict hooks that wrap each local shard with its offsets).  A reader rebuilds its own shard from whichever files hold
its rows, so a model saved on 8 GPUs resumes on 2, on 1, or with another sharding plan.

    save_sharded(module, directory)                 # every rank; rank 0 also writes meta.json
    load_sharded(module, directory)                 # every rank, any world size / plan

Works for ``ShardedEmbeddingBagCollection`` (fused backend: flat weight buffer, row-wise optimizer state) and
``CollectiveShardedEmbeddingBagCollection`` (one tensor per table).
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Dict, List

import torch
from torch import nn

from ..ops import embedding_ops as E

_KIND_NAME = {E.SH_LOCAL: "data_parallel", E.SH_TABLE_WISE: "table_wise", E.SH_ROW_MOD: "row_wise", E.SH_ROW_BLOCK: "row_wise"}


@dataclasses.dataclass
class ShardMetadata:
    table: str
    global_rows: int
    dim: int
    sharding_type: str            # data_parallel | table_wise | row_wise
    row_partition: str            # mod | block | none
    rank: int
    world_size: int
    local_rows: int

    def to_json(self) -> Dict[str, object]:
        return dataclasses.asdict(self)


def _kinds(module: nn.Module) -> List[int]:
    return list(getattr(module, "_kinds", None) or getattr(module, "kinds"))


def _state_tensors(module: nn.Module, ti: int, n_rows: int, dim: int) -> Dict[str, torch.Tensor]:
    """Optimizer state of table ``ti`` as ``[local_rows, k]`` tensors (views where possible)."""
    out: Dict[str, torch.Tensor] = {}
    if hasattr(module, "state") and isinstance(module.state, list):          # collective backend: dict per table
        for k, v in module.state[ti].items():
            out[k] = v.view(n_rows, -1) if v.numel() else v.reshape(0, 1)
        return out
    s_off = int(module.s_offsets[ti]) if getattr(module, "s_offsets", None) is not None else 0
    for name in ("state1", "state2"):
        st = getattr(module, name, None)
        if st is None:
            continue
        per_row = 1 if module.opt.kind == E.OPT_ROWWISE_ADAGRAD else dim
        out[name] = st[s_off:s_off + n_rows * per_row].view(n_rows, per_row)
    return out


def sharded_state_dict(module: nn.Module) -> Dict[str, object]:
    """This rank's shard of every table: rows, their global ids, optimizer state and the sharding record."""
    kinds = _kinds(module)
    out: Dict[str, object] = {"tables": {}, "step": int(getattr(module, "_step", 0))}
    for ti, t in enumerate(module.tables):
        w = module.embedding_bags[t.name].weight.detach()
        rows = module.global_rows_of(ti).cpu()
        k = kinds[ti]
        meta = ShardMetadata(t.name, int(t.num_embeddings), int(t.embedding_dim), _KIND_NAME[k],
                             "mod" if k == E.SH_ROW_MOD else ("block" if k == E.SH_ROW_BLOCK else "none"),
                             int(module.rank), int(module.world), int(w.shape[0]))
        entry = {"metadata": meta.to_json(), "global_row_ids": rows, "weight": w.cpu().clone()}
        for name, st in _state_tensors(module, ti, int(w.shape[0]), int(t.embedding_dim)).items():
            entry[name] = st.detach().cpu().clone()
        out["tables"][t.name] = entry
    return out


def save_sharded(module: nn.Module, directory: str) -> str:
    os.makedirs(directory, exist_ok=True)
    sd = sharded_state_dict(module)
    path = os.path.join(directory, "shard_rank%d_of%d.pt" % (module.rank, module.world))
    torch.save(sd, path)
    if module.rank == 0:
        meta = {"world_size": int(module.world), "tables": {n: e["metadata"] for n, e in sd["tables"].items()},
                "format": "recsdk_b200 sharded embedding checkpoint v1"}
        with open(os.path.join(directory, "meta.json"), "w") as f:
            json.dump(meta, f, indent=1)
    return path


def load_sharded_from(module: nn.Module, shards: List[Dict[str, object]], strict: bool = True) -> Dict[str, int]:
    """Fill this rank's shard from the state dicts of ALL ranks of the saving job (any world size, any plan).
    -> rows restored per table.  Data-parallel / table-wise writers hold whole tables; only one copy is read."""
    restored: Dict[str, int] = {}
    for ti, t in enumerate(module.tables):
        w = module.embedding_bags[t.name].weight
        mine = module.global_rows_of(ti).cpu()
        n_local = int(w.shape[0])
        if n_local == 0:
            restored[t.name] = 0
            continue
        # global row -> position in this rank's shard
        pos = torch.full((int(t.num_embeddings),), -1, dtype=torch.int64)
        pos[mine] = torch.arange(n_local, dtype=torch.int64)
        states = _state_tensors(module, ti, n_local, int(t.embedding_dim))
        filled = torch.zeros(n_local, dtype=torch.bool)
        for sd in shards:
            entry = sd["tables"].get(t.name)
            if entry is None:
                continue
            md = entry["metadata"]
            if int(md["global_rows"]) != int(t.num_embeddings) or int(md["dim"]) != int(t.embedding_dim):
                raise ValueError("table %s: checkpoint shape [%d, %d] differs from the model's [%d, %d]"
                                 % (t.name, md["global_rows"], md["dim"], t.num_embeddings, t.embedding_dim))
            gids = entry["global_row_ids"]
            if gids.numel() == 0:
                continue
            dst = pos[gids]
            take = (dst >= 0) & ~filled[dst.clamp(min=0)]
            if not bool(take.any()):
                continue
            d = dst[take]
            with torch.no_grad():
                w[d.to(w.device)] = entry["weight"][take].to(w.device, w.dtype)
                for name, st in states.items():
                    if name in entry and st.numel():
                        src = entry[name][take].to(st.device, st.dtype)
                        if src.shape[1:] == st.shape[1:]:
                            st[d.to(st.device)] = src
            filled[d] = True
        restored[t.name] = int(filled.sum())
        if strict and not bool(filled.all()):
            raise ValueError("table %s: %d of %d local rows are in no shard of the checkpoint"
                             % (t.name, n_local - restored[t.name], n_local))
    if shards and hasattr(module, "_step"):
        module._step = max(int(sd.get("step", 0)) for sd in shards)
    return restored


def load_sharded(module: nn.Module, directory: str, strict: bool = True) -> Dict[str, int]:
    """Read every ``shard_rank*_of*.pt`` of ``directory`` (written by any world size) and keep this rank's rows."""
    meta_path = os.path.join(directory, "meta.json")
    if not os.path.exists(meta_path):
        raise FileNotFoundError("%s has no meta.json: not a finished sharded checkpoint" % directory)
    with open(meta_path) as f:
        world = int(json.load(f)["world_size"])
    shards = []
    for r in range(world):
        p = os.path.join(directory, "shard_rank%d_of%d.pt" % (r, world))
        if not os.path.exists(p):
            raise FileNotFoundError("missing shard file %s" % p)
        shards.append(torch.load(p, map_location="cpu", weights_only=False))
    return load_sharded_from(module, shards, strict)

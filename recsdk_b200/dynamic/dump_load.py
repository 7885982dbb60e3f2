"""``DynamicEmbDump`` / ``DynamicEmbLoad`` / ``set_score`` / ``get_score`` / ``incremental_dump`` over every
dynamic collection of a model (``dynamic_emb/distributed/dump_load.py:39-272``,
``incremental_dump.py:103-404``).  Files: ``<path>/<module path>/<table>_emb_{keys,values,scores,opt_values}
.rank_<r>.world_size_<w>`` (raw little-endian int64 / fp32) plus ``<table>_opt_args.json`` written by rank 0."""
from __future__ import annotations

import os
import shutil
from typing import Dict, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import nn

from .embedding import _ShardedDynamicBase


def find_dynamic_modules(model: nn.Module) -> Dict[str, _ShardedDynamicBase]:
    return {path: m for path, m in model.named_modules() if isinstance(m, _ShardedDynamicBase)}


def find_sharded_modules(module: nn.Module, path: str = "") -> List[Tuple[str, str, nn.Module]]:
    """(path, name, module) of every sharded dynamic collection, paths rooted at ``"model"`` as in the reference's dump
    layout (``dynamic_emb/distributed/dump_load.py:39-55``)."""
    if not isinstance(module, nn.Module):
        raise ValueError("param `module` must be an instance of torch.nn.Module, but got:%s" % type(module))
    root = path + "model"
    out = []
    for p, m in module.named_modules():
        if isinstance(m, _ShardedDynamicBase):
            out.append((root + ("." + p if p else ""), p.rsplit(".", 1)[-1] if p else "model", m))
    return out


def get_dynamic_emb_module(model: nn.Module) -> List[nn.Module]:
    """The batched table modules (``BatchedDynamicEmbeddingTablesV2``) below ``model`` (``dump_load.py:84-89``)."""
    if not isinstance(model, nn.Module):
        raise ValueError("param `model` must be an instance of torch.nn.Module, but got:%s" % type(model))
    from .batched_dynamicemb_table import BatchedDynamicEmbeddingTablesV2

    return [m for m in model.modules() if isinstance(m, BatchedDynamicEmbeddingTablesV2)]


def check_emb_collection_modules(module: nn.Module, ret_list: List[nn.Module]) -> None:
    ret_list.extend(get_dynamic_emb_module(module))


def _barrier(pg) -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier(group=pg)


def DynamicEmbDump(path: str, model: nn.Module, table_names: Optional[Dict[str, List[str]]] = None, optim: bool = False,
                   pg=None, allow_overwrite: bool = False) -> None:
    mods = find_dynamic_modules(model)
    rank = dist.get_rank(pg) if dist.is_initialized() else 0
    if rank == 0:
        if os.path.exists(path) and os.listdir(path):
            if not allow_overwrite:
                raise FileExistsError("%s exists and is not empty (pass allow_overwrite=True)" % path)
            shutil.rmtree(path)
        os.makedirs(path, exist_ok=True)
    _barrier(pg)
    for mpath, m in mods.items():
        names = None if table_names is None else table_names.get(mpath)
        m.dump(os.path.join(path, mpath or "root"), optim, names)
    _barrier(pg)


def DynamicEmbLoad(path: str, model: nn.Module, table_names: Optional[Dict[str, List[str]]] = None, optim: bool = False,
                   pg=None) -> Dict[str, Dict[str, int]]:
    out = {}
    for mpath, m in find_dynamic_modules(model).items():
        d = os.path.join(path, mpath or "root")
        if not os.path.isdir(d):
            raise FileNotFoundError("no checkpoint directory for module %r under %s" % (mpath, path))
        out[mpath] = m.load(d, optim, None if table_names is None else table_names.get(mpath))
    _barrier(pg)
    return out


def set_score(model: nn.Module, table_score: Union[int, Dict[str, Dict[str, int]]]) -> None:
    for mpath, m in find_dynamic_modules(model).items():
        if isinstance(table_score, int):
            m.lookup.set_score({n: table_score for n in m.lookup.table_names})
        elif mpath in table_score:
            m.lookup.set_score(table_score[mpath])


def get_score(model: nn.Module) -> Dict[str, Dict[str, int]]:
    return {mpath: m.lookup.get_score() for mpath, m in find_dynamic_modules(model).items()}


def incremental_dump(model: nn.Module, score_threshold: Union[int, Dict[str, Dict[str, int]]], pg=None
                     ) -> Tuple[Dict[str, Dict[str, Tuple[torch.Tensor, torch.Tensor]]], Dict[str, Dict[str, int]]]:
    """Entries whose score is >= the threshold, gathered over all ranks, as host tensors; also returns the
    current scores to pass as the next call's threshold."""
    result, scores = {}, {}
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(pg) > 1
    for mpath, m in find_dynamic_modules(model).items():
        thr = score_threshold if isinstance(score_threshold, int) else score_threshold.get(mpath, {})
        local, cur = m.lookup.incremental_dump(thr if isinstance(thr, dict) else
                                               {n: int(thr) for n in m.lookup.table_names})
        if multi:
            merged = {}
            for name, (k, v) in local.items():
                parts = [None] * dist.get_world_size(pg)
                dist.all_gather_object(parts, (k, v), group=pg)
                merged[name] = (torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts]))
            local = merged
        result[mpath], scores[mpath] = local, cur
    return result, scores

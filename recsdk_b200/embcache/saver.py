"""Checkpointing of multi-tier tables: every rank flushes its device cache to the host table and writes its
keys / embeddings / optimizer state / filter state under ``<dir>/<table>/rank<r>/``; after a barrier rank 0
merges the rank directories into one file set per table and writes ``meta.ini``; loading re-shards by
``key % world_size`` so the world size may change between save and load.  Incremental saves hold only the keys
touched since the previous save.  Reference: ``torchrec_embcache/saver.py:31-171``; file layout
``csrc/embedding_cache/embcache_manager.cpp:549-618`` (save), ``:620-800`` (merge), ``:905-981`` (load).
"""
from __future__ import annotations

import os
import shutil
from datetime import datetime, timezone
from typing import List, Optional

import torch
import torch.distributed as dist

from .train_pipeline import embcache_modules

META = "meta.ini"
TIMESTAMP_FORMAT = "%Y%m%d%H%M%S"          # name of a checkpoint directory in the reference's flow (``saver.py:24``)


def _read_meta(path: str) -> dict:
    out = {}
    with open(path) as f:
        for line in f:
            if "=" in line:
                k, v = line.strip().split("=", 1)
                out[k.strip()] = v.strip()
    return out


class Saver:
    def __init__(self, process_group=None) -> None:
        self.pg = process_group

    def _world(self):
        if dist.is_available() and dist.is_initialized():
            return dist.get_world_size(self.pg), dist.get_rank(self.pg)
        return 1, 0

    def _barrier(self) -> None:
        if dist.is_available() and dist.is_initialized():
            dist.barrier(group=self.pg)

    def save(self, module: torch.nn.Module, path: str, incremental: bool = False) -> str:
        world, rank = self._world()
        mods = embcache_modules(module)
        if not mods:
            raise ValueError("module holds no embcache tables")
        step = max(m.swap_step for m in mods)
        # Two ways to name a checkpoint.  The reference's: the caller passes the checkpoint directory itself, named by a UTC
        # timestamp (``Saver.timestamp_dir_name()``), and finds the newest one with ``get_latest_load_path(parent)``.  This
        # package's: the caller passes the parent and the directory is named after the kind and the training step.
        if Saver.is_timestamp_format(os.path.basename(os.path.normpath(path))):
            out = path
        else:
            out = os.path.join(path, "%s_%010d" % ("incremental" if incremental else "full", step))
        if rank == 0:
            os.makedirs(out, exist_ok=True)
        self._barrier()
        for m in mods:
            m.embedding_to_host()
            m.manager.save(out, rank, incremental)
        self._barrier()
        if rank == 0:
            tables: List[str] = []
            for m in mods:
                m.manager.merge_files(out, world)
                for t in m.full_tables:
                    tables.append(t.name)
                    for r in range(world):
                        shutil.rmtree(os.path.join(out, t.name, "rank%d" % r), ignore_errors=True)
            with open(os.path.join(out, META), "w") as f:            # plain ``key=value`` lines, as the reference writes them
                f.write("incremental=%s\nsave_world_size=%d\nstep=%d\ntables=%s\n" % (incremental, world, step, ",".join(tables)))
        self._barrier()
        return out

    def load(self, module: torch.nn.Module, path: str, incremental: bool = False) -> None:
        world, rank = self._world()
        if not os.path.exists(os.path.join(path, META)):
            raise FileNotFoundError("%s has no %s: not a finished checkpoint" % (path, META))
        meta = _read_meta(os.path.join(path, META))
        if (meta.get("incremental", "False") == "True") != incremental:
            raise ValueError("checkpoint kind (full / incremental) does not match the request")
        for m in embcache_modules(module):
            if not incremental:
                m.invalidate_device_cache()
            else:
                m.embedding_to_host()
                m.invalidate_device_cache()
            m.manager.load(path, rank, world, incremental)
        self._barrier()

    @staticmethod
    def is_timestamp_format(dir_name: str) -> bool:
        """True for names like ``20250131235959`` (UTC, ``%Y%m%d%H%M%S``)."""
        try:
            datetime.strptime(dir_name, TIMESTAMP_FORMAT)
            return len(dir_name) == 14
        except (ValueError, TypeError):
            return False

    @staticmethod
    def timestamp_dir_name() -> str:
        return datetime.now(tz=timezone.utc).strftime(TIMESTAMP_FORMAT)

    @staticmethod
    def get_latest_load_path(path: str, incremental: Optional[bool] = None) -> Optional[str]:
        """Newest finished checkpoint under ``path`` (None when there is none): the highest training step, and among
        timestamp-named directories of equal step - or written without a step, as the reference writes them - the latest name."""
        best, best_key = None, None
        if not os.path.isdir(path):
            return None
        for d in sorted(os.listdir(path)):
            full = os.path.join(path, d)
            if not os.path.exists(os.path.join(full, META)):
                continue
            meta = _read_meta(os.path.join(full, META))
            if incremental is not None and (meta.get("incremental", "False") == "True") != incremental:
                continue
            key = (int(meta.get("step", "-1")), d if Saver.is_timestamp_format(d) else "")
            if best_key is None or key > best_key:
                best, best_key = full, key
        return best

"""Rank / device mapping from the launcher's environment or a rank-table JSON file.
Reference: ``training/common/python/communication/hccl/hccl_info.py:40-111``, ``hccl_mgmt.py:26-150`` (there the
table maps ranks to Ascend devices; here to CUDA devices of one or more hosts)."""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Dict, List, Optional


@dataclasses.dataclass
class RankInfo:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    local_world_size: int = 1
    device_id: int = 0
    host: str = "127.0.0.1"

    @property
    def node_rank(self) -> int:
        return self.rank // max(self.local_world_size, 1)


def rank_info_from_env(env: Optional[Dict[str, str]] = None) -> RankInfo:
    e = os.environ if env is None else env
    world = int(e.get("WORLD_SIZE", "1"))
    rank = int(e.get("RANK", "0"))
    lws = int(e.get("LOCAL_WORLD_SIZE", str(world)))
    lr = int(e.get("LOCAL_RANK", str(rank % max(lws, 1))))
    vis = e.get("CUDA_VISIBLE_DEVICES")
    dev = lr
    if vis:
        ids = [x for x in vis.split(",") if x != ""]
        if lr >= len(ids):
            raise ValueError("LOCAL_RANK %d has no device in CUDA_VISIBLE_DEVICES=%s" % (lr, vis))
    if not (0 <= rank < world):
        raise ValueError("RANK %d outside WORLD_SIZE %d" % (rank, world))
    return RankInfo(rank, world, lr, lws, dev, e.get("MASTER_ADDR", "127.0.0.1"))


def rank_info_from_table(path: str, rank: int) -> RankInfo:
    """Rank table: ``{"server_list": [{"server_id": host, "device": [{"device_id": "0", "rank_id": "0"}, ...]}, ...]}``."""
    with open(path) as f:
        table = json.load(f)
    entries: List[tuple] = []
    for srv in table.get("server_list", []):
        devs = srv.get("device", [])
        for d in devs:
            entries.append((int(d["rank_id"]), int(d["device_id"]), srv.get("server_id", "127.0.0.1"), len(devs)))
    entries.sort()
    ranks = [r for r, *_ in entries]
    if ranks != list(range(len(ranks))):
        raise ValueError("rank table must list ranks 0..N-1 exactly once")
    for r, dev, host, lws in entries:
        if r == rank:
            first = min(rr for rr, _d, h, _l in entries if h == host)
            return RankInfo(rank, len(entries), rank - first, lws, dev, host)
    raise KeyError("rank %d not in the rank table" % rank)


# ----------------------------------------------------------------------------------------------------------------------
# Getter functions under the reference's names (``communication/hccl/hccl_info.py:40-111``, ``hccl_mgmt.py``).  The launcher's
# variables are read in this order: torchrun's (``RANK`` / ``WORLD_SIZE`` / ``LOCAL_WORLD_SIZE``), then Open MPI's.
# ----------------------------------------------------------------------------------------------------------------------
def _env_int(names, what: str, at_least: int) -> int:
    for n in names:
        v = os.environ.get(n)
        if v is not None:
            if not v.strip().lstrip("+").isdigit():
                raise ValueError("the value should be number, but got the value: %s" % v)
            if int(v) < at_least:
                raise ValueError("the value must be greater than or equal to %d, but got %s" % (at_least, v))
            return int(v)
    raise RuntimeError("Environment variable %s has not been exported, please launch with torchrun or mpirun first" % what)


def get_rank_id() -> int:
    return _env_int(("RANK", "OMPI_COMM_WORLD_RANK"), "RANK", 0)


def get_rank_size() -> int:
    return _env_int(("WORLD_SIZE", "OMPI_COMM_WORLD_SIZE"), "WORLD_SIZE", 1)


def get_local_rank_size() -> int:
    return _env_int(("LOCAL_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_SIZE"), "LOCAL_WORLD_SIZE", 1)


def get_rank_to_device_dict() -> Dict[int, int]:
    """rank -> device id: from the rank table named by ``RANK_TABLE_FILE`` when set, else local rank ``i`` -> the ``i``-th
    entry of ``CUDA_VISIBLE_DEVICES`` (or ``i`` itself)."""
    path = os.environ.get("RANK_TABLE_FILE", "")
    if path:
        with open(path) as f:
            table = json.load(f)
        out: Dict[int, int] = {}
        for srv in table.get("server_list", []):
            for d in srv.get("device", []):
                if not str(d.get("rank_id", "")).isdigit():
                    raise ValueError("rank table: rank_id wrong")
                out[int(d["rank_id"])] = int(d["device_id"])
        if not out:
            raise ValueError("rank table holds no device")
        return out
    n = get_local_rank_size()
    vis = [x for x in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if x.strip().isdigit()]
    return {i: (int(vis[i]) if i < len(vis) else i) for i in range(n)}


def get_device_id() -> int:
    d = get_rank_to_device_dict()
    dev = d.get(get_rank_id() % get_local_rank_size() if not os.environ.get("RANK_TABLE_FILE") else get_rank_id())
    if dev is None:
        raise RuntimeError("no device is assigned to rank %d" % get_rank_id())
    return int(dev)


def get_min_device_id() -> int:
    return min(get_rank_to_device_dict().values())


def get_device_list() -> List[int]:
    """Device ids of this job on this host, in rank order."""
    d = get_rank_to_device_dict()
    return [d[r] for r in sorted(d)]

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

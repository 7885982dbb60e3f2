"""Host-side liveness of the ranks of a job, checked between steps.

Every rank writes a heartbeat (step number and wall-clock time) to the job's key-value store after each step and a
"left" mark when it stops on purpose.  Before launching the next step's kernels a rank calls ``check_peers``: a peer
that announced its departure, or whose heartbeat is older than ``stale_after_s``, raises ``PeerLostError`` on the
host - before any collective or peer-memory kernel that would wait for it is in flight.  Device-side waits are
bounded as well (status word), this check just turns a lost peer into a clean error one step earlier.
The reference has no rank-failure detection (its LCCL waits spin without a limit:
``cust_op/ascendc_op/ai_core_op/lccl/v220/op_kernel/sync_collectives.h:66,101``).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional


class PeerLostError(RuntimeError):
    def __init__(self, ranks: List[int], reason: str) -> None:
        super().__init__("ranks %s %s" % (ranks, reason))
        self.ranks, self.reason = ranks, reason


class Heartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "recsdk_hb", stale_after_s: float = 60.0) -> None:
        self.store, self.rank, self.world, self.prefix, self.stale_after_s = store, rank, world, prefix, stale_after_s

    def _key(self, kind: str, r: int) -> str:
        return "%s/%s/%d" % (self.prefix, kind, r)

    def beat(self, step: int) -> None:
        self.store.set(self._key("beat", self.rank), "%d:%.3f" % (step, time.time()))

    def leave(self) -> None:
        """Announce an orderly departure (call between steps, with none of this rank's kernels or collectives in flight)."""
        self.store.set(self._key("left", self.rank), "1")

    def _get(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:  # noqa: BLE001 - a store without the key
            return None

    def peers(self) -> Dict[int, Dict[str, float]]:
        out = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            b = self._get(self._key("beat", r))
            step, when = (int(b.split(":")[0]), float(b.split(":")[1])) if b else (-1, 0.0)
            out[r] = {"step": step, "age_s": time.time() - when if b else float("inf"), "left": self._get(self._key("left", r)) is not None}
        return out

    def check_peers(self, require_beat: bool = False) -> None:
        info = self.peers()
        left = [r for r, i in info.items() if i["left"]]
        if left:
            raise PeerLostError(left, "left the job")
        stale = [r for r, i in info.items() if (i["step"] >= 0 or require_beat) and i["age_s"] > self.stale_after_s]
        if stale:
            raise PeerLostError(stale, "have not reported for more than %.0f s" % self.stale_after_s)

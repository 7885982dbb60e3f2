"""Failure detection without touching a GPU: gloo ranks, failures made on the host.
(a) a rank leaves between steps: the others learn of it from the store before their next collective;
(b) a rank stops reporting: its heartbeat goes stale;
(c) a rank that never joins a collective: the short process-group timeout ends it with an error."""
import datetime
import os
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from recsdk_b200.parallel.health import Heartbeat, PeerLostError


def _worker(rank, world, d, scenario, ret):
    store = dist.FileStore(os.path.join(d, "store"), world)
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    hb = Heartbeat(store, rank, world, stale_after_s=1.0)
    try:
        x = torch.ones(4)
        dist.all_reduce(x)                                   # step 0 works
        hb.beat(0)
        if scenario == "leave":
            if rank == 1:
                hb.leave()                                   # orderly exit between steps, nothing in flight
                return
            time.sleep(0.5)
            try:
                hb.check_peers()
                dist.all_reduce(x)                           # must not be reached
                ret[rank] = "not detected"
            except PeerLostError as e:
                ret[rank] = "lost %s" % e.ranks
        elif scenario == "stale":
            if rank == 1:
                time.sleep(2.5)                              # stops reporting (a stuck host thread), then goes away
                return
            time.sleep(1.8)
            try:
                hb.check_peers()
                ret[rank] = "not detected"
            except PeerLostError as e:
                ret[rank] = "stale %s" % e.ranks
        else:                                                # "timeout": rank 1 never joins the second collective
            if rank == 1:
                time.sleep(6.0)
                return
            t0 = time.time()
            try:
                dist.all_reduce(x)
                ret[rank] = "no error"
            except Exception as e:  # noqa: BLE001 - gloo reports the timeout as a RuntimeError
                ret[rank] = "error after %.0f s" % (time.time() - t0)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


@pytest.mark.parametrize("scenario,expect", [("leave", "lost [1]"), ("stale", "stale [1]"), ("timeout", "error after")])
def test_lost_rank_is_detected_on_the_host(scenario, expect):
    with tempfile.TemporaryDirectory() as d:
        ret = mp.Manager().dict()
        ctx = mp.spawn(_worker, args=(2, d, scenario, ret), nprocs=2, join=False)
        deadline = time.time() + 60
        while not ctx.join(timeout=1.0):
            assert time.time() < deadline, "workers did not finish"
        assert str(ret.get(0, "")).startswith(expect), dict(ret)

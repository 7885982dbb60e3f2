"""CPU affinity helpers: pin the calling process (and the threads it spawns afterwards) to the cores that sit next
to its GPU, so host-side input processing does not migrate across NUMA nodes.
Reference: ``training/common/python/perf_factory/bind_cpu.py:13-107`` (decorator style)."""
from __future__ import annotations

import functools
import os
from typing import Callable, List, Optional, Sequence


def cores_for_rank(local_rank: int, local_world_size: int, cores: Optional[Sequence[int]] = None, reserve: int = 0) -> List[int]:
    """Even contiguous split of the usable cores among the local ranks; ``reserve`` cores per rank are left out
    (for the framework's own IO threads)."""
    usable = sorted(cores) if cores is not None else sorted(os.sched_getaffinity(0))
    if local_world_size <= 0 or not (0 <= local_rank < local_world_size):
        raise ValueError("bad local rank / world size")
    per = max(1, len(usable) // local_world_size)
    mine = usable[local_rank * per:(local_rank + 1) * per] or usable[-1:]
    return mine[reserve:] if len(mine) > reserve else mine


def bind_current_process(cores: Sequence[int]) -> List[int]:
    os.sched_setaffinity(0, set(cores))
    return sorted(os.sched_getaffinity(0))


def bind_cpu(local_rank: Optional[int] = None, local_world_size: Optional[int] = None, reserve: int = 0) -> Callable:
    """Decorator: run the function with the process pinned to its rank's cores (taken from ``LOCAL_RANK`` /
    ``LOCAL_WORLD_SIZE`` when not given); the previous affinity is restored afterwards."""
    def deco(fn: Callable) -> Callable:
        @functools.wraps(fn)
        def wrapped(*a, **kw):
            lr = int(os.environ.get("LOCAL_RANK", "0")) if local_rank is None else local_rank
            lws = int(os.environ.get("LOCAL_WORLD_SIZE", "1")) if local_world_size is None else local_world_size
            before = os.sched_getaffinity(0)
            try:
                bind_current_process(cores_for_rank(lr, lws, sorted(before), reserve))
                return fn(*a, **kw)
            finally:
                os.sched_setaffinity(0, before)
        return wrapped
    return deco


def bind_rank_from_env(min_cores: int = 2) -> Optional[List[int]]:
    """Pin this process to its rank's share of the cores (``LOCAL_RANK`` / ``LOCAL_WORLD_SIZE``) when there are several
    local ranks and every rank would get at least ``min_cores``.  Opt-in: ``RECSDK_B200_BIND_CPU=1`` (on the 2-GPU HSTU
    training benchmark it made no measurable difference, so it is off by default).
    Returns the cores bound to, or None when nothing was changed."""
    if os.environ.get("RECSDK_B200_BIND_CPU", "0") != "1":
        return None
    lws = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    if lws <= 1:
        return None
    usable = sorted(os.sched_getaffinity(0))
    if len(usable) // lws < min_cores:
        return None
    return bind_current_process(cores_for_rank(lr, lws, usable))


def get_available_cpu_num_and_range():
    """-> (number of usable cores, [(first, last) core of every physical package that holds usable cores]); the package of a
    core is read from sysfs, all cores count as one package when that is not available
    (``perf_factory/bind_cpu.py:13-56`` of the reference)."""
    usable = sorted(os.sched_getaffinity(0))
    groups = {}
    for c in usable:
        try:
            with open("/sys/devices/system/cpu/cpu%d/topology/physical_package_id" % c) as f:
                pkg = int(f.read().strip())
        except (OSError, ValueError):
            pkg = 0
        groups.setdefault(pkg, []).append(c)
    return len(usable), [(min(v), max(v)) for _k, v in sorted(groups.items())]


def bind_cpu_task() -> Optional[List[int]]:
    """Bind the calling process to its local rank's share of the usable cores (``LOCAL_RANK`` / ``LOCAL_WORLD_SIZE`` or the
    Open MPI equivalents); nothing happens for a single local rank.  -> the cores bound to, or None."""
    lws = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("OMPI_COMM_WORLD_LOCAL_SIZE", "1")))
    lr = int(os.environ.get("LOCAL_RANK", os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", "0")))
    if lws <= 1 or not (0 <= lr < lws):
        return None
    return bind_current_process(cores_for_rank(lr, lws))

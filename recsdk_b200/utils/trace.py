"""Lightweight phase tracing with CUDA events.

``RECSDK_B200_TRACE=1`` turns it on.  Code calls ``mark("name")`` at phase boundaries on the current stream;
``report()`` synchronises once and returns, per phase name, the mean device time from that mark to the next one
(so the time is attributed to the phase that *starts* at the mark).  Marks are a no-op when tracing is off and
are skipped during CUDA-graph capture.  ``torch.profiler.record_function`` ranges with the same names are
emitted as well, so the phases show up in a Kineto trace when one is taken.
The reference exposes timing through ``TimeCost`` logs on the host (``torchrec_embcache/csrc/utils``) and
``record_function`` ranges in its pipelines (``hybrid_train_pipeline.py:450-473``).
"""
from __future__ import annotations

import collections
import os
from typing import Dict, List, Tuple

import torch

ENABLED = os.environ.get("RECSDK_B200_TRACE", "0") == "1"
_marks: List[Tuple[str, "torch.cuda.Event"]] = []


def enable(on: bool = True) -> None:
    global ENABLED
    ENABLED = on


def mark(name: str) -> None:
    if not ENABLED or not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing():
        return
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    _marks.append((name, ev))


def reset() -> None:
    _marks.clear()


def report(reset_after: bool = True) -> Dict[str, Dict[str, float]]:
    """-> {phase: {"mean_us", "count", "total_ms"}}; the span of the last mark of the list is dropped."""
    if not _marks:
        return {}
    torch.cuda.synchronize()
    agg = collections.OrderedDict()
    for (name, ev), (_n2, ev2) in zip(_marks[:-1], _marks[1:]):
        ms = ev.elapsed_time(ev2)
        a = agg.setdefault(name, [0.0, 0])
        a[0] += ms
        a[1] += 1
    out = {k: {"mean_us": 1e3 * v[0] / max(v[1], 1), "count": v[1], "total_ms": v[0]} for k, v in agg.items()}
    if reset_after:
        reset()
    return out

"""Own peer-memory bootstrap (``recsdk_b200/parallel/ipc.py``).

CPU: the rendezvous logic on a fake store - time limit that names the missing ranks, refusal of ranks on another host or
in the same process.  GPU (one device): two processes map each other's allocation through CUDA IPC handles and read what
the other wrote with plain copies (no kernel of one process ever waits for the other)."""
import datetime
import json
import os
import subprocess
import sys
import threading
import time

import pytest
import torch

from recsdk_b200.parallel.ipc import IpcAllocator, PeerInitTimeout

HERE = os.path.dirname(os.path.abspath(__file__))


class FakeStore:
    def __init__(self):
        self.d, self.cv = {}, threading.Condition()

    def set(self, k, v):
        with self.cv:
            self.d[k] = bytes(v)
            self.cv.notify_all()

    def get(self, k):
        return self.d[k]

    def wait(self, keys, timeout: datetime.timedelta):
        end = time.time() + timeout.total_seconds()
        with self.cv:
            while not all(k in self.d for k in keys):
                left = end - time.time()
                if left <= 0:
                    raise RuntimeError("wait timed out")
                self.cv.wait(left)


class _StubLib:
    def rb_ipc_can_access(self, a, b):
        return 1


def _alloc(store, rank, world, timeout):
    a = IpcAllocator.__new__(IpcAllocator)
    a.pg, a.device, a.world, a.rank, a.timeout_s, a.store = None, torch.device("cpu"), world, rank, timeout, store
    a.prefix, a._seq, a._buffers, a.peers = "rb_ipc/t", 0, [], []
    return a


def test_bootstrap_times_out_and_names_the_missing_rank(monkeypatch):
    from recsdk_b200.ops import _lib

    monkeypatch.setattr(_lib, "lib", lambda: _StubLib())
    store = FakeStore()
    a = _alloc(store, 0, 3, 0.3)
    store.set("rb_ipc/t/hello/1", json.dumps({"host": "h", "pid": 1, "device": 1}).encode())
    t0 = time.time()
    with pytest.raises(PeerInitTimeout) as e:
        a._bootstrap()
    assert "[2]" in str(e.value) and time.time() - t0 < 5


def test_bootstrap_refuses_other_hosts_and_shared_processes(monkeypatch):
    import socket

    from recsdk_b200.ops import _lib

    monkeypatch.setattr(_lib, "lib", lambda: _StubLib())
    store = FakeStore()
    store.set("rb_ipc/t/hello/1", json.dumps({"host": "elsewhere", "pid": 1, "device": 1}).encode())
    with pytest.raises(RuntimeError, match="one node"):
        _alloc(store, 0, 2, 1.0)._bootstrap()
    store = FakeStore()
    store.set("rb_ipc/t/hello/1", json.dumps({"host": socket.gethostname(), "pid": os.getpid(), "device": 1}).encode())
    with pytest.raises(RuntimeError, match="share a process"):
        _alloc(store, 0, 2, 1.0)._bootstrap()
    store = FakeStore()
    store.set("rb_ipc/t/hello/1", json.dumps({"host": socket.gethostname(), "pid": os.getpid() + 1, "device": 1}).encode())
    a = _alloc(store, 0, 2, 1.0)
    a._bootstrap()
    assert [p["device"] for p in a.peers] == [0, 1]


_CHILD = r"""
import sys, datetime, torch
import torch.distributed as dist
from recsdk_b200.parallel.ipc import IpcAllocator, _DeviceBlock
rank, path = int(sys.argv[1]), sys.argv[2]
dev = torch.device("cuda", 0)
torch.cuda.set_device(dev)
store = dist.FileStore(path, 2)
a = IpcAllocator(None, dev, store=store, init_timeout_s=60, name="t", world=2, rank=rank)
buf = a.alloc(1 << 20)
assert int(buf.local.sum()) == 0                      # zero-filled
buf.local.fill_(17 + rank)
torch.cuda.synchronize()
store.set("filled/%d" % rank, b"1")
store.wait(["filled/%d" % (1 - rank)], datetime.timedelta(seconds=60))
peer = torch.as_tensor(_DeviceBlock(buf.ptrs[1 - rank], 1 << 20), device=dev)
got = peer.clone()
torch.cuda.synchronize()
assert int(got[0]) == 17 + (1 - rank) and bool((got == 17 + (1 - rank)).all()), int(got[0])
store.set("read/%d" % rank, b"1")
store.wait(["read/%d" % (1 - rank)], datetime.timedelta(seconds=60))
a.close()
print("IPC_OK", rank)
"""


@pytest.mark.gpu
def test_two_processes_map_each_others_buffers(tmp_path):
    path = str(tmp_path / "store")
    env = dict(os.environ, PYTHONPATH=os.path.dirname(HERE) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    procs = [subprocess.Popen([sys.executable, "-c", _CHILD, str(r), path], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                              text=True) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    for r, (p, (so, se)) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "IPC_OK %d" % r in so, se[-2000:]

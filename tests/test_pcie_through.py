"""Multi-table row swap through host memory the GPU addresses directly, and the shared-memory segments behind it."""
import os
import subprocess
import sys

import pytest
import torch

from recsdk_b200.ops.pcie_through import MappedHostBuffer, swap_multi_tables

HERE = os.path.dirname(os.path.abspath(__file__))


def _scenario(device, host_tensor):
    g = torch.Generator().manual_seed(4)
    dims = [8, 16, 4]
    tables = [torch.randn(50 + 10 * i, d, generator=g).to(device) for i, d in enumerate(dims)]
    before = [t.clone().cpu() for t in tables]
    out_idx = [torch.tensor([3, 7, -1, 11]), None, torch.tensor([0, 1])]
    in_idx = [torch.tensor([7, 20]), torch.tensor([5, -1, 6]), None]
    host_out = [host_tensor(4, dims[0]), None, host_tensor(2, dims[2])]
    host_in = [host_tensor(2, dims[0]), host_tensor(3, dims[1]), None]
    for h in host_in:
        if h is not None:
            h.copy_(torch.randn(h.shape, generator=g))
    new_rows = [None if h is None else h.clone() for h in host_in]
    swap_multi_tables(tables, [None if i is None else i.to(device) for i in out_idx], host_out,
                      [None if i is None else i.to(device) for i in in_idx], host_in)
    if device != "cpu":
        torch.cuda.synchronize()
    # swap-out saw the OLD rows (slot 7 of table 0 is in both lists)
    assert torch.equal(host_out[0][0], before[0][3]) and torch.equal(host_out[0][1], before[0][7])
    assert torch.equal(host_out[0][3], before[0][11]) and torch.equal(host_out[2], before[2][:2])
    got = [t.cpu() for t in tables]
    assert torch.equal(got[0][7], new_rows[0][0]) and torch.equal(got[0][20], new_rows[0][1])
    assert torch.equal(got[1][5], new_rows[1][0]) and torch.equal(got[1][6], new_rows[1][2])
    untouched = torch.ones(got[0].shape[0], dtype=torch.bool)
    untouched[[7, 20]] = False
    assert torch.equal(got[0][untouched], before[0][untouched]) and torch.equal(got[2], before[2])


def test_swap_contract_cpu():
    _scenario("cpu", lambda n, d: torch.zeros(n, d))


@pytest.mark.gpu
def test_swap_multi_tables_gpu_pinned_and_shared_segment():
    _scenario("cuda", lambda n, d: torch.zeros(n, d).pin_memory())
    seg = MappedHostBuffer("/rb_test_swap_%d" % os.getpid(), 1 << 16, create=True)
    try:
        off = [0]

        def from_seg(n, d):
            t = seg.tensor(torch.float32)[off[0]:off[0] + n * d].view(n, d)
            off[0] += n * d
            t.zero_()
            return t

        assert seg.registered
        _scenario("cuda", from_seg)
    finally:
        seg.close(unlink=True)


_CHILD = r"""
import sys, torch
from recsdk_b200.ops.pcie_through import MappedHostBuffer
seg = MappedHostBuffer(sys.argv[1], 0, create=False, register=False)
t = seg.tensor(torch.int32)
assert seg.nbytes == 4096 and int(t[0]) == 1234
t[1] = 4321
seg.close()
print("ATTACHED")
"""


def test_shared_segment_between_processes():
    name = "/rb_test_seg_%d" % os.getpid()
    seg = MappedHostBuffer(name, 4096, create=True, register=False)
    try:
        t = seg.tensor(torch.int32)
        t.zero_()
        t[0] = 1234
        env = dict(os.environ, PYTHONPATH=os.path.dirname(HERE) + os.pathsep + os.environ.get("PYTHONPATH", ""))
        r = subprocess.run([sys.executable, "-c", _CHILD, name], env=env, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and "ATTACHED" in r.stdout, r.stderr[-2000:]
        assert int(t[1]) == 4321
        with pytest.raises(OSError):
            MappedHostBuffer("/rb_no_such_segment_%d" % os.getpid(), 0, create=False, register=False)
        with pytest.raises(ValueError):
            MappedHostBuffer("no_slash", 16)
    finally:
        seg.close(unlink=True)

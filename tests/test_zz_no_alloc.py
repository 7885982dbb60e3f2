"""The allocation-free de-duplication entry point (``rb_sort_segments_noalloc``).

Some users of this library cannot allocate device memory when they need to de-duplicate ids: a
serving process whose pools already own the whole GPU, a request thread that must not take the
allocator's device-wide synchronisation, or a C host without PyTorch's caching allocator.  For them
the library keeps the sort workspace in a fixed device array.  This test calls that entry point
through its exported C symbol, twice in a row (the second call finds the first call's leftovers in
the shared scratch), and requires bit-identical results to the regular ``rb_sort_segments``.
Collected last on purpose, so that a failure here cannot hide any other test of the suite.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_KEYS = 1 << 18
ERR_TOO_LARGE = -20


def _load():
    from recsdk_b200 import _build

    lib = ctypes.CDLL(str(_build.build_cuda()))
    fn = lib.rb_sort_segments_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def _reference(keys, vals, end_bit):
    from recsdk_b200.ops import _lib

    n, dev = keys.numel(), keys.device
    L = _lib.lib()
    temp_bytes = int(L.rb_sort_segments_temp_bytes(n))
    ko, vo, uo = torch.empty_like(keys), torch.empty_like(vals), torch.empty_like(keys)
    counts = torch.empty(n + 1, dtype=torch.int32, device=dev)
    seg = torch.empty(n + 1, dtype=torch.int32, device=dev)
    nr = torch.zeros(1, dtype=torch.int32, device=dev)
    temp = torch.empty(temp_bytes, dtype=torch.uint8, device=dev)
    rc = L.rb_sort_segments(keys.data_ptr(), vals.data_ptr(), n, end_bit, ko.data_ptr(), vo.data_ptr(), uo.data_ptr(),
                            counts.data_ptr(), seg.data_ptr(), nr.data_ptr(), temp.data_ptr(), temp_bytes,
                            torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return ko, vo, uo, seg, nr


def _noalloc(fn, keys, vals, end_bit):
    n, dev = keys.numel(), keys.device
    ko, vo, uo = torch.empty_like(keys), torch.empty_like(vals), torch.empty_like(keys)
    seg = torch.empty(n + 1, dtype=torch.int32, device=dev)
    nr = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = fn(keys.data_ptr(), vals.data_ptr(), n, end_bit, ko.data_ptr(), vo.data_ptr(), uo.data_ptr(), seg.data_ptr(),
            nr.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, (ko, vo, uo, seg, nr)


def test_noalloc_matches_regular_entry_point_twice():
    fn = _load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(5)
    # first call: many runs; second call: fewer keys and fewer runs, so stale counts of the first call
    # sit beyond the second call's run count in the shared scratch
    for n, hi in ((200_000, 50_000), (70_001, 900)):
        keys = torch.randint(0, hi, (n,), generator=g, device=dev, dtype=torch.int64)
        keys[::97] = -1                                   # "not owned" marker used by the embedding backward
        vals = torch.arange(n, device=dev, dtype=torch.int32)
        end_bit = max(1, int(hi + 1).bit_length())
        rc, got = _noalloc(fn, keys, vals, end_bit)
        assert rc == 0, "rb_sort_segments_noalloc returned %d" % rc
        want = _reference(keys, vals, end_bit)
        torch.cuda.synchronize()
        runs = int(want[4].item())
        assert int(got[4].item()) == runs
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
        assert torch.equal(got[2][:runs], want[2][:runs])
        assert torch.equal(got[3], want[3])


def test_noalloc_rejects_oversize():
    fn = _load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n = MAX_KEYS + 1
    keys = torch.zeros(n, dtype=torch.int64, device=dev)
    vals = torch.zeros(n, dtype=torch.int32, device=dev)
    rc, _ = _noalloc(fn, keys, vals, 8)
    assert rc == ERR_TOO_LARGE


def test_noalloc_empty_batch_and_second_device():
    """An empty batch writes a run count of zero (and ``seg_offsets[0] = 0``) without touching the other outputs; on a
    machine with a second GPU the same entry point resolves that device's own copy of the scratch array."""
    fn = _load()
    devices = [torch.device("cuda", i) for i in range(min(torch.cuda.device_count(), 2))]
    for dev in devices:
        with torch.cuda.device(dev):
            seg = torch.full((1,), 7, dtype=torch.int32, device=dev)
            nr = torch.full((1,), 7, dtype=torch.int32, device=dev)
            rc = fn(None, None, 0, 8, None, None, None, seg.data_ptr(), nr.data_ptr(), torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            torch.cuda.synchronize(dev)
            assert int(nr.item()) == 0 and int(seg.item()) == 0
            g = torch.Generator(device=dev).manual_seed(11)
            keys = torch.randint(0, 300, (5000,), generator=g, device=dev, dtype=torch.int64)
            vals = torch.arange(5000, device=dev, dtype=torch.int32)
            rc, got = _noalloc(fn, keys, vals, 9)
            assert rc == 0
            want = _reference(keys, vals, 9)
            torch.cuda.synchronize(dev)
            runs = int(want[4].item())
            assert int(got[4].item()) == runs and torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
            assert torch.equal(got[3][:runs + 1], want[3][:runs + 1])

"""Device-side waits are bounded: a barrier whose peer never arrives gives up after its time limit, reports
``RB_ERR_PEER_TIMEOUT`` through the status word and leaves the context usable (no trap, no hang).  The "missing
peer" is a flag word in this GPU's own memory that nothing sets; a single launch, one GPU."""
import numpy as np
import pytest
import torch

from recsdk_b200.ops import _lib

pytestmark = pytest.mark.gpu


def test_barrier_times_out_with_status_and_context_survives():
    dev = torch.device("cuda", 0)
    pad_self = torch.zeros(64 * 16, dtype=torch.int32, device=dev)
    pad_absent = torch.zeros(64 * 16, dtype=torch.int32, device=dev)       # stands in for a rank that never joins
    ptrs = np.array([pad_self.data_ptr(), pad_absent.data_ptr()], dtype=np.uint64)
    epoch = torch.zeros(4, dtype=torch.int32, device=dev)
    status = _lib.status_tensor(dev)
    status.zero_()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = _lib.lib().rb_peer_barrier(ptrs.ctypes.data, epoch.data_ptr(), 0, 2, 0, status.data_ptr(), 50, _lib.stream_ptr(dev))
    t1.record()
    assert rc == 0
    torch.cuda.synchronize(dev)
    ms = t0.elapsed_time(t1)
    assert 30.0 < ms < 2000.0, ms                                           # gave up at about the 50 ms limit
    assert int(status[0].item()) == 2                                       # RB_ERR_PEER_TIMEOUT
    with pytest.raises(RuntimeError):
        _lib.check_status(dev)
    _lib.check_status(dev)                                                  # the status word was reset by the failed check
    x = torch.arange(1024, device=dev, dtype=torch.float32)
    assert float((x * 2).sum().item()) == 2.0 * 1023 * 1024 / 2            # the context still runs kernels

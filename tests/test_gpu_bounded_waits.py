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


def test_exchange_wait_times_out_and_status_poller_raises():
    """The push exchange's wait kernel gives up on a flag that no rank raises (a 2-rank control block whose second rank is a
    buffer nothing writes), and the pipelines' asynchronous status watch turns the status word into ``PeerTimeoutError``
    within two polling periods - no synchronisation in between, the context stays usable."""
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    ctl_self = torch.zeros(int(L.rb_a2a_ctl_ints()), dtype=torch.int32, device=dev)
    ctl_absent = torch.zeros_like(ctl_self)
    ptrs = np.array([ctl_self.data_ptr(), ctl_absent.data_ptr()], dtype=np.uint64)
    loc = torch.zeros(int(L.rb_a2a_loc_ints()), dtype=torch.int32, device=dev)
    loc[2] = 1                                   # epoch of phase 2 is 1: the wait expects flag >= 1 from both ranks
    ctl_self[16 * 16 + 2 * 16 + 0] = 1           # rank 0 (this one) raised its flag; rank 1 never does
    status = _lib.status_tensor(dev)
    status.zero_()
    poller = _lib.StatusPoller(dev, every=2)
    rc = L.rb_a2a_wait(ptrs.ctypes.data, loc.data_ptr(), 2, 2, 0, status.data_ptr(), 50, _lib.stream_ptr(dev))
    assert rc == 0
    with pytest.raises(_lib.PeerTimeoutError):
        for _ in range(6):
            poller.poll()
    torch.cuda.synchronize(dev)
    assert int(status[0].item()) == 0            # the poller cleared it
    assert float((torch.ones(8, device=dev) * 2).sum().item()) == 16.0

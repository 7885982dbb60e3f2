"""Process-group environment and peer-mapped device memory.

``ShardingEnv`` carries (world size, rank, process group) like the reference's user flow
(``ShardingEnv.from_process_group``; ``hybrid_torchrec/distributed/sharding_plan.py:18-28``).

``PeerGroup`` is the B200 counterpart of the reference's LCAL communicator
(``training/common/src/core/lccl/include/lcal_comm.h:33-99``): it allocates device buffers that every
GPU of the node maps into its own address space, so kernels read and write peers' HBM directly
over NVLink / NVSwitch.  Allocation and handle exchange use PyTorch symmetric memory (CUDA VMM
handles exchanged over the process group); the kernels that use the mappings are this library's own.
"""
from __future__ import annotations

import dataclasses
import os
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..ops import _lib


@dataclasses.dataclass
class ShardingEnv:
    world_size: int
    rank: int
    process_group: Optional["dist.ProcessGroup"] = None

    @staticmethod
    def from_process_group(pg: Optional["dist.ProcessGroup"]) -> "ShardingEnv":
        if pg is None and not (dist.is_available() and dist.is_initialized()):
            return ShardingEnv(1, 0, None)
        return ShardingEnv(dist.get_world_size(pg), dist.get_rank(pg), pg)

    @staticmethod
    def from_local(world_size: int, rank: int) -> "ShardingEnv":
        return ShardingEnv(world_size, rank, None)


class PeerBuffer:
    """One symmetric allocation: ``local`` is this rank's tensor, ``ptrs[r]`` the address of rank
    ``r``'s copy as mapped here, ``multicast_ptr`` the NVSwitch multicast mapping (0 if none)."""

    def __init__(self, local: torch.Tensor, ptrs: List[int], multicast_ptr: int, handle=None) -> None:
        self.local = local
        self.ptrs = [int(p) for p in ptrs]
        self.multicast_ptr = int(multicast_ptr or 0)
        self._handle = handle
        self._ptr_arr = np.asarray(self.ptrs, dtype=np.uint64)

    def ptr_array(self) -> int:
        """Host address of a uint64[world] array of the peer pointers (argument of the C launchers)."""
        return self._ptr_arr.ctypes.data

    def ptr_tensor(self, device: torch.device, offset_bytes: int = 0) -> torch.Tensor:
        return torch.tensor([p + offset_bytes for p in self.ptrs], dtype=torch.int64, device=device)


class PeerGroup:
    """All GPUs of one process group on one NVSwitch node."""

    PAD_INTS = 64 * 16

    def __init__(self, pg: Optional["dist.ProcessGroup"], device: torch.device, timeout_ms: Optional[int] = None) -> None:
        self.pg = pg if pg is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.device = device
        self.world = dist.get_world_size(self.pg) if self.pg is not None else 1
        self.rank = dist.get_rank(self.pg) if self.pg is not None else 0
        # limit of every device-side wait for a peer: long enough for the start-up skew of a cold job (first launches page
        # the kernels in), short enough that a lost rank surfaces as an error within seconds
        self.timeout_ms = int(timeout_ms if timeout_ms is not None else os.environ.get("RECSDK_B200_PEER_TIMEOUT_MS", "10000"))
        # NVSwitch multicast (multimem.ld_reduce / multimem.st in the all-reduce) is opt-in: RECSDK_B200_MULTIMEM=1.
        # Without it the peer buffers are not bound to a multicast object at all (plain peer loads / stores only), which
        # is also what jobs whose ranks may leave need.
        self.use_multimem = os.environ.get("RECSDK_B200_MULTIMEM", "0") == "1"
        if not self.use_multimem:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self._symm = None
        # who allocates and exchanges the peer buffers: PyTorch symmetric memory ("symm", default; also provides the
        # multicast mapping) or this package's own CUDA-IPC bootstrap ("ipc", recsdk_b200/parallel/ipc.py)
        self.backend = os.environ.get("RECSDK_B200_PEER_BACKEND", "symm")
        if self.backend not in ("symm", "ipc"):
            raise ValueError("RECSDK_B200_PEER_BACKEND must be 'symm' or 'ipc'")
        self._ipc = None
        if self.world > 1 and self.backend == "ipc":
            from .ipc import IpcAllocator

            if self.use_multimem:
                raise ValueError("the ipc peer backend has no multicast mapping: unset RECSDK_B200_MULTIMEM")
            self._ipc = IpcAllocator(self.pg, device, name="pg%s" % getattr(self.pg, "group_name", "world"))
        elif self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem

            self._symm = symm_mem
        if self.world > 1 and device.type == "cuda" and "RECSDK_B200_GEMM_CONCURRENT" not in os.environ:
            # the exchange and the gradient buckets run on side streams beside the MLP GEMMs: use the GEMM variant whose CTAs
            # leave room on the SM for their blocks
            _lib.lib().rb_gemm_set_concurrent(1)
        pad = self.alloc(self.PAD_INTS * 4, zero=True)
        self.pads = pad
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.abort_word = torch.zeros(1, dtype=torch.int32, device=device)
        if self.world > 1:
            torch.cuda.synchronize(device)
            dist.barrier(group=self.pg)

    def alloc(self, nbytes: int, zero: bool = False) -> PeerBuffer:
        nbytes = (int(nbytes) + 255) // 256 * 256
        if self.world == 1:
            t = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            if zero:
                t.zero_()
            return PeerBuffer(t, [t.data_ptr()], 0)
        if self._ipc is not None:
            b = self._ipc.alloc(nbytes)                     # zero-filled by the allocator
            return PeerBuffer(b.local, b.ptrs, 0, b)
        t = self._symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        if zero:
            t.zero_()
        hdl = self._symm.rendezvous(t, group=self.pg.group_name)
        mc = 0
        if self.use_multimem:
            try:
                mc = int(hdl.multicast_ptr or 0)
            except Exception:  # noqa: BLE001
                mc = 0
        return PeerBuffer(t, list(hdl.buffer_ptrs), mc, hdl)

    def host_barrier(self) -> None:
        """Host-side rendezvous of all ranks (set-up paths only)."""
        if self.world > 1:
            dist.barrier(group=self.pg)

    # -- collectives on the current stream ---------------------------------------
    def barrier(self, slot: int = 0) -> None:
        """Device-side barrier of all ranks, ordered with the current stream; never blocks the host."""
        if self.world == 1:
            return
        rc = _lib.lib().rb_peer_barrier(self.pads.ptr_array(), self.epoch.data_ptr(), self.rank, self.world, slot,
                                        _lib.status_tensor(self.device).data_ptr(), self.timeout_ms,
                                        _lib.stream_ptr(self.device))
        _lib.check(rc, "rb_peer_barrier")

    def allgather_push_2d(self, dst: PeerBuffer, src: torch.Tensor, dst_row_bytes: int, dst_col_bytes: int) -> None:
        """``dst_r[row, dst_col_bytes : +row_bytes] = src[row]`` on every rank ``r`` (no barrier)."""
        assert src.is_contiguous() and src.dim() == 2
        row_bytes = src.shape[1] * src.element_size()
        rc = _lib.lib().rb_allgather_push_2d(dst.ptr_array(), src.data_ptr(), src.shape[0], row_bytes, dst_row_bytes,
                                             dst_col_bytes, self.world, _lib.num_sms(self.device),
                                             _lib.stream_ptr(self.device))
        _lib.check(rc, "rb_allgather_push_2d")

    def allreduce_mean_f32(self, buf: PeerBuffer, n: int, offset_bytes: int = 0, scale: Optional[float] = None) -> None:
        """In-place averaged all-reduce of ``n`` fp32 values at ``offset_bytes`` of a peer buffer."""
        if self.world == 1:
            return
        ptrs = np.asarray([p + offset_bytes for p in buf.ptrs], dtype=np.uint64)
        mc = buf.multicast_ptr + offset_bytes if buf.multicast_ptr else None
        rc = _lib.lib().rb_allreduce_f32(ptrs.ctypes.data, mc, self.pads.ptr_array(), self.epoch.data_ptr(), n,
                                         (1.0 / self.world) if scale is None else float(scale), self.rank,
                                         self.world, 2, _lib.status_tensor(self.device).data_ptr(), self.timeout_ms,
                                         self.abort_word.data_ptr(), _lib.num_sms(self.device),
                                         _lib.stream_ptr(self.device))
        _lib.check(rc, "rb_allreduce_f32")

"""Own peer-memory bootstrap: symmetric device buffers shared between the ranks of one node through CUDA IPC handles.

``IpcAllocator(pg, device)`` gives ``PeerGroup`` the same thing PyTorch's symmetric memory does - a local buffer plus
the address of every other rank's buffer mapped into this process - with this package's own allocation
(``csrc/cuda/ipc.cu``), handle exchange and time limits:

* every rank allocates, exports a 64-byte handle and publishes it in the job's key-value store (the TCP store of
  ``torch.distributed``; any object with ``set`` / ``get`` / ``wait`` works);
* ``store.wait`` with ``init_timeout_s`` bounds the rendezvous: a rank that never arrives ends the set-up with
  ``PeerInitTimeout`` that names the missing ranks, instead of a hang;
* ranks must sit on one node and see each other's device (checked with ``cudaDeviceCanAccessPeer``); a rank on another
  host is refused at bootstrap.

Select it with ``RECSDK_B200_PEER_BACKEND=ipc`` (default ``symm``: PyTorch symmetric memory, which also offers the
NVSwitch multicast mapping).  Role in the reference: LCAL's own communicator bootstrap (socket exchange of IPC buffer
handles, init timeout) under LCCL.
"""
from __future__ import annotations

import ctypes
import datetime
import os
import socket
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib


class PeerInitTimeout(RuntimeError):
    """Not every rank published its handle within the time limit."""


class _DeviceBlock:
    """A raw device allocation exposed through the CUDA array interface (``torch.as_tensor`` wraps it without a copy)."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.ptr, self.nbytes = int(ptr), int(nbytes)
        self.__cuda_array_interface__ = {"shape": (self.nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 2}


class IpcBuffer:
    def __init__(self, local: torch.Tensor, ptrs: List[int], owner: "IpcAllocator", block: _DeviceBlock, mapped: List[int]) -> None:
        self.local, self.ptrs, self._owner, self._block, self._mapped = local, ptrs, owner, block, mapped


class IpcAllocator:
    def __init__(self, pg: Optional["dist.ProcessGroup"], device: torch.device, store: Any = None,
                 init_timeout_s: Optional[float] = None, name: str = "default", world: Optional[int] = None,
                 rank: Optional[int] = None) -> None:
        """``world`` / ``rank`` with a ``store`` replace the process group (a bootstrap before, or without, one)."""
        self.pg, self.device = pg, device
        self.world = int(world) if world is not None else (dist.get_world_size(pg) if pg is not None else 1)
        self.rank = int(rank) if rank is not None else (dist.get_rank(pg) if pg is not None else 0)
        self.timeout_s = float(init_timeout_s if init_timeout_s is not None else os.environ.get("RECSDK_B200_PEER_INIT_TIMEOUT_S", "120"))
        self.store = store
        if self.store is None and self.world > 1:
            from torch.distributed.distributed_c10d import _get_default_store

            self.store = _get_default_store()
        self.prefix = "rb_ipc/%s" % name
        self._seq = 0
        self._buffers: List[IpcBuffer] = []
        self.peers: List[Dict[str, Any]] = []
        if self.world > 1:
            self._bootstrap()

    # ------------------------------------------------------------------ store helpers (bounded)
    def _publish(self, tag: str, payload: bytes) -> None:
        self.store.set("%s/%s/%d" % (self.prefix, tag, self.rank), payload)

    def _collect(self, tag: str) -> List[bytes]:
        keys = ["%s/%s/%d" % (self.prefix, tag, r) for r in range(self.world)]
        try:
            self.store.wait(keys, datetime.timedelta(seconds=self.timeout_s))
        except Exception as e:  # noqa: BLE001 - the store raises its own timeout type
            missing = []
            for r, k in enumerate(keys):
                try:
                    self.store.wait([k], datetime.timedelta(milliseconds=1))
                except Exception:  # noqa: BLE001
                    missing.append(r)
            raise PeerInitTimeout("peer bootstrap %r: ranks %s did not arrive within %.0f s" % (tag, missing, self.timeout_s)) from e
        return [bytes(self.store.get(k)) for k in keys]

    def _bootstrap(self) -> None:
        import json

        me = {"host": socket.gethostname(), "pid": os.getpid(), "device": int(self.device.index or 0)}
        self._publish("hello", json.dumps(me).encode())
        self.peers = [json.loads(b.decode()) for b in self._collect("hello")]
        L = _lib.lib()
        for r, p in enumerate(self.peers):
            if p["host"] != me["host"]:
                raise RuntimeError("rank %d runs on host %s: IPC peer memory needs all ranks on one node" % (r, p["host"]))
            if r != self.rank and p["pid"] == me["pid"]:
                raise RuntimeError("ranks %d and %d share a process: IPC handles cannot be opened by their own process" % (r, self.rank))
            if int(L.rb_ipc_can_access(me["device"], p["device"])) != 1:
                raise RuntimeError("device %d cannot map memory of device %d (rank %d)" % (me["device"], p["device"], r))

    # ------------------------------------------------------------------ allocation
    def alloc(self, nbytes: int) -> IpcBuffer:
        """Collective over the group: every rank calls it with the same size, in the same order."""
        L = _lib.lib()
        torch.cuda.set_device(self.device)
        raw = ctypes.c_void_p()
        _lib.check(L.rb_ipc_alloc(int(nbytes), ctypes.byref(raw)), "rb_ipc_alloc")
        block = _DeviceBlock(raw.value, nbytes)
        local = torch.as_tensor(block, device=self.device)
        ptrs, mapped = [int(raw.value)], []
        if self.world > 1:
            self._seq += 1
            tag = "buf%d" % self._seq
            h = (ctypes.c_ubyte * int(L.rb_ipc_handle_bytes()))()
            _lib.check(L.rb_ipc_export(raw, h), "rb_ipc_export")
            self._publish(tag, bytes(h))
            blobs = self._collect(tag)
            ptrs = []
            for r, blob in enumerate(blobs):
                if r == self.rank:
                    ptrs.append(int(raw.value))
                    continue
                m = ctypes.c_void_p()
                hb = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
                _lib.check(L.rb_ipc_open(hb, ctypes.byref(m)), "rb_ipc_open (rank %d)" % r)
                ptrs.append(int(m.value))
                mapped.append(int(m.value))
        buf = IpcBuffer(local, ptrs, self, block, mapped)
        self._buffers.append(buf)
        return buf

    def close(self) -> None:
        """Unmap the peers' buffers, meet, then free the own ones (collective; optional - process exit frees everything)."""
        L = _lib.lib()
        for b in self._buffers:
            for m in b._mapped:
                L.rb_ipc_close(ctypes.c_void_p(m))
            b._mapped = []
        if self.world > 1:
            self._publish("bye", b"1")
            self._collect("bye")
        for b in self._buffers:
            b.local = None
            L.rb_ipc_free(ctypes.c_void_p(b._block.ptr))
        self._buffers = []

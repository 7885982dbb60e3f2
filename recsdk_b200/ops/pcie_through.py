"""Rows swapped between device tables and host memory that the GPU addresses directly, several tables per call, and the
named shared-memory segments that provide such memory (``csrc/cuda/pcie_through.cu``).

    seg = MappedHostBuffer("/rb_swap_in", nbytes, create=True)          # another process attaches with create=False
    swap_multi_tables(tables, swap_out_index, host_out, swap_in_index, host_in)

``host_out[t]`` / ``host_in[t]`` are ``[n, row]`` tensors over pinned or registered host memory (``MappedHostBuffer.tensor``
or ``tensor.pin_memory()``); on CPU tensors the same contract runs as plain indexing.  Swap-out precedes swap-in, so a
slot may hand its old row to the host and take a new one in the same call.  Role in the reference: the
``RmaSwapMultiTables`` operator and ``rma_shm_svm`` (``training/common/src/core/pcie_through``).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib

MAX_TABLES = 8


class MappedHostBuffer:
    """A POSIX shared-memory segment mapped into this process; with ``register`` (default on CUDA machines) it is
    page-locked and mapped for the GPU, so kernels read and write it in place."""

    def __init__(self, name: str, nbytes: int = 0, create: bool = True, register: Optional[bool] = None) -> None:
        if not name.startswith("/") or "/" in name[1:]:
            raise ValueError("segment names look like '/name' (one leading slash, no others)")
        if register is None:
            register = torch.cuda.is_available()
        self.name, self.registered = name, bool(register)
        h, p, n = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_longlong(0)
        rc = _lib.lib().rb_shm_open(name.encode(), int(nbytes), int(create), int(register), ctypes.byref(h), ctypes.byref(p),
                                    ctypes.byref(n))
        if rc != 0:
            reason = {-1: "bad name", -2: "segment does not exist or cannot be opened", -3: "cannot size the segment",
                      -4: "segment smaller than requested", -5: "mmap failed", -6: "out of memory"}.get(rc)
            raise OSError("rb_shm_open(%s): %s" % (name, reason or ("CUDA error %d while registering" % rc)))
        self._h, self.ptr, self.nbytes = h, int(p.value), int(n.value)
        self._buf = (ctypes.c_uint8 * self.nbytes).from_address(self.ptr)

    def tensor(self, dtype: torch.dtype = torch.uint8, shape: Optional[Sequence[int]] = None) -> torch.Tensor:
        t = torch.frombuffer(self._buf, dtype=torch.uint8).view(dtype)
        return t.view(*shape) if shape is not None else t

    def close(self, unlink: bool = False) -> None:
        if self._h is not None:
            self._buf = None
            _lib.lib().rb_shm_close(self._h, int(unlink))
            self._h = None

    def __del__(self) -> None:
        try:
            self.close(False)
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


def _addr_array(tensors: Sequence[Optional[torch.Tensor]]) -> np.ndarray:
    return np.asarray([0 if t is None else t.data_ptr() for t in tensors], dtype=np.uint64)


def swap_multi_tables(tables: List[torch.Tensor], swap_out_index: Optional[List[Optional[torch.Tensor]]],
                      host_out: Optional[List[Optional[torch.Tensor]]], swap_in_index: Optional[List[Optional[torch.Tensor]]],
                      host_in: Optional[List[Optional[torch.Tensor]]]) -> None:
    """``host_out[t][i] = tables[t][swap_out_index[t][i]]`` then ``tables[t][swap_in_index[t][i]] = host_in[t][i]`` for every
    table (index -1 skips an entry).  Tables are 2-D, row-major; at most 8 per call."""
    T = len(tables)
    if not 1 <= T <= MAX_TABLES:
        raise ValueError("between 1 and %d tables per call" % MAX_TABLES)
    none = [None] * T
    swap_out_index, host_out = swap_out_index or none, host_out or none
    swap_in_index, host_in = swap_in_index or none, host_in or none
    if not tables[0].is_cuda:
        for t in range(T):
            if swap_out_index[t] is not None and swap_out_index[t].numel():
                keep = swap_out_index[t] >= 0
                host_out[t][keep] = tables[t][swap_out_index[t][keep]]
        for t in range(T):
            if swap_in_index[t] is not None and swap_in_index[t].numel():
                keep = swap_in_index[t] >= 0
                tables[t][swap_in_index[t][keep]] = host_in[t][keep].to(tables[t].dtype)
        return
    dev = tables[0].device
    for t in range(T):
        tab = tables[t]
        assert tab.is_cuda and tab.dim() == 2 and tab.is_contiguous() and (tab.shape[1] * tab.element_size()) % 16 == 0
        for idx, hst in ((swap_out_index[t], host_out[t]), (swap_in_index[t], host_in[t])):
            if idx is None:
                continue
            assert idx.is_cuda and idx.dtype == torch.int64 and idx.is_contiguous()
            assert hst is not None and hst.is_contiguous() and hst.dtype == tab.dtype and hst.shape[1:] == tab.shape[1:]
            assert hst.shape[0] >= idx.numel() and (hst.is_cuda or hst.is_pinned()), "host rows must be pinned / registered"
    rows = np.asarray([t.shape[0] for t in tables], dtype=np.int64)
    rb = np.asarray([t.shape[1] * t.element_size() for t in tables], dtype=np.int64)
    n_out = np.asarray([0 if i is None else i.numel() for i in swap_out_index], dtype=np.int64)
    n_in = np.asarray([0 if i is None else i.numel() for i in swap_in_index], dtype=np.int64)
    a_tab, a_oi, a_ho = _addr_array(tables), _addr_array(swap_out_index), _addr_array(host_out)
    a_ii, a_hi = _addr_array(swap_in_index), _addr_array(host_in)
    rc = _lib.lib().rb_swap_multi_tables(a_tab.ctypes.data, rows.ctypes.data, rb.ctypes.data, T, a_oi.ctypes.data, n_out.ctypes.data,
                                         a_ho.ctypes.data, a_ii.ctypes.data, n_in.ctypes.data, a_hi.ctypes.data,
                                         _lib.num_sms(dev), _lib.status_tensor(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "rb_swap_multi_tables")


rma_swap_multi_tables = swap_multi_tables        # name of the reference's operator (tf_plugin/src/ram_swap_multi_tables.cpp)

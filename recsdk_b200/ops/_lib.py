"""ctypes binding of ``_C_cuda.so`` (the sm_100a kernels).

Every exported launcher takes raw device pointers, sizes and a ``cudaStream_t`` and returns an
``int`` (0 = ok, >0 = ``cudaError_t``, <0 = argument error).  Signatures are declared with a
one-letter-per-argument code: ``p`` pointer, ``i`` int32, ``l`` int64, ``f`` float.

On a machine with a GPU the library must load; a missing or broken ``.so`` raises instead of
silently falling back to PyTorch ops.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Dict, Optional

import torch

from .. import _build

from ._signatures import SIGNATURES as _SIGS

_CT = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_longlong, "f": ctypes.c_float,
       "d": ctypes.c_double, "v": None}

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_load_error: Optional[BaseException] = None


def _declare(lib: ctypes.CDLL) -> None:
    for name, sig in _SIGS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.restype = _CT[sig[0]]
        fn.argtypes = [_CT[c] for c in sig[1:]]


# kernels launched by one call of a launcher (default 1); used for the launch counter only
_KERNELS_PER_CALL = {"rb_sort_segments": 8, "rb_sort_pairs_i64_i32": 4, "rb_tbe_backward_update": 2, "rb_tbe_backward_update_rows": 2, "rb_a2a_ctl_ints": 0, "rb_a2a_loc_ints": 0, "rb_a2a_loc_n_owned_index": 0,
                     "rb_allreduce_push_staging_bytes": 0, "rb_allreduce_push_max_blocks": 0, "rb_sort_segments_temp_bytes": 0}
launch_count = 0


class _CountingLib:
    """Thin proxy over the ``CDLL`` that counts how many of this library's kernels were launched."""

    def __init__(self, handle: ctypes.CDLL) -> None:
        self._h = handle
        self._cache: Dict[str, object] = {}

    def __getattr__(self, name: str):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._h, name)
            n = _KERNELS_PER_CALL.get(name, 1)

            def fn(*args, _raw=raw, _n=n):
                global launch_count
                launch_count += _n
                return _raw(*args)

            self._cache[name] = fn
        return fn


def lib():
    """Load (building first when the sources are newer) and return the kernel library."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            so = _build.CUDA_SO
            if os.environ.get("RECSDK_B200_NO_BUILD", "0") != "1":
                try:
                    so = _build.build_cuda()
                except Exception:
                    if not so.exists():
                        raise
            handle = ctypes.CDLL(str(so), mode=ctypes.RTLD_GLOBAL)
            _declare(handle)
            _lib = _CountingLib(handle)
        except BaseException as e:  # noqa: BLE001 - re-raised below with context
            _load_error = e
            raise RuntimeError(
                "recsdk_b200: the sm_100a kernel library could not be built/loaded (%s). "
                "GPU execution has no PyTorch fallback." % (e,)
            ) from e
    return _lib


def available() -> bool:
    """True when a CUDA device is present (the kernels are then mandatory)."""
    return torch.cuda.is_available()


def stream_ptr(device: Optional[torch.device] = None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    return t.data_ptr()


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc > 0:
        raise RuntimeError("%s: CUDA error %d (%s)" % (what, rc, _cuda_err_name(rc)))
    if rc <= -1000:
        raise RuntimeError("%s: cuTensorMapEncodeTiled failed with CUresult %d" % (what, -rc - 1000))
    raise ValueError("%s: invalid arguments (code %d)" % (what, rc))


def _cuda_err_name(rc: int) -> str:
    try:
        rt = ctypes.CDLL("libcudart.so")
        rt.cudaGetErrorString.restype = ctypes.c_char_p
        return rt.cudaGetErrorString(rc).decode()
    except Exception:  # noqa: BLE001
        return "?"


_DT_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def dtype_code(dt: torch.dtype) -> int:
    return _DT_CODE[dt]


_num_sms_cache: Dict[int, int] = {}


def num_sms(device: Optional[torch.device] = None) -> int:
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _num_sms_cache:
        _num_sms_cache[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _num_sms_cache[idx]


# ---------------------------------------------------------------------------
# device status word (bounded waits / bounds checks report here)
# ---------------------------------------------------------------------------
_status: Dict[int, torch.Tensor] = {}

STATUS_NAMES = {0: "ok", 1: "mbarrier wait timed out", 2: "peer flag wait timed out",
                3: "index out of bounds", 4: "fixed-size buffer overflow"}


class KernelStatusError(RuntimeError):
    """A kernel of this library reported a problem through the device status word."""

    def __init__(self, code: int) -> None:
        super().__init__("recsdk_b200 kernel status %d: %s" % (code, STATUS_NAMES.get(code, "?")))
        self.code = code


class PeerTimeoutError(KernelStatusError):
    """A bounded device-side wait for another rank ran out: the peer is late, has left or has failed.  The collectives
    of the steps since then did not complete, so the job must stop or recover instead of training on."""


class CapacityError(KernelStatusError):
    """A fixed-size device buffer (an owner's receive list, a long-segment list) was too small for a batch and entries were
    dropped; results of that step are incomplete.  Raise the bound named in the module's documentation."""


def raise_for_status(code: int) -> None:
    if code == 0:
        return
    if code == 2:
        raise PeerTimeoutError(code)
    if code == 4:
        raise CapacityError(code)
    raise KernelStatusError(code)


class StatusPoller:
    """Asynchronous watch on the status word: ``poll()`` every step costs one small device-to-host copy every ``every``
    steps and no synchronisation; a non-zero word raises at the next check (at most ``2 * every`` steps late)."""

    def __init__(self, device: torch.device, every: int = 16) -> None:
        self.device, self.every = device, max(1, int(every))
        self._host = torch.zeros(8, dtype=torch.int32).pin_memory() if torch.cuda.is_available() else None
        self._event: Optional[torch.cuda.Event] = None
        self._n = 0

    def poll(self) -> None:
        if self._host is None or self.device.type != "cuda":
            return
        self._n += 1
        if self._n % self.every:
            return
        if self._event is not None:
            self._event.synchronize()              # recorded `every` steps ago: long complete
            code = int(self._host[0])
            if code != 0:
                status_tensor(self.device).zero_()
                self._event = None
                raise_for_status(code)
        if torch.cuda.is_current_stream_capturing():
            return
        self._host.copy_(status_tensor(self.device), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._event = ev


def status_tensor(device: Optional[torch.device] = None) -> torch.Tensor:
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _status:
        _status[idx] = torch.zeros(8, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device: Optional[torch.device] = None, reset: bool = True) -> None:
    """Synchronising read of the status word; raises if any kernel reported a problem."""
    st = status_tensor(device)
    code = int(st[0].item())
    if code != 0:
        if reset:
            st.zero_()
        raise_for_status(code)

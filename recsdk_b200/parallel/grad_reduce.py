"""Bucketed, overlapped all-reduce of the dense gradients (data-parallel part of a model).

One bucket per flat-parameter module (``FusedMLP``-style: ``flat_grad``) plus one bucket for every remaining small
parameter.  Each bucket is averaged by ``rb_allreduce_push`` (``csrc/cuda/collectives.cu``): the fp32 gradients are
converted to bf16 while they are pushed into the slice owner's staging area over NVLink, summed in fp32 from local
memory, scaled by 1/world once and pushed back; small buckets use the one-shot form.  A bucket is launched on a side
stream as soon as its module's backward has produced its last weight gradient, so only the buckets of the first layers
are exposed after the backward.  The reference leaves this exchange to DDP over HCCL
(``docs/en/torch/torch_rec_v1/03_quick_start/quick_start.md:239-262``); its in-kernel collectives are
``cust_op/ascendc_op/ai_core_op/lccl/v220/op_kernel/all2all.h``.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import numpy as np
import torch
from torch import nn

from ..ops import _lib
from ..utils import trace
from .comm import PeerGroup

_ONE_SHOT_BYTES = int(os.environ.get("RECSDK_B200_ALLREDUCE_ONESHOT_BYTES", str(1 << 20)))
_TINY_ELEMS = 1 << 14
_BLOCKS = int(os.environ.get("RECSDK_B200_ALLREDUCE_BLOCKS", "0"))      # 0: the kernel's default grid


class _Bucket:
    def __init__(self, grad: torch.Tensor, module: Optional[nn.Module], params: Sequence[nn.Parameter] = ()) -> None:
        self.grad = grad                  # flat fp32 view that the kernel reduces in place
        self.module = module              # flat module (hooked) or None for the small-parameter bucket
        self.params = list(params)
        self.n = grad.numel()
        self.launched = False
        self.done_event: Optional[torch.cuda.Event] = None
        self.staging = self.result = self.flags = None     # np.uint64[world] peer addresses
        self.epoch: Optional[torch.Tensor] = None
        self.one_shot = False


class DenseGradReducer:
    """``reducer = DenseGradReducer(peer, module)``; call ``reducer.sync()`` between backward and the optimizer step.

    ``overlap=True`` launches a flat module's bucket from the end of that module's backward (one backward per
    ``sync()``; with gradient accumulation over several backward passes use ``overlap=False``)."""

    def __init__(self, peer: Optional[PeerGroup], module: nn.Module, exclude_param_ids: Optional[set] = None,
                 wire_dtype: torch.dtype = torch.bfloat16, overlap: bool = True, average: bool = True) -> None:
        self.peer = peer
        self.world = peer.world if peer is not None else 1
        self.wire_bf16 = 1 if wire_dtype == torch.bfloat16 else 0
        self.scale = (1.0 / self.world) if average else 1.0
        self.buckets: List[_Bucket] = []
        self.blocks = _BLOCKS
        self._small: List[nn.Parameter] = []
        if self.world == 1:
            return
        self.device = peer.device
        exclude = exclude_param_ids or set()
        flat_mods = [m for m in module.modules() if hasattr(m, "flat_grad") and hasattr(m, "flat_param")]
        flat_ids = {id(m.flat_param) for m in flat_mods}
        # tiny flat modules (a logit head) share the small-parameter bucket: their gradient buffer is re-homed into it
        tiny = [m for m in flat_mods if m.flat_grad.numel() < _TINY_ELEMS and hasattr(m, "set_grad_buffer")]
        for m in flat_mods:
            if m not in tiny:
                if m.flat_grad.numel() % 8:
                    raise ValueError("flat gradient buffers must hold a multiple of 8 elements")
                self.buckets.append(_Bucket(m.flat_grad, m))
        small = [p for p in module.parameters() if p.requires_grad and id(p) not in flat_ids and id(p) not in exclude
                 and not getattr(p, "_in_backward_optimizers", False)]
        self._small = small
        pad8 = lambda k: (k + 7) // 8 * 8  # noqa: E731
        n = sum(pad8(p.numel()) for p in small) + sum(pad8(m.flat_grad.numel()) for m in tiny)
        if n:
            self._small_flat = torch.zeros(n, dtype=torch.float32, device=self.device)
            views, off = [], 0
            for p in small:
                views.append(self._small_flat[off:off + p.numel()].view_as(p))
                off += pad8(p.numel())
            for m in tiny:
                m.set_grad_buffer(self._small_flat[off:off + m.flat_grad.numel()])
                off += pad8(m.flat_grad.numel())
            self._small_views = views
            self.buckets.append(_Bucket(self._small_flat, None, small))
        self._alloc()
        self.side = torch.cuda.Stream(self.device)
        if overlap:
            for b in self.buckets:
                if b.module is not None and hasattr(b.module, "set_grad_ready_hook"):
                    b.module.set_grad_ready_hook(lambda _m, b=b: self._launch(b, from_hook=True))

    # ------------------------------------------------------------------ resources
    def _alloc(self) -> None:
        """One peer allocation for all buckets: [staging | result] per bucket, then the flag rows."""
        L = _lib.lib()
        W = self.world
        max_blocks = int(L.rb_allreduce_push_max_blocks())
        flag_bytes = 2 * 16 * max_blocks * 4
        offs, total = [], 0
        for b in self.buckets:
            wire = 2 if self.wire_bf16 else 4
            b.one_shot = b.n * wire <= _ONE_SHOT_BYTES
            sb = int(L.rb_allreduce_push_staging_bytes(b.n, W, self.wire_bf16))
            sb = (sb + 255) // 256 * 256
            offs.append((total, total + sb, sb))
            total += 2 * sb
        flag_off = total
        total += flag_bytes * len(self.buckets)
        self._buf = self.peer.alloc(total, zero=True)
        base = np.asarray(self._buf.ptrs, dtype=np.uint64)
        for i, (b, (so, ro, _sb)) in enumerate(zip(self.buckets, offs)):
            b.staging = base + np.uint64(so)
            b.result = base + np.uint64(ro)
            b.flags = base + np.uint64(flag_off + i * flag_bytes)
            b.epoch = torch.zeros(2, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        self.peer.host_barrier()

    # ------------------------------------------------------------------ launches
    def _launch(self, b: _Bucket, from_hook: bool = False) -> None:
        if b.launched:
            return
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)
        grad = b.module.flat_grad if b.module is not None else b.grad
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev)
            rc = _lib.lib().rb_allreduce_push(grad.data_ptr(), b.n, b.staging.ctypes.data, b.result.ctypes.data,
                                              b.flags.ctypes.data, b.epoch.data_ptr(), self.scale, self.peer.rank,
                                              self.world, self.wire_bf16, int(b.one_shot), self.blocks,
                                              _lib.status_tensor(self.device).data_ptr(), self.peer.timeout_ms,
                                              self.side.cuda_stream)
            _lib.check(rc, "rb_allreduce_push")
            done = torch.cuda.Event()
            done.record(self.side)
        b.done_event, b.launched = done, True

    def sync(self) -> None:
        """Reduce every bucket that has not been launched yet and make the current stream wait for all of them."""
        if self.world == 1:
            return
        trace.mark("dense.grad_allreduce")
        if self._small:
            grads = [p.grad for p in self._small]
            have = [(v, g) for v, g in zip(self._small_views, grads) if g is not None]
            miss = [v for v, g in zip(self._small_views, grads) if g is None]
            if have:
                torch._foreach_copy_([v for v, _ in have], [g for _, g in have])
            for v in miss:
                v.zero_()
        for b in self.buckets:
            self._launch(b)
        main = torch.cuda.current_stream(self.device)
        for b in self.buckets:
            main.wait_event(b.done_event)
            b.launched = False
        if self._small:
            have = [(v, p) for v, p in zip(self._small_views, self._small) if p.grad is not None]
            if have:
                torch._foreach_copy_([p.grad for _, p in have], [v for v, _ in have])
            for v, p in zip(self._small_views, self._small):
                if p.grad is None:
                    p.grad = v.clone()
        trace.mark("step.optimizer")

"""HSTU ranking inference over the paged KV cache.

One request batch = for every user the not-yet-cached tail of the history followed by the candidates to score.
History K/V of every layer stay in the paged cache between requests (device pages, spilled to pinned host
chunks); candidates are request-scoped: their K/V are appended behind the history for the attention kernel and
dropped again afterwards.  Candidates see the whole history and themselves only (target group size 1), so
their scores do not depend on which other candidates share the request.

Per layer:  SiLU(uvqk GEMM) with the activation fused in the GEMM epilogue -> append K/V to the pages -> paged
tcgen05 attention (bias evaluated in the kernel) -> fused norm-gate -> output GEMM with the residual added.
The request flow (lookup -> allocate -> onboard -> layers -> offload) is the reference's
(``inference/kvcache_manager/docs/codeview.md``, ``recsys_kvcache_manager/kvcache_manager.py``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..inference.kvcache_manager import HostKVTaskStatus, KVCacheManager, KVIndexMeta
from ..ops import gemm, hstu_ops
from ..ops.hstu_attention import hstu_attention_paged, hstu_attention_ref
from .hstu import HSTU


def _linear(mlp, x: torch.Tensor, silu: bool) -> torch.Tensor:
    """One-layer ``FusedMLP`` applied without autograd: the tcgen05 GEMM with bias (and SiLU) in its epilogue."""
    if x.is_cuda:
        return gemm.gemm16(x, mlp.w16[0], bias=mlp.b32[0], epi=gemm.EPI_SILU if silu else gemm.EPI_NONE)
    y = torch.nn.functional.linear(x.float(), mlp.w16[0].float()[:, : x.shape[1]], mlp.b32[0])
    return (torch.nn.functional.silu(y) if silu else y).to(x.dtype)


class HSTURanker:
    """``rank(...) -> scores`` for an :class:`HSTU` model; owns no weights, reads the model's."""

    def __init__(self, model: HSTU, kv: KVCacheManager) -> None:
        self.model, self.kv = model, kv
        c = model.cfg
        kc = kv.gpu.cfg
        assert (kc.num_layers, kc.num_heads, kc.head_dim) == (c.num_layers, c.num_heads, c.head_dim)
        self.device = kv.gpu.device

    @torch.no_grad()
    def rank(self, user_ids: torch.Tensor, history_lengths: torch.Tensor, num_candidates: torch.Tensor, x_new: torch.Tensor,
             timestamps: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``user_ids`` / ``history_lengths`` (total history after this request) / ``num_candidates``: host
        tensors [B].  ``x_new`` [nnz, d_model]: per user the embeddings of the uncached history tail, then of the
        candidates (the split is whatever the cache says is missing; see :meth:`plan`).  ``timestamps``: optional
        [sum(history + candidates)] per key position.  Returns the candidates' scores, user after user."""
        kv, m, c = self.kv, self.model, self.model.cfg
        H, Dh = c.num_heads, c.head_dim
        hd = H * Dh
        total = (history_lengths + num_candidates).int()
        meta, look = kv.lookup_kvcache(user_ids, total)
        md = kv.allocate_kvcache(meta, look)
        handle = kv.onboard_launch(meta, look, md)
        if handle.status == HostKVTaskStatus.FAILED:
            raise RuntimeError("host prefix could not be brought on board; re-plan the request from token 0")
        assert x_new.shape[0] == md.new_history_nnz, "x_new must hold exactly the uncached tokens (%d)" % md.new_history_nnz
        dev = x_new.device
        nt = num_candidates.to(dev, torch.int32)
        max_q = int((total - look.cached_lengths).max().item())
        x = x_new
        cuda = x.is_cuda
        for li, layer in enumerate(m.layers):
            xn = hstu_ops.ln_mul(x, None, layer.norm_in_w, layer.norm_in_b)
            uvqk = _linear(layer.uvqk, xn, silu=True)
            u, v, q, k = uvqk[:, :hd], uvqk[:, hd:2 * hd], uvqk[:, 2 * hd:3 * hd], uvqk[:, 3 * hd:]
            if handle.layer_events:
                handle.stream_wait_layer(li)
            kv.gpu.append_kvcache(li, k.unflatten(1, (H, Dh)), v.unflatten(1, (H, Dh)), md)
            if cuda:
                a = hstu_attention_paged(q.unflatten(1, (H, Dh)), kv.gpu.cache[li], md.new_history_offsets, md.total_history_offsets,
                                         md.kv_indices, md.kv_indptr, kv.gpu.cfg.page_size, max_q, 1.0 / math.sqrt(Dh),
                                         1.0 / c.max_seq_len, num_target=nt, target_group_size=1, ts=timestamps,
                                         ts_w=layer.ts_w if timestamps is not None else None, ts_divisor=c.time_bucket_divisor,
                                         pos_w=layer.pos_w)
            else:
                a = self._attention_cpu(li, q.unflatten(1, (H, Dh)), md, nt, timestamps, layer)
            y = hstu_ops.ln_mul(a.reshape(-1, hd), u.contiguous(), layer.norm_attn_w, layer.norm_attn_b)
            x = x + _linear(layer.out, y, silu=False)
        h = hstu_ops.ln_mul(x, None, m.norm_out_w, m.norm_out_b)
        # candidates are the last num_candidates[b] query rows of every user
        new_off = md.new_history_offsets.long()
        ends = new_off[1:]
        ncl = nt.long()
        starts = ends - ncl
        seg = torch.repeat_interleave(torch.arange(ncl.numel(), device=dev), ncl, output_size=int(num_candidates.sum()))
        cum = torch.cumsum(ncl, 0) - ncl
        idx = starts[seg] + (torch.arange(seg.numel(), device=dev) - cum[seg])
        hc = h[idx]
        scores = (hc.float() * x_new[idx].float()).sum(-1)             # affinity of the contextualised candidate
        # request-scoped tokens leave the cache; full new history chunks may go to the host tier
        kv.gpu.truncate(meta.user_ids, history_lengths)
        kv.offload_launch(KVIndexMeta(meta.user_ids, history_lengths.cpu().int()), md)
        return scores

    def plan(self, user_ids: torch.Tensor, history_lengths: torch.Tensor) -> torch.Tensor:
        """How many history tokens of each user are already cached (either tier): the caller sends embeddings
        for the rest."""
        _meta, look = self.kv.lookup_kvcache(user_ids, history_lengths.int())
        return torch.minimum(look.cached_lengths, history_lengths.int())

    def _attention_cpu(self, li, q, md, nt, timestamps, layer):
        """Reference math over K/V gathered from the pages (CPU tensors / tests)."""
        cache = self.kv.gpu.cache[li]
        indptr, tl = md.kv_indptr.tolist(), md.total_history_lengths.tolist()
        ks, vs = [], []
        for b in range(len(tl)):
            pages = md.kv_indices[indptr[b]:indptr[b + 1]].long()
            ks.append(cache[pages, 0].reshape(-1, cache.shape[-2], cache.shape[-1])[: tl[b]])
            vs.append(cache[pages, 1].reshape(-1, cache.shape[-2], cache.shape[-1])[: tl[b]])
        c = self.model.cfg
        return hstu_attention_ref(q, torch.cat(ks), torch.cat(vs), md.new_history_offsets, md.total_history_offsets,
                                  1.0 / math.sqrt(c.head_dim), 1.0 / c.max_seq_len, True, None, nt, 1, timestamps,
                                  layer.ts_w if timestamps is not None else None, c.time_bucket_divisor, layer.pos_w)


"""``torch.ops.mxrec.*``: the reference's operator names and argument orders, bound to this library's kernels.

Importing this module registers the schemas (``cust_op/framework/torch_plugin/torch_library/*`` of the reference:
``hstu/hstu_dense.cpp:157-173``, ``hstu/hstu_jagged.cpp:188-246``, ``hstu/hstu_paged.cpp:75-94``,
``in_linear_silu/in_linear_silu.cpp:191-197``, ``relative_attn_bias/*.cpp``, ``ln_mul/ln_mul.cpp:69``,
``norm_multiply_dropout.cpp:180``, ``token_mixing.cpp:63``, ``concat_jagged_tensor.cpp:245-255``,
``multislice_concat.cpp:121``, ``gather_for_rank1.cpp:93-94``, ``reverse_sequence.cpp:85``,
``split_embedding_codegen_forward_unweighted.cpp:123-142``).  ``mask_type``: 0 lower-triangular, 1 upper-triangular
(unsupported, as in the reference), 2 none, 3 custom mask tensor.

The tcgen05 attention kernels evaluate the relative position / time bias themselves; a materialised ``attn_bias``
or a custom ``mask`` tensor is served by the fp32 PyTorch statement of the same math.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import gemm, hstu_ops
from .hstu_attention import hstu_attention, hstu_attention_paged, hstu_attention_ref
from .hstu_attention_bwd import hstu_attn_bwd

_LIB = torch.library.Library("mxrec", "DEF")
_REGISTERED = set()


def _def(schema: str, fn) -> None:
    """Forward ops are registered as composite-implicit so that autograd flows through the differentiable functions
    they call; ops that write into an argument or are themselves backward passes get an explicit kernel."""
    name = schema.split("(")[0]
    if name in _REGISTERED:
        return
    _LIB.define(schema)
    explicit = "backward" in name or "(a!)" in schema
    _LIB.impl(name, fn, "CompositeExplicitAutograd" if explicit else "CompositeImplicitAutograd")
    _REGISTERED.add(name)


# ------------------------------------------------------------------------------------------------ HSTU attention
def _dense_ref(q, k, v, mask, attn_bias, mask_type, silu_scale, alpha=1.0):
    """[B,S,N,D] tensors; fp32 math; returns (out, P-derivative pieces are recomputed by autograd)."""
    B, S, N, D = q.shape
    s = torch.einsum("bind,bjnd->bnij", q.float(), k.float())
    if attn_bias is not None:
        s = s + attn_bias.float()
    scale = silu_scale if silu_scale != 0.0 else 1.0 / S
    p = torch.nn.functional.silu(s * alpha) * scale
    if mask_type == 0:
        p = p * torch.tril(torch.ones(S, k.shape[1], device=q.device))
    elif mask_type == 1:
        raise NotImplementedError("upper-triangular masks are not supported")
    elif mask_type == 3:
        if mask is None:
            raise ValueError("mask_type 3 needs a mask tensor")
        p = p * mask.float()
    return torch.einsum("bnij,bjnd->bind", p.to(q.dtype).float(), v.float()).to(q.dtype)


class _DenseBiasFn(torch.autograd.Function):
    """Dense-layout HSTU attention with the reference's ``attn_bias`` / custom-mask operands: forward on the tcgen05 kernel
    (the bias tile is read beside the S tile, the mask applied to P), gradients - including the bias gradient - from the
    fp32 statement of the same math."""

    @staticmethod
    def forward(ctx, q, k, v, attn_bias, mask, mask_type, scale):
        from .hstu_attention import hstu_attn_fwd

        B, S, N, D = q.shape
        offs = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=q.device)
        out = hstu_attn_fwd(q.reshape(B * S, N, D), k.reshape(B * S, N, D), v.reshape(B * S, N, D), offs, offs, S, 1.0, scale,
                            causal=mask_type == 0, attn_bias=attn_bias, attn_mask=mask if mask_type == 3 else None)
        ctx.save_for_backward(q, k, v, attn_bias if attn_bias is not None else q.new_zeros(0),
                              mask if mask is not None else q.new_zeros(0))
        ctx.meta = (mask_type, scale, attn_bias is not None, mask is not None)
        return out.view(B, S, N, D)

    @staticmethod
    def backward(ctx, grad):
        q, k, v, bias, mask = ctx.saved_tensors
        mask_type, scale, has_b, has_m = ctx.meta
        with torch.enable_grad():
            qq, kk, vv = (t.detach().float().requires_grad_(True) for t in (q, k, v))
            bb = bias.detach().float().requires_grad_(True) if has_b else None
            out = _dense_ref(qq, kk, vv, mask if has_m else None, bb, mask_type, scale)
            gs = torch.autograd.grad(out, [qq, kk, vv] + ([bb] if has_b and ctx.needs_input_grad[3] else []), grad.float())
        db = gs[3].to(bias.dtype) if has_b and ctx.needs_input_grad[3] else None
        return gs[0].to(q.dtype), gs[1].to(k.dtype), gs[2].to(v.dtype), db, None, None, None


def _dense_kernel_ok(q, k, attn_bias, mask, mask_type) -> bool:
    B, S, N, D = q.shape
    if not (q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and k.shape[1] == S and mask_type in (0, 2, 3)):
        return False
    for t in (attn_bias, mask if mask_type == 3 else None):
        if t is not None and (t.dim() != 4 or t.shape[0] != B or t.shape[1] not in (1, N) or t.shape[2] != S or t.shape[3] != S):
            return False
    return not (mask_type == 3 and mask is None)


def hstu_dense(q, k, v, mask=None, attn_bias=None, mask_type: int = 0, max_seq_len: int = 0, silu_scale: float = 0.0):
    B, S, N, D = q.shape
    if (attn_bias is not None or mask_type == 3) and _dense_kernel_ok(q, k, attn_bias, mask, mask_type):
        return _DenseBiasFn.apply(q, k, v, attn_bias, mask, mask_type, silu_scale if silu_scale != 0.0 else 1.0 / S)
    if attn_bias is None and mask_type in (0, 2) and q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and k.shape[1] == S:
        offs = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=q.device)
        out = hstu_attention(q.reshape(B * S, N, D), k.reshape(B * S, N, D), v.reshape(B * S, N, D), offs, max_len_q=S, alpha=1.0,
                             scale=silu_scale if silu_scale != 0.0 else 1.0 / S, causal=mask_type == 0)
        return out.view(B, S, N, D)
    return _dense_ref(q, k, v, mask, attn_bias, mask_type, silu_scale)


def hstu_dense_backward(grad, q, k, v, mask=None, attn_bias=None, mask_type: int = 0, max_seq_len: int = 0, silu_scale: float = 0.0):
    B, S, N, D = q.shape
    if attn_bias is None and mask_type in (0, 2) and q.is_cuda and q.dtype == torch.bfloat16 and D == 64:
        offs = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=q.device)
        dq, dk, dv, _, _ = hstu_attn_bwd(grad.reshape(B * S, N, D), q.reshape(B * S, N, D), k.reshape(B * S, N, D), v.reshape(B * S, N, D),
                                         offs, offs, 1.0, silu_scale if silu_scale != 0.0 else 1.0 / S, mask_type == 0, None, None, 0,
                                         None, None, 1.0, None, max_len_k=S)
        return dq.view_as(q), dk.view_as(k), dv.view_as(v), torch.zeros(0, device=q.device, dtype=q.dtype)
    with torch.enable_grad():
        qq, kk, vv = (t.detach().float().requires_grad_(True) for t in (q, k, v))
        bb = attn_bias.detach().float().requires_grad_(True) if attn_bias is not None else None
        out = _dense_ref(qq, kk, vv, mask, bb, mask_type, silu_scale)
        gs = torch.autograd.grad(out, [qq, kk, vv] + ([bb] if bb is not None else []), grad.float())
    dbias = gs[3].to(q.dtype) if bb is not None else torch.zeros(0, device=q.device, dtype=q.dtype)
    return gs[0].to(q.dtype), gs[1].to(q.dtype), gs[2].to(q.dtype), dbias


def _jagged_common(q, k, v, mask, attn_bias, mask_type, max_seq_len, silu_scale, seq_offset, seq_offset_k, num_context, num_target,
                   target_group_size, alpha):
    if mask_type == 1:
        raise NotImplementedError("upper-triangular masks are not supported")
    # both are optional in the operator schema (None = the default)
    target_group_size, alpha = (0 if target_group_size is None else int(target_group_size)), (1.0 if alpha is None else float(alpha))
    scale = silu_scale if silu_scale != 0.0 else 1.0 / max(max_seq_len, 1)
    if (attn_bias is not None or mask_type == 3) and seq_offset_k is seq_offset and q.is_cuda and q.dtype == torch.bfloat16 \
            and q.shape[2] in (64, 128) and v.shape[2] == q.shape[2] and num_context is None and num_target is None \
            and not (mask_type == 3 and (mask is None or mask.dim() != 4)):
        # the reference's main convention (relative bias passed as attn_bias): forward on the kernel
        return _JaggedBiasFn.apply(q, k, v, attn_bias, mask, mask_type, scale, seq_offset, max_seq_len, alpha)
    if attn_bias is not None or mask_type == 3:
        # remaining combinations (delta queries, context / target masks with a dense bias): padded fp32 path
        return _jagged_ref_bias(q, k, v, mask, attn_bias, mask_type, scale, seq_offset, seq_offset_k, num_context, num_target,
                                target_group_size, alpha)
    return hstu_attention(q, k, v, seq_offset, seq_offset_k, max_len_q=max_seq_len, alpha=alpha, scale=scale, causal=mask_type == 0,
                          num_context=num_context, num_target=num_target, target_group_size=target_group_size)


class _JaggedBiasFn(torch.autograd.Function):
    """Jagged HSTU attention with a padded dense ``attn_bias`` ``[B, N, S_max, S_max]`` and / or custom mask: forward on the
    tcgen05 kernel, gradients from the fp32 statement."""

    @staticmethod
    def forward(ctx, q, k, v, attn_bias, mask, mask_type, scale, offsets, max_seq_len, alpha):
        from .hstu_attention import hstu_attn_fwd

        out = hstu_attn_fwd(q, k, v, offsets, offsets, max_seq_len, alpha, scale, causal=mask_type == 0, attn_bias=attn_bias,
                            attn_mask=mask if mask_type == 3 else None)
        ctx.save_for_backward(q, k, v, attn_bias if attn_bias is not None else q.new_zeros(0),
                              mask if mask is not None else q.new_zeros(0), offsets)
        ctx.meta = (mask_type, scale, alpha, attn_bias is not None, mask is not None)
        return out

    @staticmethod
    def backward(ctx, grad):
        q, k, v, bias, mask, offsets = ctx.saved_tensors
        mask_type, scale, alpha, has_b, has_m = ctx.meta
        with torch.enable_grad():
            qq, kk, vv = (t.detach().float().requires_grad_(True) for t in (q, k, v))
            bb = bias.detach().float().requires_grad_(True) if has_b else None
            out = _jagged_ref_bias(qq, kk, vv, mask if has_m else None, bb, mask_type, scale, offsets, offsets, None, None, 0, alpha)
            want_b = has_b and ctx.needs_input_grad[3]
            gs = torch.autograd.grad(out, [qq, kk, vv] + ([bb] if want_b else []), grad.float())
        return (gs[0].to(q.dtype), gs[1].to(k.dtype), gs[2].to(v.dtype), gs[3].to(bias.dtype) if want_b else None) + (None,) * 6


def _jagged_ref_bias(q, k, v, mask, attn_bias, mask_type, scale, qo, ko, num_context, num_target, gs, alpha):
    from .hstu_attention import hstu_mask

    out = torch.zeros_like(q, dtype=torch.float32)
    ql, kl = qo.tolist(), ko.tolist()
    for b in range(len(ql) - 1):
        lq, lk = ql[b + 1] - ql[b], kl[b + 1] - kl[b]
        if lq == 0:
            continue
        s = torch.einsum("ind,jnd->nij", q[ql[b]:ql[b + 1]].float(), k[kl[b]:kl[b + 1]].float())
        if attn_bias is not None:
            s = s + attn_bias[b, :, :lq, :lk].float()
        p = torch.nn.functional.silu(s * alpha) * scale
        if mask_type == 3:
            m = mask[b, :, :lq, :lk].float() if mask.dim() == 4 else mask[b, :lq, :lk].float()[None]
        else:
            nc = int(num_context[b]) if num_context is not None else 0
            nt = int(num_target[b]) if num_target is not None else 0
            m = hstu_mask(lq, lk, mask_type == 0, nc, nt, gs, q.device)[None]
        p = (p * m).to(q.dtype).float()
        out[ql[b]:ql[b + 1]] = torch.einsum("nij,jnd->ind", p, v[kl[b]:kl[b + 1]].float())
    return out.to(q.dtype)


def hstu_jagged_equal(q, k, v, mask=None, attn_bias=None, mask_type: int = 0, max_seq_len: int = 0, silu_scale: float = 0.0,
                      seq_offset=None, num_context=None, num_target=None, target_group_size: int = 0, alpha: float = 1.0,
                      deterministic: bool = False):
    return _jagged_common(q, k, v, mask, attn_bias, mask_type, max_seq_len, silu_scale, seq_offset, seq_offset, num_context,
                          num_target, target_group_size, alpha)


def hstu_jagged_delta(q, k, v, mask=None, attn_bias=None, mask_type: int = 0, max_seq_len: int = 0, max_seq_len_k: int = 0,
                      silu_scale: float = 0.0, seq_offset=None, seq_offset_k=None, num_context=None, num_target=None,
                      target_group_size: int = 0, alpha: float = 1.0, deterministic: bool = False):
    return _jagged_common(q, k, v, mask, attn_bias, mask_type, max_seq_len, silu_scale, seq_offset, seq_offset_k, num_context,
                          num_target, target_group_size, alpha)


def _jagged_backward(grad, q, k, v, mask, attn_bias, mask_type, max_seq_len, silu_scale, qo, ko, num_context, num_target, gs, alpha):
    gs, alpha = (0 if gs is None else int(gs)), (1.0 if alpha is None else float(alpha))     # both are optional in the schema
    scale = silu_scale if silu_scale != 0.0 else 1.0 / max(max_seq_len, 1)
    if attn_bias is None and mask_type in (0, 2):
        dq, dk, dv, _, _ = hstu_attn_bwd(grad, q, k, v, qo, ko, alpha, scale, mask_type == 0, num_context, num_target, gs, None, None,
                                         1.0, None)
        return dq, dk, dv, torch.zeros(0, device=q.device, dtype=q.dtype)
    with torch.enable_grad():
        qq, kk, vv = (t.detach().float().requires_grad_(True) for t in (q, k, v))
        bb = attn_bias.detach().float().requires_grad_(True) if attn_bias is not None else None
        out = _jagged_ref_bias(qq, kk, vv, mask, bb, mask_type, scale, qo, ko, num_context, num_target, gs, alpha)
        g = torch.autograd.grad(out, [qq, kk, vv] + ([bb] if bb is not None else []), grad.float())
    dbias = g[3].to(q.dtype) if bb is not None else torch.zeros(0, device=q.device, dtype=q.dtype)
    return g[0].to(q.dtype), g[1].to(q.dtype), g[2].to(q.dtype), dbias


def hstu_jagged_backward_equal(grad, q, k, v, mask=None, attn_bias=None, mask_type: int = 0, max_seq_len: int = 0,
                               silu_scale: float = 0.0, seq_offset=None, num_context=None, num_target=None,
                               target_group_size: int = 0, alpha: float = 1.0, deterministic: bool = False):
    return _jagged_backward(grad, q, k, v, mask, attn_bias, mask_type, max_seq_len, silu_scale, seq_offset, seq_offset, num_context,
                            num_target, target_group_size, alpha)


def hstu_jagged_backward_delta(grad, q, k, v, mask=None, attn_bias=None, mask_type: int = 0, max_seq_len: int = 0,
                               max_seq_len_k: int = 0, silu_scale: float = 0.0, seq_offset=None, seq_offset_k=None,
                               num_context=None, num_target=None, target_group_size: int = 0, alpha: float = 1.0,
                               deterministic: bool = False):
    return _jagged_backward(grad, q, k, v, mask, attn_bias, mask_type, max_seq_len, silu_scale, seq_offset, seq_offset_k, num_context,
                            num_target, target_group_size, alpha)


def hstu_paged(q, k, v, kv_cache, mask=None, attn_bias=None, mask_type: int = 0, max_seq_len: int = 0, max_seq_len_k: int = 0,
               silu_scale: float = 0.0, seq_offset=None, seq_offset_k=None, seq_offset_t=None, page_offsets=None, page_ids=None,
               last_page_len=None, num_target=None, target_group_size: int = 0, alpha: float = 1.0, deterministic: bool = False):
    """``q`` / ``k`` / ``v``: the new tokens ``[nnz, N, D]`` (``seq_offset``); ``kv_cache`` ``[pages, 2, page, N, D]``
    holds the history and has room for the new tokens, which are appended here before the attention runs
    (``seq_offset_k``: total key lengths; ``seq_offset_t`` is unused: targets are given by ``num_target``)."""
    page_size = kv_cache.shape[2]
    N, D = q.shape[1], q.shape[2]
    target_group_size, alpha = (0 if target_group_size is None else int(target_group_size)), (1.0 if alpha is None else float(alpha))
    qo, ko = seq_offset.to(torch.int64), seq_offset_k.to(torch.int64)
    lens_q, lens_k = qo[1:] - qo[:-1], ko[1:] - ko[:-1]
    bidx = torch.repeat_interleave(torch.arange(lens_q.numel(), device=q.device), lens_q)
    pos = torch.arange(q.shape[0], device=q.device) - qo[:-1][bidx] + (lens_k - lens_q)[bidx]
    page = page_ids.long()[page_offsets.long()[bidx] + pos // page_size]
    kv_cache[page, 0, pos % page_size] = k
    kv_cache[page, 1, pos % page_size] = v
    scale = silu_scale if silu_scale != 0.0 else 1.0 / max(max_seq_len_k, 1)
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and attn_bias is None and mask_type == 0:
        return hstu_attention_paged(q, kv_cache, seq_offset, seq_offset_k, page_ids, page_offsets, page_size, max_seq_len, alpha, scale,
                                    num_target=num_target, target_group_size=target_group_size)
    ks, vs = [], []
    po = page_offsets.tolist()
    for b in range(lens_k.numel()):
        pg = page_ids[po[b]:po[b + 1]].long()
        ks.append(kv_cache[pg, 0].reshape(-1, N, D)[: int(lens_k[b])])
        vs.append(kv_cache[pg, 1].reshape(-1, N, D)[: int(lens_k[b])])
    return hstu_attention_ref(q, torch.cat(ks), torch.cat(vs), seq_offset, seq_offset_k, alpha, scale, True, None, num_target,
                              target_group_size)


# ------------------------------------------------------------------------------------------------ in_linear_silu
def in_linear_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], attr_dict: List[int]) -> List[torch.Tensor]:
    """``SiLU(x W^T + b)`` split column-wise into ``len(attr_dict)`` tensors (U, V, Q, K for HSTU)."""
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16):
        y = gemm.gemm16(x.contiguous(), weight.contiguous(), bias=None if bias is None else bias.float(), epi=gemm.EPI_SILU)
    else:
        y = torch.nn.functional.silu(torch.nn.functional.linear(x.float(), weight.float(), None if bias is None else bias.float())).to(x.dtype)
    return list(torch.split(y, list(attr_dict), dim=1))


def in_linear_silu_backward(x, weight, bias, user_grad, value_grad, query_grad, key_grad, linear_output, attr_dict: List[int]):
    """-> [dx, dweight, dbias]; ``linear_output`` is the pre-activation ``x W^T + b``."""
    dy = torch.cat([user_grad, value_grad, query_grad, key_grad], dim=1).float()
    z = linear_output.float()
    sg = torch.sigmoid(z)
    dz = dy * (sg * (1 + z * (1 - sg)))
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16):
        dz16 = dz.to(x.dtype)
        dx = gemm.gemm16(dz16, weight.contiguous(), b_mn=True)
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=x.device)
        gemm.gemm16(dz16, x.contiguous(), a_mn=True, b_mn=True, out=dw, epi=gemm.EPI_F32_ATOMIC,
                    splits=gemm.pick_splits(weight.shape[0], weight.shape[1], x.shape[0]))
        dw = dw.to(weight.dtype)
    else:
        dx = (dz @ weight.float()).to(x.dtype)
        dw = (dz.t() @ x.float()).to(weight.dtype)
    db = dz.sum(0).to(bias.dtype) if bias is not None else torch.zeros(0, device=x.device)
    return [dx, dw, db]


# ------------------------------------------------------------------------------------------------ small ops
def relative_attn_bias_time_with_index(timestamps, timestamps_weights, bucket_divisor: float) -> List[torch.Tensor]:
    out, idx = hstu_ops.relative_attn_bias_time(timestamps, timestamps_weights, bucket_divisor, with_index=True)
    return [out, idx]


def norm_multiply_dropout(x, u, weight, bias, eps: float = 1e-5, dropout_ratio: float = 0.0) -> List[torch.Tensor]:
    return [hstu_ops.ln_mul(x, u, weight, bias, eps, dropout_ratio)]


def _jagged_pair_positions(offsets_a, offsets_b, n_prefix: int):
    """Destination row of every row of A and of B in the per-sample layout ``[first n_prefix rows of B | A | rest of B]``
    (``n_prefix`` is clipped to the sample's B length)."""
    oa, ob = offsets_a.long(), offsets_b.long()
    la, lb = oa[1:] - oa[:-1], ob[1:] - ob[:-1]
    B = la.numel()
    dev = oa.device
    base = oa[:-1] + ob[:-1]
    pre = lb.clamp(max=int(n_prefix))
    sa = torch.repeat_interleave(torch.arange(B, device=dev), la)
    ra = torch.arange(int(oa[-1]), device=dev) - oa[:-1][sa]
    sb = torch.repeat_interleave(torch.arange(B, device=dev), lb)
    rb = torch.arange(int(ob[-1]), device=dev) - ob[:-1][sb]
    dst_a = base[sa] + pre[sa] + ra
    dst_b = base[sb] + rb + torch.where(rb < pre[sb], torch.zeros_like(rb), la[sb])
    return dst_a, dst_b


def concat_2d_jagged(maxSeqlen: int, valuesA, valuesB, offsetA, offsetB, isReplace: bool = False, nPrefixFromRight: int = 0):
    """Per sample the rows of A followed by the rows of B; with ``nPrefixFromRight = n`` the first ``n`` rows of B come
    first: ``[B[:n] | A | B[n:]]`` (``concat_2d_jagged/README.md`` of the reference; ``maxSeqlen`` and ``isReplace`` are
    reserved there and have no effect)."""
    if nPrefixFromRight < 0:
        raise ValueError("nPrefixFromRight must not be negative")
    if nPrefixFromRight == 0:
        return hstu_ops.concat_2d_jagged(valuesA, valuesB, offsetA, offsetB)[0]
    dst_a, dst_b = _jagged_pair_positions(offsetA, offsetB, nPrefixFromRight)
    src = torch.cat([valuesA, valuesB])
    order = torch.empty(src.shape[0], dtype=torch.long, device=src.device)
    order[torch.cat([dst_a, dst_b])] = torch.arange(src.shape[0], device=src.device)
    return src.index_select(0, order)


def split_2d_jagged(values, maxSeqlen: int, offsetA, offsetB, dense_size: int = 0, nPrefixToRight: int = 0
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inverse of ``concat_2d_jagged``: -> (A, B); ``nPrefixToRight`` rows at the head of every sample go back to the front
    of B (``dense_size`` is reserved in the reference)."""
    if nPrefixToRight < 0:
        raise ValueError("nPrefixToRight must not be negative")
    if nPrefixToRight == 0:
        return hstu_ops.split_2d_jagged(values, offsetA, offsetB)
    dst_a, dst_b = _jagged_pair_positions(offsetA, offsetB, nPrefixToRight)
    return values.index_select(0, dst_a), values.index_select(0, dst_b)


def multislice_concat(x, concat_num: int, concat_size: List[int], slice_begin: List[int], slice_length: List[int]) -> List[torch.Tensor]:
    """``concat_num`` outputs; output ``i`` is the column-wise concatenation of the next ``concat_size[i]`` slices
    ``x[:, begin:begin + length]`` taken in order from ``slice_begin`` / ``slice_length`` (``multislice_concat/README.md`` of the
    reference).  One gather launch per output on the GPU."""
    concat_size, slice_begin, slice_length = list(concat_size), list(slice_begin), list(slice_length)
    if concat_num != len(concat_size) or sum(concat_size) != len(slice_begin) or len(slice_begin) != len(slice_length):
        raise ValueError("concat_size needs concat_num entries and slice_begin / slice_length one entry per slice")
    D = x.shape[1]
    for b, n in zip(slice_begin, slice_length):
        if b < 0 or n < 1 or b + n > D:
            raise ValueError("slice [%d, %d) is outside the %d columns of the input" % (b, b + n, D))
    out, at = [], 0
    for k in concat_size:
        out.append(hstu_ops.multislice_concat(x, slice_begin[at:at + k], slice_length[at:at + k]))
        at += k
    return out


def index_select_for_rank1_backward(grad, x, index) -> List[torch.Tensor]:
    dx = torch.zeros_like(x, dtype=torch.float32)
    dx.index_add_(0, index.long(), grad.float())
    return [dx.to(x.dtype)]


def split_embedding_codegen_forward_unweighted_cuda(dev_weights, uvm_weights, lxu_cache_weights, weights_placements, weights_offsets,
                                                    D_offsets, total_D: int, max_D: int, indices, offsets, pooling_mode: int,
                                                    lxu_cache_locations, uvm_cache_stats, output_dtype: int, is_experimental: bool,
                                                    hash_indices=None, offset_per_key=None, rows_per_table=None):
    """FBGEMM-TBE-compatible lookup over one flat weight buffer.  ``pooling_mode``: 0 sum, 1 mean, 2 none;
    ``hash_indices``, when given, replace ``indices`` (ids already mapped to rows)."""
    from . import mxrec_tbe as T

    idx = hash_indices if hash_indices is not None else indices
    geo = T._Geometry(dev_weights, weights_offsets, D_offsets, None, rows_per_table)
    out_dtype = {0: torch.float32, 1: torch.float16, 5: torch.bfloat16}.get(int(output_dtype), torch.float32)
    return T._forward(geo, dev_weights, idx, offsets.long(), int(pooling_mode), int(max_D), out_dtype)


_def("hstu_dense(Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? attn_bias=None, int mask_type=0, int max_seq_len=0, "
     "float silu_scale=0.0) -> Tensor", hstu_dense)
_def("hstu_dense_backward(Tensor grad, Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? attn_bias=None, int mask_type=0, "
     "int max_seq_len=0, float silu_scale=0.0) -> (Tensor, Tensor, Tensor, Tensor)", hstu_dense_backward)
_def("hstu_jagged.equal(Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? attn_bias=None, int mask_type=0, int max_seq_len=0, "
     "float silu_scale=0.0, Tensor? seq_offset=None, Tensor? num_context=None, Tensor? num_target=None, int? target_group_size=0, "
     "float? alpha=1.0, bool deterministic=False) -> Tensor", hstu_jagged_equal)
_def("hstu_jagged.delta(Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? attn_bias=None, int mask_type=0, int max_seq_len=0, "
     "int max_seq_len_k=0, float silu_scale=0.0, Tensor? seq_offset=None, Tensor? seq_offset_k=None, Tensor? num_context=None, "
     "Tensor? num_target=None, int? target_group_size=0, float? alpha=1.0, bool deterministic=False) -> Tensor", hstu_jagged_delta)
_def("hstu_jagged_backward.equal(Tensor grad, Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? attn_bias=None, int mask_type=0, "
     "int max_seq_len=0, float silu_scale=0.0, Tensor? seq_offset=None, Tensor? num_context=None, Tensor? num_target=None, "
     "int? target_group_size=0, float? alpha=1.0, bool deterministic=False) -> (Tensor, Tensor, Tensor, Tensor)", hstu_jagged_backward_equal)
_def("hstu_jagged_backward.delta(Tensor grad, Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? attn_bias=None, int mask_type=0, "
     "int max_seq_len=0, int max_seq_len_k=0, float silu_scale=0.0, Tensor? seq_offset=None, Tensor? seq_offset_k=None, "
     "Tensor? num_context=None, Tensor? num_target=None, int? target_group_size=0, float? alpha=1.0, bool deterministic=False) "
     "-> (Tensor, Tensor, Tensor, Tensor)", hstu_jagged_backward_delta)
_def("hstu_paged(Tensor q, Tensor k, Tensor v, Tensor(a!) kv_cache, Tensor? mask=None, Tensor? attn_bias=None, int mask_type=0, "
     "int max_seq_len=0, int max_seq_len_k=0, float silu_scale=0.0, Tensor? seq_offset=None, Tensor? seq_offset_k=None, "
     "Tensor? seq_offset_t=None, Tensor? page_offsets=None, Tensor? page_ids=None, Tensor? last_page_len=None, Tensor? num_target=None, "
     "int? target_group_size=0, float? alpha=1.0, bool deterministic=False) -> Tensor", hstu_paged)
_def("in_linear_silu(Tensor x, Tensor weight, Tensor? bias, int[] attr_dict) -> Tensor[]", in_linear_silu)
_def("in_linear_silu_backward(Tensor x, Tensor weight, Tensor? bias, Tensor user_grad, Tensor value_grad, Tensor query_grad, "
     "Tensor key_grad, Tensor linear_output, int[] attr_dict) -> Tensor[]", in_linear_silu_backward)
_def("relative_attn_bias_pos(Tensor rel_pos_bias, Tensor identity, int[] past_valid_lens) -> Tensor", hstu_ops.relative_attn_bias_pos)
_def("relative_attn_bias_time(Tensor timestamps, Tensor timestamps_weights, float bucket_divisor) -> Tensor",
     lambda t, w, d: hstu_ops.relative_attn_bias_time(t, w, d))
_def("relative_attn_bias_time_with_index(Tensor timestamps, Tensor timestamps_weights, float bucket_divisor) -> Tensor[]",
     relative_attn_bias_time_with_index)
_def("relative_attn_bias_time_backward(Tensor rab_time_grad, Tensor bucket_timestamps, int num_buckets) -> Tensor",
     hstu_ops.relative_attn_bias_time_backward)
_def("ln_mul(Tensor x, Tensor u, Tensor gamma, Tensor beta) -> Tensor", lambda x, u, g, b: hstu_ops.ln_mul(x, u, g, b))
_def("norm_multiply_dropout(Tensor x, Tensor u, Tensor weight, Tensor bias, float eps=1e-05, float dropout_ratio=0.0) -> Tensor[]",
     norm_multiply_dropout)
_def("token_mixing(Tensor x, Tensor gamma, Tensor beta, float epsilon=1e-07) -> Tensor", hstu_ops.token_mixing)
_def("concat_2d_jagged(SymInt maxSeqlen, Tensor valuesA, Tensor valuesB, Tensor offsetA, Tensor offsetB, bool isReplace=False, "
     "SymInt nPrefixFromRight=0) -> Tensor", concat_2d_jagged)
_def("split_2d_jagged(Tensor values, SymInt maxSeqlen, Tensor offsetA, Tensor offsetB, SymInt dense_size=0, SymInt nPrefixToRight=0) "
     "-> (Tensor, Tensor)", split_2d_jagged)
_def("multislice_concat(Tensor input, int concat_num, int[] concat_size, int[] slice_begin, int[] slice_length) -> Tensor[]",
     multislice_concat)
_def("gather_for_rank1(Tensor x, Tensor index) -> Tensor", hstu_ops.gather_for_rank1)
_def("index_select_for_rank1_backward(Tensor grad, Tensor x, Tensor index) -> Tensor[]", index_select_for_rank1_backward)
_def("reverse_sequence(Tensor input, Tensor seq_lengths) -> Tensor", hstu_ops.reverse_sequence)
_def("split_embedding_codegen_forward_unweighted_cuda(Tensor dev_weights, Tensor uvm_weights, Tensor lxu_cache_weights, "
     "Tensor weights_placements, Tensor weights_offsets, Tensor D_offsets, int total_D, int max_D, Tensor indices, Tensor offsets, "
     "int pooling_mode, Tensor lxu_cache_locations, Tensor uvm_cache_stats, int output_dtype, bool is_experimental, "
     "Tensor? hash_indices=None, Tensor? offset_per_key=None, Tensor? rows_per_table=None) -> Tensor",
     split_embedding_codegen_forward_unweighted_cuda)


# ------------------------------------------------------------------------------------------------ optional parity ops
def _fuxi_kernels(q, k, v, tsb, pob, mask, mask_type: int, scale: float, offs: List[int], max_len: int):
    """Fuxi forward on this library's kernels, ``q/k/v`` ``[T, N, D]`` bf16 with sequence offsets ``offs``: the SiLU part on
    the tcgen05 attention kernel (causal flag or custom mask in the kernel), the two bias parts as masked-bias x V GEMMs on
    the tcgen05 GEMM (one per sequence; per head when the custom mask differs between heads)."""
    from .gemm import gemm16
    from .hstu_attention import hstu_attn_fwd

    T, N, D = q.shape
    dev = q.device
    offsets = torch.tensor(offs, dtype=torch.int32, device=dev)
    part1 = hstu_attn_fwd(q, k, v, offsets, offsets, max_len, 1.0, scale, causal=mask_type == 0,
                          attn_mask=mask if mask_type == 3 else None)
    if tsb is None and pob is None:
        return part1
    out = torch.empty(T, N, 3 * D, dtype=q.dtype, device=dev)
    out[:, :, :D] = part1
    vf = v.reshape(T, N * D)
    for b in range(len(offs) - 1):
        lo, L = offs[b], offs[b + 1] - offs[b]
        if L == 0:
            continue
        Lp = (L + 7) // 8 * 8
        for part, bias in ((1, tsb), (2, pob)):
            dst = out[lo:lo + L, :, part * D:(part + 1) * D]
            if bias is None:
                dst.zero_()
                continue
            bm = bias[min(b, bias.shape[0] - 1), :L, :L]
            per_head = mask_type == 3 and mask.shape[1] > 1
            heads = range(N) if per_head else (None,)
            for h in heads:
                a = torch.zeros(L, Lp, dtype=q.dtype, device=dev)              # row stride a multiple of 16 bytes for TMA
                if mask_type == 0:
                    a[:, :L] = torch.tril(bm)
                elif mask_type == 3:
                    a[:, :L] = bm * mask[b, h if per_head else 0, :L, :L].to(bm.dtype)
                else:
                    a[:, :L] = bm
                if per_head:
                    dst[:, h, :] = gemm16(a[:, :L], v[lo:lo + L, h, :], b_mn=True)
                else:
                    dst.copy_(gemm16(a[:, :L], vf[lo:lo + L], b_mn=True).view(L, N, D))
    return out


class _FuxiFn(torch.autograd.Function):
    """Kernel forward; gradients from the fp32 statement (``_fuxi_ref``)."""

    @staticmethod
    def forward(ctx, q, k, v, tsb, pob, mask, mask_type, scale, offs, max_len):
        ctx.save_for_backward(q, k, v, *(t if t is not None else q.new_zeros(0) for t in (tsb, pob, mask)))
        ctx.meta = (mask_type, scale, offs, tsb is not None, pob is not None, mask is not None)
        return _fuxi_kernels(q, k, v, tsb, pob, mask, mask_type, scale, offs, max_len)

    @staticmethod
    def backward(ctx, grad):
        q, k, v, tsb, pob, mask = ctx.saved_tensors
        mask_type, scale, offs, has_t, has_p, has_m = ctx.meta
        with torch.enable_grad():
            leaves = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
            tb = tsb.detach().float().requires_grad_(True) if has_t else None
            pb = pob.detach().float().requires_grad_(True) if has_p else None
            out = _fuxi_ref(leaves[0], leaves[1], leaves[2], tb, pb, mask if has_m else None, mask_type, scale, "jagged", offs)
            wanted = leaves + [t for t in (tb, pb) if t is not None]
            gs = list(torch.autograd.grad(out, wanted, grad.float()))
        dq, dk, dv = (g.to(q.dtype) for g in gs[:3])
        rest = gs[3:]
        dt = rest.pop(0).to(tsb.dtype) if has_t else None
        dp = rest.pop(0).to(pob.dtype) if has_p else None
        return dq, dk, dv, dt, dp, None, None, None, None, None


def hstu_fuxi(q, k, v, timestampBias=None, positionBias=None, mask=None, maskType: int = 0, maxSeqLen: int = 0, siluScale: float = 0.0,
              layout: str = "normal", seqOffset: Optional[List[int]] = None):
    """Fuxi variant: ``cat[(SiLU(QK^T) s m) V, (tsBias m) V, (posBias m) V]`` on the last dim (only the first part when no
    bias is given).  ``layout`` "normal": ``[B,S,N,D]``; "jagged": ``[sum_len,N,D]`` with ``seqOffset``
    (``hstu_dense_forward_fuxi/README.md`` of the reference).  bf16 CUDA inputs with head dim 64 / 128 run on the tcgen05
    attention and GEMM kernels; everything else on the fp32 PyTorch statement."""
    if maskType == 1:
        raise NotImplementedError("upper-triangular masks are not supported")
    scale = siluScale if siluScale != 0.0 else 1.0 / max(maxSeqLen, 1)
    D = q.shape[-1]
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and v.shape[-1] == D and (q.shape[-2] * D) % 8 == 0 \
            and not (maskType == 3 and (mask is None or mask.dim() != 4)) \
            and all(t is None or t.dtype == q.dtype for t in (timestampBias, positionBias)):
        if layout == "jagged":
            offs = [int(x) for x in seqOffset]
            return _FuxiFn.apply(q.contiguous(), k.contiguous(), v.contiguous(), timestampBias, positionBias, mask, maskType, scale,
                                 offs, max(maxSeqLen, max(b - a for a, b in zip(offs, offs[1:]))))
        B, S, N, _ = q.shape
        offs = [i * S for i in range(B + 1)]
        out = _FuxiFn.apply(q.reshape(B * S, N, D), k.reshape(B * S, N, D), v.reshape(B * S, N, D), timestampBias, positionBias, mask,
                            maskType, scale, offs, S)
        return out.view(B, S, N, -1)
    return _fuxi_ref(q, k, v, timestampBias, positionBias, mask, maskType, scale, layout, seqOffset)


def _fuxi_ref(q, k, v, timestampBias, positionBias, mask, maskType: int, scale: float, layout: str, seqOffset):
    """The fuxi statement in fp32 PyTorch ops (oracle of the kernel path and its gradient)."""

    def one(qq, kk, vv, b):                                        # [L,N,D] each
        L = qq.shape[0]
        s = torch.einsum("ind,jnd->nij", qq.float(), kk.float())
        if maskType == 0:
            m = torch.tril(torch.ones(L, L, device=qq.device))[None]
        elif maskType == 3:
            m = mask[b, :, :L, :L].float()
        else:
            m = torch.ones(1, L, L, device=qq.device)
        parts = [torch.einsum("nij,jnd->ind", torch.nn.functional.silu(s) * scale * m, vv.float())]
        if timestampBias is not None or positionBias is not None:
            tb = timestampBias[b, :L, :L].float()[None] if timestampBias is not None else torch.zeros(1, L, L, device=qq.device)
            pb = positionBias[min(b, positionBias.shape[0] - 1), :L, :L].float()[None] if positionBias is not None \
                else torch.zeros(1, L, L, device=qq.device)
            parts.append(torch.einsum("nij,jnd->ind", (tb * m).expand(qq.shape[1], L, L), vv.float()))
            parts.append(torch.einsum("nij,jnd->ind", (pb * m).expand(qq.shape[1], L, L), vv.float()))
        return torch.cat(parts, dim=-1).to(qq.dtype)

    if layout == "jagged":
        offs = list(seqOffset)
        return torch.cat([one(q[offs[b]:offs[b + 1]], k[offs[b]:offs[b + 1]], v[offs[b]:offs[b + 1]], b) for b in range(len(offs) - 1)])
    return torch.stack([one(q[b], k[b], v[b], b) for b in range(q.shape[0])])


def hstu_dense_backward_fuxi(grad, q, k, v, mask=None, biasPosition=None, biasTimestamp=None, layout: str = "jagged", maskType: int = 0,
                             maxSeqLen: int = 0, siluScale: float = 0.0, seqOffset: Optional[List[int]] = None):
    """Backward of ``hstu_fuxi`` in the jagged layout (``hstu_dense_backward_fuxi/HstuDenseNpuFusionFuxi.cpp:161-164`` of the
    reference): ``grad`` is ``[sum_len, N, D]`` or, with biases, ``[sum_len, N, 3D]`` (SiLU part, timestamp part, position part).
    -> ``(dq, dk, dv, d_biasPosition, d_biasTimestamp)``; the bias gradients are summed over the heads (and over the batch for a
    position bias shared by the batch), empty tensors when no bias was given.  fp32 autograd over the statement of the forward."""
    if layout != "jagged":
        raise ValueError("hstu_dense_backward_fuxi supports the jagged layout only")
    if seqOffset is None:
        raise ValueError("the jagged layout needs seqOffset")
    if maskType == 1:
        raise NotImplementedError("upper-triangular masks are not supported")
    if maskType == 3 and mask is None:
        raise ValueError("maskType 3 (custom) needs a mask")
    scale = siluScale if siluScale != 0.0 else 1.0 / max(maxSeqLen, 1)
    with torch.enable_grad():
        leaves = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
        tb = biasTimestamp.detach().float().requires_grad_(True) if biasTimestamp is not None else None
        pb = biasPosition.detach().float().requires_grad_(True) if biasPosition is not None else None
        out = _fuxi_ref(leaves[0], leaves[1], leaves[2], tb, pb, mask, maskType, scale, "jagged", [int(x) for x in seqOffset])
        if out.shape != grad.shape:
            raise ValueError("grad has shape %s, the forward output %s" % (tuple(grad.shape), tuple(out.shape)))
        wanted = leaves + [t for t in (pb, tb) if t is not None]
        gs = list(torch.autograd.grad(out, wanted, grad.float()))
    dq, dk, dv = (g.to(q.dtype) for g in gs[:3])
    rest = gs[3:]
    dp = rest.pop(0).to(biasPosition.dtype) if pb is not None else q.new_zeros(0)
    dt = rest.pop(0).to(biasTimestamp.dtype) if tb is not None else q.new_zeros(0)
    return dq, dk, dv, dp, dt


class _DisentangleFn(torch.autograd.Function):
    """CUDA forward: the four products are plain (library) GEMMs in the input dtype, everything between them - both
    relative-position gathers, scale, mask, softmax, the two matrix outputs - is one pass of ``rb_disentangle_softmax``.
    Gradients come from the fp32 statement."""

    @staticmethod
    def forward(ctx, q, k, v, pos_k, pos_q, rel, mask, kinds, scale):
        from . import _lib

        B, N, S, _ = q.shape
        P = pos_k.shape[0]
        qk = torch.matmul(q, k.transpose(-1, -2)).contiguous()
        c2p = torch.matmul(q, pos_k.permute(1, 2, 0).to(q.dtype)).contiguous() if "c2p" in kinds else None      # [B,N,S,P]
        p2c = torch.matmul(k, pos_q.permute(1, 2, 0).to(q.dtype)).contiguous() if "p2c" in kinds else None
        rel2 = rel.reshape(S, S).long().contiguous()
        m8 = (mask != 0).to(torch.uint8).reshape(-1, S, S).contiguous()
        probs, score = torch.empty_like(qk), torch.empty_like(qk)
        rc = _lib.lib().rb_disentangle_softmax(qk.data_ptr(), _lib.ptr(c2p), _lib.ptr(p2c), rel2.data_ptr(), m8.data_ptr(),
                                               S * S if m8.shape[0] == B else 0, B, N, S, P, P // 2, float(scale),
                                               _lib.dtype_code(q.dtype), probs.data_ptr(), score.data_ptr(),
                                               _lib.stream_ptr(q.device))
        _lib.check(rc, "rb_disentangle_softmax")
        out = torch.matmul(probs, v)
        ctx.save_for_backward(q, k, v, pos_k, pos_q, rel, mask)
        ctx.meta = (kinds, scale)
        return out, probs, score

    @staticmethod
    def backward(ctx, g_out, g_probs, g_score):
        q, k, v, pos_k, pos_q, rel, mask = ctx.saved_tensors
        kinds, scale = ctx.meta
        with torch.enable_grad():
            leaves = [t.detach().float().requires_grad_(True) for t in (q, k, v, pos_k, pos_q)]
            outs = _disentangle_ref(*leaves, rel, mask, kinds, scale)
            gs = torch.autograd.grad(outs, leaves, [g.float() for g in (g_out, g_probs, g_score)], allow_unused=True)
        cast = [None if g is None else g.to(t.dtype) for g, t in zip(gs, (q, k, v, pos_k, pos_q))]
        return cast[0], cast[1], cast[2], cast[3], cast[4], None, None, None, None


def disentangle_attention(query_layer, key_layer, value_layer, pos_key_layer, pos_query_layer, relative_pos, attn_mask,
                          pos_attr_type: str, score_scale: float):
    """DeBERTa disentangled attention; CUDA tensors run the fused gather / mask / softmax kernel between plain GEMMs, CPU
    tensors the fp32 statement (``_disentangle_ref``, same contract)."""
    if query_layer.is_cuda and query_layer.dtype in (torch.float32, torch.float16, torch.bfloat16) \
            and key_layer.shape == query_layer.shape and relative_pos.numel() == query_layer.shape[2] ** 2 \
            and attn_mask.numel() in (query_layer.shape[2] ** 2, query_layer.shape[0] * query_layer.shape[2] ** 2):
        return _DisentangleFn.apply(query_layer, key_layer, value_layer, pos_key_layer, pos_query_layer, relative_pos, attn_mask,
                                    pos_attr_type, score_scale)
    return _disentangle_ref(query_layer, key_layer, value_layer, pos_key_layer, pos_query_layer, relative_pos, attn_mask,
                            pos_attr_type, score_scale)


def _disentangle_ref(query_layer, key_layer, value_layer, pos_key_layer, pos_query_layer, relative_pos, attn_mask,
                     pos_attr_type: str, score_scale: float):
    """DeBERTa disentangled attention.  ``query/key/value`` ``[b,n,s,d]``, ``pos_key/pos_query`` ``[2s,n,d]``, ``relative_pos``
    ``[1,1,s,s]`` int64, ``attn_mask`` ``[b,1,s,s]``; ``pos_attr_type`` in ``c2p``, ``p2c``, ``c2p|p2c``.
    Returns ``(outputs, probs, weights)`` where ``weights`` is the pre-softmax score (content + position terms)
    (``ai_core_op/disentangle_attention/v220/README.md`` of the reference).  PyTorch composition (fp32 math)."""
    q, k, v = query_layer.float(), key_layer.float(), value_layer.float()
    span = pos_key_layer.shape[0] // 2
    score = torch.matmul(q, k.transpose(-1, -2)) * score_scale
    rel = relative_pos.long()
    kinds = pos_attr_type.split("|")
    if "c2p" in kinds:
        c2p_att = torch.einsum("bnqd,pnd->bnqp", q, pos_key_layer.float())
        c2p_pos = torch.clamp(rel + span, 0, 2 * span - 1).expand(q.shape[0], q.shape[1], -1, -1)
        score = score + torch.gather(c2p_att, -1, c2p_pos) * score_scale
    if "p2c" in kinds:
        p2c_att = torch.einsum("bnkd,pnd->bnkp", k, pos_query_layer.float())
        p2c_pos = torch.clamp(-rel + span, 0, 2 * span - 1).expand(q.shape[0], q.shape[1], -1, -1)
        score = score + torch.gather(p2c_att, -1, p2c_pos).transpose(-1, -2) * score_scale
    keep = attn_mask.bool()
    probs = torch.softmax(score.masked_fill(~keep, float("-inf")), dim=-1)
    probs = torch.nan_to_num(probs).masked_fill(~keep, 0.0)
    out = torch.matmul(probs, v)
    dt = query_layer.dtype
    return out.to(dt), probs.to(dt), score.to(dt)


_def("hstu_fuxi(Tensor q, Tensor k, Tensor v, Tensor? timestampBias=None, Tensor? positionBias=None, Tensor? mask=None, int maskType=0, "
     "int maxSeqLen=0, float siluScale=0.0, str layout=\"normal\", int[]? seqOffset=None) -> Tensor", hstu_fuxi)
_def("hstu_dense_backward_fuxi(Tensor grad, Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? biasPosition=None, "
     "Tensor? biasTimestamp=None, str layout=\"jagged\", int maskType=0, int maxSeqLen=0, float siluScale=0.0, int[]? seqOffset=None) "
     "-> (Tensor, Tensor, Tensor, Tensor, Tensor)", hstu_dense_backward_fuxi)
_def("disentangle_attention(Tensor query_layer, Tensor key_layer, Tensor value_layer, Tensor pos_key_layer, Tensor pos_query_layer, "
     "Tensor relative_pos, Tensor attn_mask, str pos_attr_type, float score_scale) -> (Tensor, Tensor, Tensor)", disentangle_attention)


# ------------------------------------------------------------------------------------------------ row IO by address, sparse optimizers
from . import by_address as _by_address  # noqa: E402

_def("embedding_lookup_by_address(Tensor address, int embedding_dim, Tensor region) -> Tensor",
     lambda address, embedding_dim, region: _by_address.embedding_lookup_by_address(address, embedding_dim, region))
_def("embedding_update_by_address(Tensor address, Tensor embedding, int update_type, Tensor(a!) region) -> ()",
     lambda address, embedding, update_type, region: _by_address.embedding_update_by_address(address, embedding, update_type, region))
_def("lazy_adam(Tensor gradient, Tensor indices, Tensor(a!) input_m, Tensor(b!) input_v, Tensor(c!) input_var, float lr, "
     "float beta1=0.9, float beta2=0.999, float epsilon=1e-08) -> ()",
     lambda gradient, indices, input_m, input_v, input_var, lr, beta1=0.9, beta2=0.999, epsilon=1e-8:
     (_by_address.lazy_adam(gradient, indices, input_m, input_v, input_var, lr, beta1, beta2, epsilon), None)[1])
_def("sgd(Tensor gradient, Tensor indices, Tensor(a!) input_var, float lr, float weightDecay=0.0) -> ()",
     lambda gradient, indices, input_var, lr, weightDecay=0.0:
     (_by_address.sgd(gradient, indices, input_var, lr, weightDecay), None)[1])


# ------------------------------------------------------------------------------------------------ TBE training lookups
def _def_autograd(name: str, schema_args: str, ret: str, fn) -> None:
    """Ops whose implementation builds its own autograd node: the same function serves the Autograd key and the backends."""
    if name in _REGISTERED:
        return
    _LIB.define(f"{name}({schema_args}) -> {ret}")
    _LIB.impl(name, fn, "Autograd")
    _LIB.impl(name, fn, "CompositeExplicitAutograd")
    _REGISTERED.add(name)


from . import mxrec_tbe as _tbe  # noqa: E402

for _name, (_kind, _args) in _tbe.lookup_schemas().items():
    _def_autograd(_name, _args, "Tensor", _tbe.make_lookup(_kind, _args))
for _name, (_kind, _args) in _tbe.raw_backward_schemas().items():
    _def(f"{_name}({_args}) -> Tensor", _tbe.make_raw_backward(_kind, _args))


# ------------------------------------------------------------------------------------------------ v2 attention / distance variant
def hstu_forward_v2(q, k, v, mask, rab, mask_type: int, max_seq_len: int, max_seq_len_k: Optional[int], silu_scale: Optional[float],
                    seq_offset, seq_offset_k, num_context, num_target, target_group_size: Optional[int], alpha: Optional[float]):
    """The second-generation jagged attention entry (``hstu_v2/hstu_forward_v2.cpp:72``): same math as ``hstu_jagged``; ``rab`` is
    the materialised bias, ``silu_scale`` 0 / None means ``1 / max_seq_len``."""
    return _jagged_common(q, k, v, mask, rab, mask_type, max_seq_len, silu_scale or 0.0, seq_offset,
                          seq_offset if seq_offset_k is None else seq_offset_k, num_context, num_target, target_group_size or 0,
                          1.0 if alpha is None else alpha)


def hstu_backward_v2(grad, q, k, v, max_seqlen_q: int, max_seqlen_k: int, seq_offset_q, seq_offset_k, rab=None, num_context=None,
                     num_target=None, scale: Optional[float] = 0.0, target_group_size: Optional[int] = 1, alpha: Optional[float] = 1.0,
                     window_size_left: int = -1, window_size_right: int = -1):
    """``(dq, dk, dv, drab)`` of the v2 attention (``hstu_v2/hstu_backward_v2.cpp:82``).  The window pair selects the mask:
    ``(-1, 0)`` causal, ``(-1, -1)`` none; other windows are rejected, as no forward produces them."""
    if (window_size_left, window_size_right) not in ((-1, 0), (-1, -1)):
        raise NotImplementedError("sliding windows other than causal (-1, 0) and full (-1, -1) are not supported")
    mask_type = 0 if window_size_right == 0 else 2
    return _jagged_backward(grad, q, k, v, None, rab, mask_type, max_seqlen_q, scale or 0.0, seq_offset_q, seq_offset_k, num_context,
                            num_target, target_group_size or 0, 1.0 if alpha is None else alpha)


def distance_in_linear_silu(x, weight, bias, attr_dict: List[int]) -> List[torch.Tensor]:
    """Forward of ``in_linear_silu`` that also returns the pre-activation ``x W^T + b`` as a fifth tensor, which the
    stand-alone backward op consumes (``in_linear_silu/in_linear_silu.cpp:96-118``)."""
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16):
        z = gemm.gemm16(x.contiguous(), weight.contiguous(), bias=None if bias is None else bias.float())
    else:
        z = torch.nn.functional.linear(x.float(), weight.float(), None if bias is None else bias.float()).to(x.dtype)
    y = torch.nn.functional.silu(z.float()).to(x.dtype)
    return list(torch.split(y, list(attr_dict), dim=1)) + [z]


_def("hstu_forward_v2(Tensor q, Tensor k, Tensor v, Tensor? mask, Tensor? rab, int mask_type, int max_seq_len, int? max_seq_len_k, "
     "float? silu_scale, Tensor seq_offset, Tensor? seq_offset_k, Tensor? num_context, Tensor? num_target, int? target_group_size, "
     "float? alpha) -> Tensor", hstu_forward_v2)
_def("hstu_backward_v2(Tensor grad, Tensor q, Tensor k, Tensor v, int max_seqlen_q, int max_seqlen_k, Tensor seq_offset_q, "
     "Tensor seq_offset_k, Tensor? rab=None, Tensor? num_context=None, Tensor? num_target=None, float? scale=0.0, "
     "int? target_group_size=1, float? alpha=1.0, int window_size_left=-1, int window_size_right=-1) "
     "-> (Tensor, Tensor, Tensor, Tensor)", hstu_backward_v2)
_def("distance_in_linear_silu(Tensor x, Tensor weight, Tensor bias, int[] attr_dict) -> Tensor[]", distance_in_linear_silu)

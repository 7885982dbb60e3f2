"""Stock-PyTorch statements of the HSTU training step and of HSTU ranking inference over a paged KV cache: the
comparison arms of the benchmark.  Nothing here touches this repository's kernels or engine: matmuls are
cuBLAS through ``torch.einsum`` / ``nn.Linear`` in bf16, the SiLU attention with relative position / time bias is
written with elementwise torch ops per sequence, the item table is ``nn.Embedding(sparse=True)`` over hashed ids
with SparseAdam, paged K/V are gathered with ``index_select``.
"""
from __future__ import annotations

import json
import math
import os

import torch
import torch.distributed as dist
from torch import nn

H, DH, DM, LAYERS, NB, DIV = 8, 64, 512, 8, 128, 0.301


def _bias(ts_q, ts_k, pos_q, pos_k, ts_w, pos_w):
    dt = (ts_q[:, None] - ts_k[None, :]).abs().clamp(1.0, 7.0e16)
    bk = torch.clamp(torch.floor(torch.log(dt) / DIV), 0, NB).long()
    d = (pos_q[:, None] - pos_k[None, :]).clamp(0, pos_w.numel() - 1)
    return ts_w[bk] + pos_w[d]


class Layer(nn.Module):
    def __init__(self, dev, max_len=4096):
        super().__init__()
        self.n1 = nn.LayerNorm(DM, device=dev)
        self.uvqk = nn.Linear(DM, 4 * H * DH, device=dev)
        self.n2 = nn.LayerNorm(H * DH, device=dev)
        self.out = nn.Linear(H * DH, DM, device=dev)
        self.ts_w = nn.Parameter(torch.randn(NB + 1, device=dev) * 0.02)
        self.pos_w = nn.Parameter(torch.randn(max_len, device=dev) * 0.02)

    def project(self, x):
        y = torch.nn.functional.silu(self.uvqk(self.n1(x)))
        u, v, q, k = y.split(H * DH, dim=1)
        return u, v.unflatten(1, (H, DH)), q.unflatten(1, (H, DH)), k.unflatten(1, (H, DH))

    def finish(self, x, a, u):
        return x + self.out(self.n2(a.flatten(1)) * u)

    def forward(self, x, offsets, ts, scale):
        u, v, q, k = self.project(x)
        outs = []
        for b in range(len(offsets) - 1):
            s0, s1 = offsets[b], offsets[b + 1]
            L = s1 - s0
            pos = torch.arange(L, device=x.device)
            s = torch.einsum("ihd,jhd->hij", q[s0:s1], k[s0:s1])
            s = s + _bias(ts[s0:s1], ts[s0:s1], pos, pos, self.ts_w, self.pos_w).to(s.dtype)
            p = torch.nn.functional.silu(s * (1.0 / math.sqrt(DH))) * scale
            p = p * torch.tril(torch.ones(L, L, device=x.device, dtype=p.dtype))
            outs.append(torch.einsum("hij,jhd->ihd", p, v[s0:s1]))
        return self.finish(x, torch.cat(outs), u)


class TorchHSTU(nn.Module):
    def __init__(self, dev, table_rows=1 << 22):
        super().__init__()
        self.rows = table_rows
        self.emb = nn.Embedding(table_rows, DM, sparse=True, device=dev)
        self.layers = nn.ModuleList([Layer(dev) for _ in range(LAYERS)])
        self.norm = nn.LayerNorm(DM, device=dev)

    def forward(self, items, negs, offsets, ts, max_len):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            x0 = self.emb(items % self.rows).to(torch.bfloat16)
            neg = self.emb(negs % self.rows).to(torch.bfloat16)
            x = x0
            for layer in self.layers:
                x = layer(x, offsets, ts, 1.0 / max_len)
            h = self.norm(x)
        T = x0.shape[0]
        last = torch.zeros(T, dtype=torch.bool, device=x0.device)
        last[torch.tensor(offsets[1:], device=x0.device) - 1] = True
        keep = (~last).nonzero(as_tuple=True)[0]
        hq, pos = h[keep].float(), x0[keep + 1].float()
        pl = (hq * pos).sum(-1, keepdim=True)
        logits = torch.cat([pl, hq @ neg.float().t()], dim=1)
        return (torch.logsumexp(logits, 1) - pl.squeeze(1)).sum() / max(keep.numel(), 1)


def _make_batch(B, gen, max_len=4096, n_items=100_000_000):
    lens = torch.exp(torch.randn(B, generator=gen) * 0.9 + math.log(1024) - 0.405).clamp(16, max_len).long()
    T = int(lens.sum())
    u = torch.rand(T, generator=gen, dtype=torch.float64)
    a = 1.05
    items = (((n_items ** (1 - a) - 1) * u + 1) ** (1 / (1 - a))).floor().clamp(1, n_items).long() - 1
    offsets = [0]
    for n in lens.tolist():
        offsets.append(offsets[-1] + n)
    gaps = torch.empty(T).exponential_(1 / 3600.0, generator=gen)
    ts = torch.cat([torch.cumsum(gaps[offsets[b]:offsets[b + 1]], 0) for b in range(B)])
    negs = torch.randint(0, n_items, (512,), generator=gen)
    return items.pin_memory(), negs.pin_memory(), offsets, ts.pin_memory(), int(lens.max()), T


def _finish(args, ClockSampler, dev, world, rank, step_fn, unit_count, metric, unit, config, h2d, d2h, extra=None):
    W = max(args.warmup, 3)
    for i in range(W):
        step_fn(i)
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    torch.cuda.synchronize(dev)
    lat, total = [], 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        total += step_fn(W + i)
        b.record()
        b.synchronize()
        lat.append(a.elapsed_time(b))
    e1.record()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    t = torch.tensor([ms, total], dtype=torch.float64, device=dev)
    if world > 1:
        tm, tsum = t.clone(), t.clone()
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum)
        ms, total = float(tm[0]), float(tsum[1])
    if rank == 0:
        lat.sort()
        val = total / (ms / 1e3)
        out = {"metric": metric, "value": val, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": W,
               "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 autocast",
               "data": "synthetic, random-init weights", "config": config,
               "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
               "gpu_launches": 0, "clocks": clocks, "impl": "torch-nccl-baseline"}
        if extra:
            out.update(extra(lat))
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def run(args, ClockSampler):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    model = TorchHSTU(dev, (1 << 22) if not args.small else (1 << 16))
    dense = [p for n, p in model.named_parameters() if not n.startswith("emb.")]
    opt = torch.optim.Adam(dense, lr=1e-3, fused=True)
    sopt = torch.optim.SparseAdam(list(model.emb.parameters()), lr=1e-3)
    gen = torch.Generator().manual_seed(1234 + rank)
    B = 32 if not args.small else 4
    host = [_make_batch(B, gen, 4096 if not args.small else 512) for _ in range(min(args.steps + 3, 12))]

    def step(i):
        items, negs, offsets, ts, max_len, T = host[i % len(host)]
        it, ng, td = items.to(dev, non_blocking=True), negs.to(dev, non_blocking=True), ts.to(dev, non_blocking=True)
        opt.zero_grad()
        sopt.zero_grad()
        loss = model(it, ng, offsets, td, max_len)
        loss.backward()
        if world > 1:
            for p in dense:
                dist.all_reduce(p.grad)
                p.grad /= world
        opt.step()
        sopt.step()
        float(loss.item())
        return T

    items, negs, offsets, ts, _, _ = host[0]
    _finish(args, ClockSampler, dev, world, rank, step, None, "HSTU train tokens/sec", "tokens/s",
            {"model": "HSTU 8L d512 8x64", "global_batch": B * world, "seq_len": "lognormal[16,4096] mean~1024",
             "parallelism": "dp%d, torch ops + cuBLAS + NCCL all_reduce; hashed nn.Embedding(sparse) table" % world, "negatives": 512},
            int(items.numel() * 8 + negs.numel() * 8 + ts.numel() * 4) * world, 4 * world)


@torch.no_grad()
def run_inference(args, ClockSampler):
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    small = args.small
    users, cached, new, cands, page = (64, 2048, 128, 1024, 64) if not small else (4, 256, 64, 32, 64)
    layers_n = LAYERS if not small else 2
    torch.manual_seed(0)
    layers = nn.ModuleList([Layer(dev) for _ in range(layers_n)]).to(torch.bfloat16)
    norm = nn.LayerNorm(DM, device=dev, dtype=torch.bfloat16)
    n_items = 4_000_000 if not small else 100_000
    table = (torch.randn(n_items, DM, device=dev) * 0.05).to(torch.bfloat16)
    total = cached + new + cands
    ppu = (total + page - 1) // page
    cache = torch.zeros(layers_n, users * ppu, 2, page, H, DH, dtype=torch.bfloat16, device=dev)
    page_ids = torch.arange(users * ppu, device=dev).view(users, ppu)
    gen = torch.Generator().manual_seed(7)
    hist_ts = torch.cumsum(torch.empty(users, cached).exponential_(1 / 300.0, generator=gen), 1)
    scale = 1.0 / 4096

    def slots(start, n):                                            # (page, slot) of token positions [start, start + n) of every user
        pos = torch.arange(start, start + n, device=dev)
        return page_ids[:, pos // page], (pos % page)[None, :].expand(users, n)

    def forward(x, ts_all, start, n_new, n_cand):
        """x [users, n, DM]: tokens at positions [start, start + n); keys = everything up to start + n."""
        n = x.shape[1]
        klen = start + n
        pg, sl = slots(start, n)
        kpg = page_ids[:, : (klen + page - 1) // page]
        pos_q = torch.arange(start, klen, device=dev)
        pos_k = torch.arange(klen, device=dev)
        mask = pos_k[None, :] <= pos_q[:, None]
        if n_cand:                                                  # candidates: history plus themselves only
            cq, ck = pos_q >= klen - n_cand, pos_k >= klen - n_cand
            mask = torch.where(cq[:, None] & ck[None, :], pos_q[:, None] == pos_k[None, :], mask)
        for li, layer in enumerate(layers):
            u, v, q, k = layer.project(x.reshape(-1, DM))
            cache[li, pg, 0, sl] = k.view(users, n, H, DH)
            cache[li, pg, 1, sl] = v.view(users, n, H, DH)
            kv = cache[li].index_select(0, kpg.reshape(-1)).view(users, -1, 2, page, H, DH)
            K = kv[:, :, 0].reshape(users, -1, H, DH)[:, :klen]
            V = kv[:, :, 1].reshape(users, -1, H, DH)[:, :klen]
            s = torch.einsum("bihd,bjhd->bhij", q.view(users, n, H, DH), K)
            dt = (ts_all[:, start:klen, None] - ts_all[:, None, :klen]).abs().clamp(1.0, 7.0e16)
            bk = torch.clamp(torch.floor(torch.log(dt) / DIV), 0, NB).long()
            d = (pos_q[:, None] - pos_k[None, :]).clamp(0, layer.pos_w.numel() - 1)
            s = s + (layer.ts_w[bk] + layer.pos_w[d][None])[:, None].to(s.dtype)
            p = torch.nn.functional.silu(s * (1.0 / math.sqrt(DH))) * scale * mask[None, None]
            a = torch.einsum("bhij,bjhd->bihd", p.to(V.dtype), V)
            x = layer.finish(x.reshape(-1, DM), a.reshape(-1, H, DH), u).view(users, n, DM)
        return norm(x)

    hist_ids = torch.randint(0, n_items, (users, cached), generator=gen).to(dev)
    for c0 in range(0, cached, 512):                                # prefill in slices to bound the score tensor
        c1 = min(c0 + 512, cached)
        forward(table[hist_ids[:, c0:c1]], hist_ts.to(dev), c0, c1 - c0, 0)
    reqs = []
    for _ in range(8):
        nts = hist_ts[:, -1:] + torch.cumsum(torch.empty(users, new).exponential_(1 / 300.0, generator=gen), 1)
        ids = torch.cat([torch.randint(0, n_items, (users, new), generator=gen), torch.randint(0, n_items, (users, cands), generator=gen)], 1)
        ts = torch.cat([hist_ts, nts, nts[:, -1:].expand(users, cands) + 1.0], 1).contiguous()
        reqs.append((ids.pin_memory(), ts.pin_memory()))
    out_host = torch.empty(users, cands, dtype=torch.float32).pin_memory()

    def step(i):
        ids, ts = reqs[i % 8]
        ids_d, ts_d = ids.to(dev, non_blocking=True), ts.to(dev, non_blocking=True)
        x = table[ids_d]
        h = forward(x, ts_d, cached, new, cands)
        out_host.copy_((h[:, new:].float() * x[:, new:].float()).sum(-1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return users * cands

    import numpy as np

    ids0, ts0 = reqs[0]
    _finish(args, ClockSampler, dev, 1, 0, step, None, "HSTU ranking inference candidates/sec", "candidates/s",
            {"model": "HSTU %dL d512 8x64" % layers_n, "users": users, "cached_tokens": cached, "new_tokens": new, "candidates": cands,
             "page_size": page, "global_batch": users, "seq_len": total, "parallelism": "1 GPU, torch gather-based paged attention"},
            int(ids0.numel() * 8 + ts0.numel() * 4), int(out_host.numel() * 4),
            extra=lambda lat: {"p50_ms": float(np.percentile(lat, 50)), "p99_ms": float(np.percentile(lat, 99))})

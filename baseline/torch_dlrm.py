"""Stock-PyTorch statement of the DLRM-large training step: the comparison arm of the benchmark.

Nothing here touches this repository's kernels or engine.  Embedding tables are row-wise sharded (``id % world``)
fp16 tensors; the id exchange and the embedding / gradient exchanges are ``all_to_all_single`` over NCCL; lookups
are ``index_select``; the sparse update is row-wise Adagrad written with torch ops (unique + index_add); the MLPs
are ``nn.Linear`` under bf16 autocast (cuBLAS) with fused Adam; dense gradients are all-reduced in one flat
bucket.  Same synthetic data, batch and model as the product arm.
"""
from __future__ import annotations

import json
import math
import os

import torch
import torch.distributed as dist
from torch import nn


class _A2A(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, pg):
        ctx.meta = (out_splits, in_splits, pg)
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=pg)
        return out

    @staticmethod
    def backward(ctx, g):
        out_splits, in_splits, pg = ctx.meta
        gi = g.new_empty((sum(in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(gi, g.contiguous(), in_splits, out_splits, group=pg)
        return gi, None, None, None


class _Lookup(torch.autograd.Function):
    """rows = weight[idx]; backward applies row-wise Adagrad to the touched rows."""

    @staticmethod
    def forward(ctx, anchor, weight, state, idx, lr, eps):
        ctx.w, ctx.state, ctx.lr, ctx.eps = weight, state, lr, eps
        ctx.save_for_backward(idx)
        return weight.index_select(0, idx)

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        uniq, inv = torch.unique(idx, return_inverse=True)
        gs = torch.zeros(uniq.numel(), g.shape[1], dtype=torch.float32, device=g.device)
        gs.index_add_(0, inv, g.float())
        acc = ctx.state[uniq] + (gs * gs).mean(dim=1)
        ctx.state[uniq] = acc
        w = ctx.w[uniq].float() - ctx.lr * gs / (acc.sqrt() + ctx.eps)[:, None]
        ctx.w[uniq] = w.to(ctx.w.dtype)
        return None, None, None, None, None, None


class TorchDLRM(nn.Module):
    def __init__(self, rows, world, rank, pg, dev, D=128):
        super().__init__()
        self.world, self.rank, self.pg, self.D, self.T = world, rank, pg, D, len(rows)
        local = [(r + world - 1) // world for r in rows]
        offs = [0]
        for r in local:
            offs.append(offs[-1] + r)
        self.register_buffer("table_off", torch.tensor(offs[:-1], dtype=torch.int64, device=dev))
        self.weight = torch.empty(offs[-1], D, dtype=torch.float16, device=dev)
        for t in range(self.T):                                  # chunked init bounds the fp32 temporaries
            b = 1.0 / math.sqrt(rows[t])
            self.weight[offs[t]:offs[t + 1]].uniform_(-b, b)
        self.state = torch.zeros(offs[-1], dtype=torch.float32, device=dev)
        self.anchor = nn.Parameter(torch.zeros(1, device=dev))

        def mlp(dims, last_relu):
            layers = []
            for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
                layers.append(nn.Linear(a, b, device=dev))
                if i < len(dims) - 2 or last_relu:
                    layers.append(nn.ReLU())
            return nn.Sequential(*layers)
        self.bottom = mlp([13, 512, 256, D], True)
        F = self.T + 1
        self.tri = torch.tril_indices(F, F, -1, device=dev)
        self.top = mlp([D + F * (F - 1) // 2, 1024, 1024, 512, 256, 1], False)

    def embed(self, ids):                                        # ids [T, B] int64 (this rank's samples)
        T, B = ids.shape
        W = self.world
        if W == 1:
            rows = _Lookup.apply(self.anchor, self.weight, self.state, (ids + self.table_off[:, None]).reshape(-1), 0.01, 1e-8)
            return rows.view(T, B, self.D).permute(1, 0, 2)
        flat = ids.reshape(-1)
        table = torch.arange(T, device=ids.device).repeat_interleave(B)
        dest = flat % W
        order = torch.argsort(dest, stable=True)
        counts = torch.bincount(dest, minlength=W)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.pg)
        in_s, out_s = counts.tolist(), recv_counts.tolist()
        send = (flat // W + self.table_off[table])[order]
        recv = send.new_empty(sum(out_s))
        dist.all_to_all_single(recv, send, out_s, in_s, group=self.pg)
        rows = _Lookup.apply(self.anchor, self.weight, self.state, recv, 0.01, 1e-8)
        back = _A2A.apply(rows, in_s, out_s, self.pg)
        out = torch.empty_like(back)
        out[order] = back
        return out.view(T, B, self.D).permute(1, 0, 2)

    def forward(self, dense, ids, labels, global_batch):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            d = self.bottom(dense)
            e = self.embed(ids).to(torch.bfloat16)
            x = torch.cat([d[:, None, :], e], dim=1)
            z = torch.bmm(x, x.transpose(1, 2))
            inter = z[:, self.tri[0], self.tri[1]]
            logit = self.top(torch.cat([d, inter], dim=1)).squeeze(1)
        return torch.nn.functional.binary_cross_entropy_with_logits(logit.float(), labels.float(), reduction="sum") / global_batch


def run(args, table_rows, ClockSampler, unavailable_note=None):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pg = dist.group.WORLD if world > 1 else None
    GB = args.global_batch if not args.small else 4096
    B = GB // world
    rows = table_rows(args.table_seed) if not args.small else [1000 + 997 * i for i in range(26)]
    if args.rows_scale != 1.0:
        rows = [max(1000, int(r * args.rows_scale)) for r in rows]
    torch.manual_seed(0)
    model = TorchDLRM(rows, world, rank, pg, dev)
    dense_params = [p for n, p in model.named_parameters() if n != "anchor"]
    opt = torch.optim.Adam(dense_params, lr=1e-3, fused=True)
    g = torch.Generator().manual_seed(100 + rank)
    rows_t = torch.tensor(rows, dtype=torch.float64)

    def make_batch():
        # Zipf(1.1)-like ids by inverse-CDF sampling of a bounded power law, as in the product arm's generator
        u = torch.rand(26, B, generator=g, dtype=torch.float64)
        a = 1.1
        n = rows_t[:, None]
        ids = (((n ** (1 - a) - 1) * u + 1) ** (1 / (1 - a))).floor().clamp_(1, None).long() - 1
        ids = torch.minimum(ids, (n - 1).long())
        return (torch.randn(B, 13, generator=g).pin_memory(), ids.pin_memory(),
                (torch.rand(B, generator=g) < 0.03).float().pin_memory())
    host = [make_batch() for _ in range(4)]

    def step(i):
        dn, ids, lb = (t.to(dev, non_blocking=True) for t in host[i % 4])
        opt.zero_grad(set_to_none=False)
        loss = model(dn, ids, lb, GB)
        loss.backward()
        if world > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in dense_params])
            dist.all_reduce(flat, group=pg)
            o = 0
            for p in dense_params:
                p.grad.copy_(flat[o:o + p.numel()].view_as(p))
                o += p.numel()
        opt.step()
        return loss

    W = max(args.warmup, 3)
    last = 0.0
    for i in range(W):
        last = float(step(i).item())
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        last = float(step(W + i).item())
    e1.record()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    if rank == 0:
        h2d = sum(x.numel() * x.element_size() for x in host[0])
        print(json.dumps({
            "metric": "DLRM train samples/sec/box", "value": GB / (ms / 1e3), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 autocast (fp16 tables)", "data": "synthetic Zipf(1.1) ids, N(0,1) dense, Bernoulli(0.03) labels, random-init weights",
            "config": {"model": "DLRM-large" if not (args.small or args.rows_scale != 1.0) else "DLRM-debug-shrunk", "global_batch": GB,
                       "seq_len": None, "tables": 26, "embedding_dim": 128, "total_rows": int(sum(rows)),
                       "parallelism": "dp%d dense + row-wise tables, NCCL all_to_all_single / all_reduce, torch ops, cuBLAS" % world,
                       "l2": "inputs larger than L2"},
            "e2e": {"value": GB / (ms / 1e3), "unit": "samples/s", "ms_per_step": ms, "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": 4 * world, "note": "the timed loop copies every batch from pinned memory and reads the loss back"},
            "gpu_launches": 0, "final_loss": last, "clocks": clocks, "impl": "torch-nccl-baseline"}))
    if world > 1:
        dist.destroy_process_group()

"""HSTU training benchmark (``bench.py --model hstu``): tokens/s for the whole job.

Config: 8 layers, d_model 512, 8 heads x 64, SiLU attention with causal mask and learned relative position /
time bias, bf16; jagged sequences with log-normal lengths truncated to [16, 4096] (mean ~1024); item ids
Zipf(1.05) over 1e8 items in a dynamic hash table of dim 512 (row-wise sharded); timestamps with Exp(1/3600 s)
gaps; sampled-softmax loss with 512 shared negatives; 32 sequences per GPU; synthetic data."""
from __future__ import annotations

import json
import os

from typing import Optional

import torch
import torch.distributed as dist


def draw_lengths(n: int, gen: torch.Generator, max_len: int = 4096) -> torch.Tensor:
    """Sequence lengths: log-normal truncated to [16, max_len], mean about 1024."""
    return torch.exp(torch.randn(n, generator=gen) * 0.75 + 6.65).clamp(16, max_len).long()


def balance_sequences(lengths: torch.Tensor, world: int, per_rank: int):
    """Deal ``world * per_rank`` sequences to ranks so that the attention cost (sum of squared lengths, plus a linear
    term for the projections) is even: longest first, each to the least-loaded rank that still has room.  Returns the
    list of index lists, one per rank.  With jagged batches the step time of a data-parallel job is the slowest rank's,
    so an uneven deal wastes the other GPUs."""
    cost = lengths.double() ** 2 + 2048.0 * lengths.double()
    order = torch.argsort(cost, descending=True).tolist()
    load, out = [0.0] * world, [[] for _ in range(world)]
    for i in order:
        r = min((r for r in range(world) if len(out[r]) < per_rank), key=lambda r: load[r])
        out[r].append(i)
        load[r] += float(cost[i])
    return out


def make_batch(B: int, gen: torch.Generator, n_items: int = 100_000_000, n_neg: int = 512, max_len: int = 4096,
               lengths: Optional[torch.Tensor] = None):
    from ..sparse.jagged_tensor import KeyedJaggedTensor
    from ..utils.data import zipf_ids

    ln = draw_lengths(B, gen, max_len) if lengths is None else lengths.long()
    T = int(ln.sum())
    ids = zipf_ids(T, n_items, 1.05, gen)
    neg = torch.randint(0, n_items, (n_neg,), generator=gen)
    gaps = -torch.log(torch.rand(T, generator=gen).clamp_min(1e-9)) * 3600.0
    off = torch.cat([torch.zeros(1, dtype=torch.int64), ln.cumsum(0)])
    ts = torch.cumsum(gaps, 0)
    ts = ts - torch.repeat_interleave(ts[off[:-1]], ln)             # restart the clock per sequence
    lengths = torch.cat([ln, torch.tensor([n_neg] + [0] * (B - 1))])
    kjt = KeyedJaggedTensor(["item", "neg"], torch.cat([ids, neg]), lengths=lengths, stride=B)
    last = torch.zeros(T, dtype=torch.bool)
    last[off[1:] - 1] = True
    keep = (~last).nonzero(as_tuple=True)[0]                         # positions that have a next item to predict
    return kjt, off, int(ln.max()), ts.float(), T, keep


def build(device, env, cfg=None, capacity: int = 1 << 22, lr: float = 1e-3, max_ids_per_rank: int = 0):
    from ..dynamic import (DynamicEmbeddingCollection, DynamicEmbInitializerArgs, DynamicEmbInitializerMode,
                           DynamicEmbScoreStrategy, DynamicEmbTableOptions, OptimizerType)
    from ..modules.embedding_configs import EmbeddingConfig
    from ..optim import CombinedOptimizer, FusedDenseOptimizer
    from .hstu import HSTU, HSTUConfig

    cfg = cfg or HSTUConfig()
    ecfg = [EmbeddingConfig(num_embeddings=100_000_000, embedding_dim=cfg.d_model, name="item", feature_names=["item", "neg"])]
    opts = {"item": DynamicEmbTableOptions(
        initializer_args=DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.NORMAL, mean=0.0, std_dev=0.02),
        score_strategy=DynamicEmbScoreStrategy.TIMESTAMP, init_capacity=capacity, max_capacity=capacity)}
    emb = DynamicEmbeddingCollection(ecfg, opts, env, device, optimizer_type=OptimizerType.ROWWISE_ADAGRAD,
                                     learning_rate=0.01, use_index_dedup=True, max_ids_per_rank=max_ids_per_rank,
                                     # several GPUs: rows and their gradients cross NVLink in the model's compute dtype
                                     output_dtype=torch.bfloat16 if env.world_size > 1 else torch.float32)
    model = HSTU(cfg, emb, device)
    opt = FusedDenseOptimizer(model, "adam", lr=lr)
    return model, opt


def run_hstu_bench(args) -> None:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        from ..common import bind_rank_from_env

        bind_rank_from_env()                                # opt-in (RECSDK_B200_BIND_CPU=1): keep every rank on its own cores
        dist.init_process_group("nccl", device_id=dev)
    out = measure_hstu_training(args, world, rank, dev)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def measure_hstu_training(args, world: int, rank: int, dev, peer=None) -> dict:
    """Times ``args.steps`` HSTU training steps after ``max(args.warmup, 3)`` warm-up steps on an initialised process
    group; every rank returns the same result dictionary (times are the max over ranks, tokens the sum)."""
    from ..ops import _lib
    from ..parallel.comm import PeerGroup, ShardingEnv

    env = ShardingEnv(world, rank, dist.group.WORLD if world > 1 else None)
    B = 32 if not args.small else 4
    max_len = 4096 if not args.small else 512
    model, opt = build(dev, env, capacity=(1 << 22) if not args.small else (1 << 16), max_ids_per_rank=B * max_len + 512)
    gen = torch.Generator().manual_seed(1234 + rank)
    shared = torch.Generator().manual_seed(4321)                      # same on every rank: the global batch's lengths
    n_batches = args.steps + max(args.warmup, 3)
    max_len = 4096 if not args.small else 512
    host = []
    for _ in range(min(n_batches, 12)):
        if world > 1:
            # the input pipeline deals the global batch's sequences to ranks by attention cost
            glob = draw_lengths(B * world, shared, max_len)
            mine = balance_sequences(glob, world, B)[rank]
            host.append(make_batch(B, gen, max_len=max_len, lengths=glob[mine]))
        else:
            host.append(make_batch(B, gen, max_len=max_len))
    pin = lambda t: t.pin_memory()  # noqa: E731
    host = [(k.pin_memory(), pin(o), m, pin(ts), T, pin(kp)) for (k, o, m, ts, T, kp) in host]
    dense_params = [p for p in model.parameters() if p.requires_grad and not getattr(p, "_in_backward_optimizers", False)]
    flat_ids = {id(m.flat_param) for m in opt.flat_modules}

    reducer = None
    if world > 1:
        from ..parallel.grad_reduce import DenseGradReducer

        peer = peer or PeerGroup(dist.group.WORLD, dev)
        # dense gradients: one push all-reduce bucket per projection (launched from the end of that layer's backward, on a
        # side stream) and one bucket for all small parameters
        reducer = DenseGradReducer(peer, model, overlap=True, average=False)

    def sync_grads():
        if reducer is not None:
            reducer.sync()

    def step(i):
        k, o, m, ts, T, kp = host[i % len(host)]
        kd, od, td = k.to(dev, non_blocking=True), o.to(dev, non_blocking=True), ts.to(dev, non_blocking=True)
        opt.zero_grad()
        loss = model(kd, od, m, td, predict_positions=kp.to(dev, non_blocking=True))
        loss.backward()
        sync_grads()
        opt.step()
        return loss, T

    last = None
    for i in range(max(args.warmup, 3)):
        last, _ = step(i)
        last = float(last.item())
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    _lib.check_status(dev)
    from bench import ClockSampler  # the clock sampler lives beside the benchmark entry point

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    torch.cuda.synchronize(dev)
    lc0 = _lib.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tokens = 0
    e0.record()
    for i in range(args.steps):
        loss, T = step(max(args.warmup, 3) + i)
        last = float(loss.item())                      # device -> host read of the result every step
        tokens += T
    e1.record()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    _lib.check_status(dev)
    t = torch.tensor([ms, float(tokens)], dtype=torch.float64, device=dev)
    if world > 1:
        tm = t.clone()
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ts_ = t.clone()
        dist.all_reduce(ts_, op=dist.ReduceOp.SUM)
        ms, tokens = float(tm[0]), float(ts_[1])
    h2d = sum(k.values().numel() * 8 + o.numel() * 8 + ts.numel() * 4 + kp.numel() * 8 for (k, o, m, ts, T, kp) in host) / len(host)
    val = tokens / (ms / 1e3)
    return {
        "metric": "HSTU train tokens/sec", "value": val, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (log-normal lengths, Zipf(1.05) ids, Exp gaps), random-init weights",
        "config": {"model": "HSTU 8L d512 8x64", "global_batch": B * world, "seq_len": "lognormal[16,4096] mean~1024",
                   "parallelism": "dp%d dense + row-wise dynamic hash embedding" % world, "negatives": 512,
                   "l2": "inputs larger than L2 (activations ~%d MB per layer)" % (tokens / args.steps / world * 2048 * 2 / 1e6)},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": int(h2d) * world, "d2h_bytes_per_step": 4 * world,
                "note": "timed loop copies every batch from pinned host memory and reads the loss back each step"},
        "gpu_launches": int(_lib.launch_count - lc0), "final_loss": last, "clocks": clocks, "impl": "ours"}


def run_hstu_inference_bench(args) -> None:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:                                           # serving replicas: every GPU holds the model and its own users
        dist.init_process_group("nccl", device_id=dev)
    out = measure_hstu_inference(args, world, rank, dev)
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(out))


def measure_hstu_inference(args, world: int, rank: int, dev) -> dict:
    """HSTU ranking latency with a warm paged KV cache: ``users`` requests per batch, each with ``cached`` history
    tokens already in the cache, ``new`` fresh history tokens and ``cands`` candidates to score.  Every timed
    request copies its item ids and timestamps from pinned host memory, looks the embeddings up on the device,
    runs all layers against the paged cache and reads the scores back to the host."""
    import numpy as np

    from ..inference import KVCacheConfig, KVCacheManager
    from ..ops import _lib
    from ..ops import embedding_ops as E
    from .hstu import HSTU, HSTUConfig
    from .hstu_inference import HSTURanker

    small = args.small
    users, cached, new, cands, page = (64, 2048, 128, 1024, 64) if not small else (4, 256, 64, 32, 64)
    cfg = HSTUConfig(num_layers=8 if not small else 2, d_model=512, num_heads=8, head_dim=64, max_seq_len=4096)
    torch.manual_seed(0)
    model = HSTU(cfg, torch.nn.Identity(), dev, torch.bfloat16).eval()
    n_items = 4_000_000 if not small else 100_000
    table = (torch.randn(n_items, cfg.d_model, device=dev) * 0.05).to(torch.bfloat16)
    total = cached + new + cands
    pages_per_user = (total + page - 1) // page
    kvc = KVCacheConfig(num_layers=cfg.num_layers, num_heads=cfg.num_heads, head_dim=cfg.head_dim, page_size=page,
                        offload_chunksize=1024 if not small else 128, num_primary_cache_pages=users * pages_per_user + 64,
                        num_buffer_pages=users * pages_per_user, host_capacity_per_layer=users * 4 * 1024 * 512 * 2 * 2,
                        max_batch_size=users, max_seq_len=4096, dtype=torch.bfloat16, device=dev)
    kv = KVCacheManager.from_config(kvc)
    ranker = HSTURanker(model, kv)
    uid = torch.arange(users, dtype=torch.int64) + 1000 + rank * users
    gen = torch.Generator().manual_seed(7 + rank)

    def ids_ts(n_per_user: int, t0: float):
        ids = torch.randint(0, n_items, (users, n_per_user), generator=gen)
        gaps = torch.empty(users, n_per_user).exponential_(1 / 300.0, generator=gen)
        return ids, t0 + torch.cumsum(gaps, 1)

    # prefill: the cached history of every user (its own request, no candidates)
    hist_ids, hist_ts = ids_ts(cached, 0.0)
    zeros = torch.zeros(users, dtype=torch.int64)
    x = E.gather_rows(table, hist_ids.reshape(-1).to(dev))
    ranker.rank(uid, torch.full((users,), cached), zeros, x, hist_ts.reshape(-1).to(dev))
    kv.offload_try_wait()
    torch.cuda.synchronize(dev)
    _lib.check_status(dev)
    del x

    # requests: [new history tail | candidates] per user, ids + key timestamps in pinned memory
    n_req = 8
    reqs = []
    for _ in range(n_req):
        nid, nts = ids_ts(new, float(hist_ts.max()))
        cid = torch.randint(0, n_items, (users, cands), generator=gen)
        ids = torch.cat([nid, cid], 1).reshape(-1).pin_memory()
        ts = torch.cat([hist_ts, nts, nts[:, -1:].expand(users, cands) + 1.0], 1).reshape(-1).contiguous().pin_memory()
        reqs.append((ids, ts))
    hist_total = torch.full((users,), cached + new)
    ncand = torch.full((users,), cands)
    scores_host = torch.empty(users * cands, dtype=torch.float32).pin_memory()

    def request(i):
        ids, ts = reqs[i % n_req]
        ids_d, ts_d = ids.to(dev, non_blocking=True), ts.to(dev, non_blocking=True)
        xq = E.gather_rows(table, ids_d)
        s = ranker.rank(uid, hist_total, ncand, xq, ts_d)
        scores_host.copy_(s, non_blocking=True)
        torch.cuda.current_stream().synchronize()                       # the caller needs the scores
        kv.gpu.truncate(uid, torch.full((users,), cached))              # next request sees the same warm state
        return s

    W = max(args.warmup, 3)
    for i in range(W):
        request(i)
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    _lib.check_status(dev)
    from bench import ClockSampler

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    lc0 = _lib.launch_count
    lat = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    e0.record()
    for i in range(args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        request(W + i)
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
    _lib.check_status(dev)
    lat_np = np.asarray(lat)
    p50, p99 = float(np.percentile(lat_np, 50)), float(np.percentile(lat_np, 99))
    if world > 1:                                           # slowest replica's time and latencies
        t = torch.tensor([ms, p50, p99], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, p50, p99 = float(t[0]), float(t[1]), float(t[2])
    val = users * cands * args.steps * world / (ms / 1e3)
    ids0, ts0 = reqs[0]
    return ({
        "metric": "HSTU ranking inference candidates/sec", "value": val, "unit": "candidates/s", "n_gpus": world, "steps": args.steps,
        "warmup": W, "ms_per_step": ms / args.steps, "p50_ms": p50, "p99_ms": p99,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (uniform item ids, Exp time gaps), random-init weights",
        "config": {"model": "HSTU 8L d512 8x64" if not small else "HSTU 2L d512 8x64", "users": users, "cached_tokens": cached,
                   "new_tokens": new, "candidates": cands, "page_size": page, "global_batch": users * world, "seq_len": total,
                   "parallelism": "%d serving replica(s), one per GPU" % world, "l2": "KV pages read per request exceed L2 (%d MB)" % (users * total * 1024 * 2 * cfg.num_layers / 1e6)},
        "e2e": {"value": val, "unit": "candidates/s", "h2d_bytes_per_step": int(ids0.numel() * 8 + ts0.numel() * 4) * world,
                "d2h_bytes_per_step": int(scores_host.numel() * 4) * world,
                "note": "each request copies ids and timestamps from pinned memory and reads all scores back"},
        "gpu_launches": int(_lib.launch_count - lc0), "clocks": clocks, "impl": "ours"})

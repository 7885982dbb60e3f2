"""DCN v2 over dynamic (hash-table) embeddings: the benchmark of the dynamic-embedding configuration.

40 features share one hash table per feature (uint64-range keys drawn Zipf(1.2) over 2^40), dim 64 fp32 rows, bag
lengths Uniform[1, 20], admission on the second sighting, LFU eviction when the table fills, 3 cross layers + deep MLP
1024-512-256, global batch 32,768; every ``--ckpt-every`` steps the rows touched since the previous dump are
collected with ``incremental_dump`` (outside the timed region unless it falls inside it by the step count).
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

F_SPARSE, DIM = 40, 64


def make_batch(B: int, gen: torch.Generator, alpha: float = 1.2, key_bits: int = 40, max_len: int = 20):
    from ..sparse.jagged_tensor import KeyedJaggedTensor
    from ..utils.data import Batch, zipf_ids

    lens = torch.randint(1, max_len + 1, (F_SPARSE * B,), generator=gen)
    n = int(lens.sum())
    ranks = zipf_ids(n, 1 << key_bits, alpha, gen)
    feat = torch.repeat_interleave(torch.arange(F_SPARSE).repeat_interleave(B), lens)
    # spread the popularity ranks over the key space (a multiplicative hash keeps them distinct) and salt per feature
    keys = ((ranks * 0x9E3779B97F4A7C15 + feat * 0x632BE59BD9B4E019) & ((1 << 62) - 1)).long()
    kjt = KeyedJaggedTensor(["c%d" % i for i in range(F_SPARSE)], keys, lengths=lens, stride=B)
    return Batch(torch.randn(B, 13, generator=gen), kjt, (torch.rand(B, generator=gen) < 0.03).float())


def build(device, env, capacity: int, lr: float = 1e-3, max_ids_per_rank: int = 0):
    from ..dynamic import (DynamicEmbeddingBagCollection, DynamicEmbInitializerArgs, DynamicEmbInitializerMode, DynamicEmbScoreStrategy,
                           DynamicEmbTableOptions, OptimizerType)
    from ..modules.embedding_configs import EmbeddingBagConfig
    from .dcn import DCNv2, DCNv2Train

    cfgs = [EmbeddingBagConfig(num_embeddings=capacity * env.world_size, embedding_dim=DIM, name="tab", feature_names=["c%d" % i for i in range(F_SPARSE)])]
    opts = {"tab": DynamicEmbTableOptions(
        initializer_args=DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.UNIFORM, lower=-0.01, upper=0.01),
        score_strategy=DynamicEmbScoreStrategy.LFU, init_capacity=capacity, max_capacity=capacity, max_load_factor=0.9, admit_threshold=2)}
    emb = DynamicEmbeddingBagCollection(cfgs, opts, env, device, optimizer_type=OptimizerType.ROWWISE_ADAGRAD, learning_rate=0.01,
                                        output_dtype=torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32,
                                        max_ids_per_rank=max_ids_per_rank)
    model = DCNv2Train(DCNv2(emb, 13, [512, 256, DIM], cross_layers=3, low_rank=0, deep_layer_sizes=[1024, 512, 256], device=device))
    dense = [p for n, p in model.named_parameters() if not n.startswith("model.sparse_arch.")]
    opt = torch.optim.Adam(dense, lr=lr, fused=torch.device(device).type == "cuda")
    return model, opt, emb, dense


def run_dcn_bench(args) -> None:
    from ..dynamic import incremental_dump
    from ..ops import _lib
    from ..parallel.comm import ShardingEnv

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    env = ShardingEnv(world, rank, dist.group.WORLD if world > 1 else None)
    GB = 32768 if not args.small else 1024
    B = GB // world
    model, opt, emb, dense = build(dev, env, (1 << 27) if not args.small else (1 << 18), max_ids_per_rank=F_SPARSE * B * 20)
    model.global_batch_size = GB
    gen = torch.Generator().manual_seed(77 + rank)
    host = [make_batch(B, gen).pin_memory() for _ in range(4)]
    ckpt_every = getattr(args, "ckpt_every", 500)
    dumps = {"count": 0, "keys": 0}
    score_floor = 0

    reducer = None
    if world > 1:
        from ..parallel.comm import PeerGroup
        from ..parallel.grad_reduce import DenseGradReducer

        reducer = DenseGradReducer(PeerGroup(dist.group.WORLD, dev), model, overlap=True, average=False)

    def step(i):
        b = host[i % len(host)].to(dev, non_blocking=True)
        opt.zero_grad()
        loss, _ = model(b)
        loss.backward()
        if reducer is not None:
            reducer.sync()
        opt.step()
        if ckpt_every and (i + 1) % ckpt_every == 0:
            out, _scores = incremental_dump(model, score_floor, env.process_group)
            dumps["count"] += 1
            dumps["keys"] += sum(k.numel() for tabs in out.values() for (k, _v) in tabs.values())
        return loss

    W = max(args.warmup, 3)
    last = 0.0
    for i in range(W):
        last = float(step(i).item())
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    _lib.check_status(dev)
    from bench import ClockSampler

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    torch.cuda.synchronize(dev)
    lc0 = _lib.launch_count
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
    _lib.check_status(dev)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    if rank == 0:
        val = GB / (ms / 1e3)
        print(json.dumps({
            "metric": "DCNv2 + dynamic hash embeddings train samples/sec", "value": val, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 (fp32 table rows)", "data": "synthetic Zipf(1.2) keys over 2^40, Uniform[1,20] bags, random-init weights",
            "config": {"model": "DCNv2 3 cross + 1024-512-256-1", "global_batch": GB, "seq_len": None, "features": F_SPARSE, "dim": DIM,
                       "capacity_per_gpu": (1 << 27) if not args.small else (1 << 18), "admission": "count >= 2", "eviction": "LFU at 0.9 load",
                       "parallelism": "dp%d dense + row-wise (key %% world) dynamic hash table" % world,
                       "l2": "table rows and activations exceed L2"},
            "e2e": {"value": val, "unit": "samples/s", "h2d_bytes_per_step": int(host[0].nbytes()) * world, "d2h_bytes_per_step": 4 * world},
            "gpu_launches": int(_lib.launch_count - lc0), "final_loss": last, "incremental_dumps": dumps, "clocks": clocks, "impl": "ours"}))
    if world > 1:
        dist.destroy_process_group()

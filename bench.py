"""Headline benchmark: DLRM-large training throughput (samples/s for the whole job).

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per rank by torchrun)
    python bench.py --impl reference ...                     (the unmodified reference; unavailable here)

Config (the named DLRM-large): 26 fp16 embedding tables of dim 128 with row counts log-uniform in
[1e4, 4e7] (seeded), one-hot ids ~ Zipf(1.1), mixed table-wise + row-wise sharding, 13 dense
features, bottom MLP 13-512-256-128, pairwise dot interaction, top MLP 479-1024-1024-512-256-1 in bf16,
labels ~ Bernoulli(0.03), global batch 65,536 (fixed as N grows: strong scaling), row-wise Adagrad on
the tables, Adam on the dense parameters, synthetic data, random-init weights.

Two numbers are reported:
* ``value``  device-timed: K replays of the captured train step (input dist + forward + backward with the
  fused sparse update + dense all-reduce + dense optimizer) from device-resident inputs, CUDA events,
  max over ranks;
* ``e2e``    the same metric through the public API, ``TrainPipelineSparseDist.progress()``: every step
  copies that step's batch from pinned host memory to the device and reads the loss back to the host.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--model", default="dlrm", choices=["dlrm", "hstu", "hstu-infer", "dcn"])
    ap.add_argument("--global-batch", type=int, default=65536)
    ap.add_argument("--small", action="store_true", help="tiny tables / batch for a quick functional check")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--table-seed", type=int, default=0)
    ap.add_argument("--ckpt-every", type=int, default=500, help="dcn: incremental dump period in steps (0 = off)")
    ap.add_argument("--repeats", type=int, default=5, help="dlrm: how many times the K-step timed loop is repeated (median reported)")
    ap.add_argument("--no-extra", action="store_true",
                    help="dlrm: skip the HSTU training / ranking-inference measurements that are appended to the JSON line")
    ap.add_argument("--rows-scale", type=float, default=1.0,
                    help="shrink every table (profiling captures on a small case); 1.0 = the named config")
    return ap.parse_args()


REFERENCE_UNAVAILABLE = ("reference is an Ascend NPU SDK: its setup.py needs python3.7 + TensorFlow wheels and its torch "
                         "path imports torch_npu/CANN/fbgemm_ascend/torchrec, none installable offline; "
                         "pip install to baseline/_ref failed at metadata generation")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_ms: int = 50) -> None:
        self.idx, self.proc, self.lines, self.period_ms = gpu_index, None, [], period_ms
        self._t0 = self._t1 = None
        self._stamps = []

    def begin_window(self) -> None:
        """Only samples taken between ``begin_window`` and ``end_window`` count (the sampler itself may start earlier,
        so that nvidia-smi's start-up does not eat a short timed region)."""
        self._t0 = time.time()

    def end_window(self) -> None:
        self._t1 = time.time()

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _pump(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())
            self._stamps.append(time.time())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:  # noqa: BLE001
            pass
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = self.lines
        if self._t0 is not None:
            t1 = self._t1 if self._t1 is not None else time.time()
            lines = [ln for ln, ts in zip(self.lines, self._stamps) if self._t0 <= ts <= t1 + 0.05]
        for ln in lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def table_rows(seed: int, n: int = 26, lo: float = 1e4, hi: float = 4e7):
    import random

    rng = random.Random(seed)
    return [int(round(math.exp(rng.uniform(math.log(lo), math.log(hi))))) for _ in range(n)]


def run_extras(args, world: int, rank: int, dev) -> dict:
    """HSTU training (every N) and HSTU ranking inference (N = 1) measured after the DLRM run, on the same process group.
    A failure here is reported inside the JSON line instead of losing the DLRM result."""
    import copy
    import traceback

    out = {}
    try:
        from recsdk_b200.models.hstu_bench import measure_hstu_training

        a = copy.copy(args)
        a.steps, a.warmup = min(args.steps, 20), max(min(args.warmup, 5), 3)
        r = measure_hstu_training(a, world, rank, dev)
        out["hstu"] = {"tokens_per_s": r["value"], "ms_per_step": r["ms_per_step"], "steps": r["steps"], "warmup": r["warmup"],
                       "e2e": r["e2e"], "config": r["config"], "gpu_launches": r["gpu_launches"], "final_loss": r["final_loss"],
                       "clocks": r["clocks"], "scaling": "weak"}
    except Exception as e:  # noqa: BLE001
        traceback.print_exc()
        out["hstu"] = {"error": "%s: %s" % (type(e).__name__, e)}
    if world == 1:
        try:
            import gc

            import torch

            gc.collect()
            torch.cuda.empty_cache()
            from recsdk_b200.models.hstu_bench import measure_hstu_inference

            a = copy.copy(args)
            a.steps, a.warmup = min(args.steps, 20), 3
            r = measure_hstu_inference(a, world, rank, dev)
            out["hstu_ranking_inference"] = {"p50_ms": r["p50_ms"], "p99_ms": r["p99_ms"], "candidates_per_s": r["value"],
                                             "steps": r["steps"], "config": r["config"], "e2e": r["e2e"]}
        except Exception as e:  # noqa: BLE001
            traceback.print_exc()
            out["hstu_ranking_inference"] = {"error": "%s: %s" % (type(e).__name__, e)}
    return out


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return
    if args.impl == "torch":
        # comparison arm: the same model and step in stock PyTorch + NCCL + cuBLAS (no code of this package)
        if args.model == "dlrm":
            from baseline.torch_dlrm import run as run_torch_dlrm

            run_torch_dlrm(args, table_rows, ClockSampler)
        elif args.model == "dcn":
            print(json.dumps({"impl": "torch-nccl-baseline", "unavailable": "no stock-PyTorch arm for the dynamic hash table configuration"}))
        elif args.model == "hstu":
            from baseline.torch_hstu import run as run_torch_hstu

            run_torch_hstu(args, ClockSampler)
        else:
            from baseline.torch_hstu import run_inference as run_torch_hstu_inference

            run_torch_hstu_inference(args, ClockSampler)
        return
    if args.model == "hstu":
        from recsdk_b200.models.hstu_bench import run_hstu_bench

        run_hstu_bench(args)
        return
    if args.model == "dcn":
        from recsdk_b200.models.dcn_bench import run_dcn_bench

        run_dcn_bench(args)
        return
    if args.model == "hstu-infer":
        from recsdk_b200.models.hstu_bench import run_hstu_inference_bench

        run_hstu_inference_bench(args)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torchrun --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from recsdk_b200.models.dlrm import DLRM, DLRMTrain
    from recsdk_b200.modules.embedding_configs import DataType, EmbeddingBagConfig
    from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection
    from recsdk_b200.ops import _lib
    from recsdk_b200.ops import embedding_ops as E
    from recsdk_b200.optim import CombinedOptimizer, FusedDenseOptimizer
    from recsdk_b200.parallel.comm import ShardingEnv
    from recsdk_b200.parallel.model_parallel import DistributedModelParallel
    from recsdk_b200.parallel.planner import EmbeddingShardingPlanner, Topology
    from recsdk_b200.parallel.train_pipeline import TrainPipelineSparseDist
    from recsdk_b200.utils.data import RandomRecDataset

    GB = args.global_batch if not args.small else 4096
    assert GB % world == 0
    B = GB // world
    rows = table_rows(args.table_seed) if not args.small else [1000 + 997 * i for i in range(26)]
    if args.rows_scale != 1.0:
        rows = [max(1000, int(r * args.rows_scale)) for r in rows]
    keys = ["f%d" % i for i in range(26)]
    cfgs = [EmbeddingBagConfig(num_embeddings=r, embedding_dim=128, name="t%d" % i, feature_names=[keys[i]],
                               data_type=DataType.FP16) for i, r in enumerate(rows)]
    env = ShardingEnv(world, rank, dist.group.WORLD if world > 1 else None)
    ebc = EmbeddingBagCollection(cfgs, device=torch.device("meta"))
    model = DLRMTrain(DLRM(ebc, 13, [512, 256, 128], [1024, 1024, 512, 256, 1], dense_device=dev),
                      global_batch_size=GB)
    plan = EmbeddingShardingPlanner(Topology(world_size=world)).plan(model)
    dmp = DistributedModelParallel(model, env, dev, plan,
                                   sparse_optimizer=E.OptimizerSpec(kind=E.OPT_ROWWISE_ADAGRAD, lr=0.01, eps=1e-8),
                                   max_local_batch=B, one_hot=True, init_seed=None)
    opt = CombinedOptimizer([dmp.fused_optimizer, FusedDenseOptimizer(dmp.module, "adam", lr=1e-3)])
    pipe = TrainPipelineSparseDist(dmp, opt, dev, return_loss=True, cuda_graph=not args.no_graph)

    # a few distinct pinned host batches, cycled; every step still copies its batch host -> device
    data = RandomRecDataset(keys, rows, B, alpha=1.1, one_hot=True, pos_rate=0.03, seed=100 + rank, pin=True)
    host_batches = [data.make_batch() for _ in range(4)]

    def loader():
        while True:
            for b in host_batches:
                yield b

    it = loader()

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # ---------------- warm-up through the public API (also captures the graph) ----------------
    sampler = ClockSampler(local_rank, period_ms=20)
    sampler.start()                                   # started early: nvidia-smi needs ~0.1 s before its first sample
    W = max(args.warmup, 3)
    capture_steps = 4 if not args.no_graph else 0     # graph mode: eager steps before the capture plus the capture itself
    last = None
    for _ in range(W + capture_steps):
        loss, _ = pipe.progress(it)
        last = float(loss.item())
    sync_all()
    _lib.check_status(dev)
    R = max(args.repeats, 1)

    # ---------------- e2e: public API, H2D every step, loss read back every step ----------------
    sync_all()
    sampler.begin_window()
    loss_host = torch.zeros(2, dtype=torch.float32).pin_memory()
    loss_ev = [torch.cuda.Event(), torch.cuda.Event()]
    e2e_runs = []
    for _ in range(R):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(args.steps):
            loss, _ = pipe.progress(it)
            # every step's loss is copied to pinned host memory and read there; the read of step k happens after step
            # k + 1 has been enqueued, so the host never idles the GPU between steps
            loss_host[k & 1].copy_(loss.detach().reshape(()), non_blocking=True)
            loss_ev[k & 1].record()
            if k:
                loss_ev[(k - 1) & 1].synchronize()
                last = float(loss_host[(k - 1) & 1])
        loss_ev[(args.steps - 1) & 1].synchronize()
        last = float(loss_host[(args.steps - 1) & 1])
        e1.record()
        sync_all()
        e2e_runs.append(e0.elapsed_time(e1) / args.steps)

    # ---------------- device-timed: the train step alone from device-resident inputs ----------------
    dev_batches = [b.to(dev) for b in host_batches]
    torch.cuda.synchronize(dev)
    if pipe._graph is not None:
        def one_step(i):
            pipe._copy_into_static(dev_batches[i % len(dev_batches)])
            pipe._graph.replay()
    else:
        def one_step(i):
            pipe._step(dev_batches[i % len(dev_batches)])
    for i in range(3):
        one_step(i)
    sync_all()
    from recsdk_b200.utils import trace as _trace

    _trace.reset()
    lc1 = _lib.launch_count
    step_runs = []
    for r in range(R):
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for i in range(args.steps):
            one_step(i)
        s1.record()
        sync_all()
        step_runs.append(s0.elapsed_time(s1) / args.steps)
    lc2 = _lib.launch_count
    sampler.end_window()
    clocks = sampler.stop()
    _lib.check_status(dev)

    # per repeat: max over ranks; then the median repeat is the reported value
    tr = torch.tensor([step_runs, e2e_runs], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tr, op=dist.ReduceOp.MAX)
    step_runs, e2e_runs = tr[0].tolist(), tr[1].tolist()
    step_ms, e2e_ms = statistics.median(step_runs), statistics.median(e2e_runs)
    launches = pipe.launches_per_step * args.steps if pipe._graph is not None and hasattr(pipe, "launches_per_step") \
        else (lc2 - lc1) // R
    kjt_bytes = host_batches[0].nbytes()
    from recsdk_b200.utils import trace

    phases = trace.report() if trace.ENABLED else None
    if rank == 0 and phases:
        print("phase timing (device time from each mark to the next, mean us): " +
              json.dumps({k: round(v["mean_us"], 1) for k, v in phases.items()}), file=sys.stderr)
    if world > 1:
        tl = torch.tensor([last], dtype=torch.float64, device=dev)
        dist.all_reduce(tl)                      # each rank's loss is its share of the global-batch mean
        last = float(tl[0])
    used_graph = pipe._graph is not None
    selfcheck = None
    if world > 1:
        # correctness evidence next to the multi-GPU number: the fused backend against the library-collective backend
        try:
            from recsdk_b200.parallel.selfcheck import run_selfcheck

            selfcheck = run_selfcheck(env, dmp.peer, dev)
        except Exception as e:  # noqa: BLE001
            import traceback

            traceback.print_exc()
            selfcheck = {"ok": False, "error": "%s: %s" % (type(e).__name__, e)}
    extras = {}
    if not args.no_extra and not args.small and args.rows_scale == 1.0:
        # the other half of the headline metric (HSTU training tokens/s at the same N) and, on one GPU, the ranking
        # request latency: measured in the same invocation so that they reach the same record
        del pipe, dmp, opt, model, dev_batches
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        extras = run_extras(args, world, rank, dev)
    if rank == 0:
        out = {
            "metric": "DLRM train samples/sec/box", "value": GB / (step_ms / 1e3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": W, "graph_capture_steps": capture_steps, "ms_per_step": step_ms,
            "repeats": {"n": R, "ms_per_step": [round(x, 4) for x in step_runs], "min": min(step_runs), "max": max(step_runs),
                        "e2e_ms_per_step": [round(x, 4) for x in e2e_runs], "reported": "median"},
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 (fp16 tables)",
            "data": "synthetic Zipf(1.1) ids, N(0,1) dense, Bernoulli(0.03) labels, random-init weights",
            "config": {"model": "DLRM-large" if not (args.small or args.rows_scale != 1.0) else "DLRM-debug-shrunk", "global_batch": GB,
                       "seq_len": None, "tables": 26, "embedding_dim": 128, "total_rows": int(sum(rows)),
                       "parallelism": "dp%d dense + table-wise/row-wise embedding shards (push exchange over NVLink peer memory)" % world,
                       "cuda_graph": used_graph,
                       "l2": "inputs larger than L2: %.1f GB of tables + >126 MB activations per step" % (sum(rows) * 256 / 1e9)},
            "e2e": {"value": GB / (e2e_ms / 1e3), "unit": "samples/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": kjt_bytes * world, "d2h_bytes_per_step": 4 * world,
                    "note": "TrainPipelineSparseDist.progress() per step: H2D of that step's batch from pinned memory (copy stream, "
                            "overlapped with the previous step) and a D2H copy of that step's loss, read on the host one step later"},
            "gpu_launches": int(launches), "final_loss": last, "clocks": clocks, "impl": "ours",
        }
        if selfcheck is not None:
            out["selfcheck"] = selfcheck
        out.update(extras)
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Kernel micro-benchmarks (CUDA-event timing, warm-up, L2 flushed between iterations).

    python -m recsdk_b200.utils.microbench gemm --m 65536 --n 1024 --k 1024
    python -m recsdk_b200.utils.microbench hstu_fwd --seqs 8 --len 2048 --heads 8 [--bias]
    python -m recsdk_b200.utils.microbench hstu_bwd --seqs 8 --len 2048 --heads 8 [--bias]
    python -m recsdk_b200.utils.microbench tbe_fwd --rows 20000000 --batch 65536 --tables 26
    python -m recsdk_b200.utils.microbench ln_mul_bwd --m 65536 --n 512
    python -m recsdk_b200.utils.microbench pooled_bwd --batch 32768 --tables 40 --n 64
    python -m recsdk_b200.utils.microbench exchange --batch 65536 --tables 26 --rows 2000000      # push exchange, one rank
    python -m recsdk_b200.utils.microbench allreduce --n 3000000                                   # push all-reduce, one rank
    python -m recsdk_b200.utils.microbench sampled_softmax --m 32768 --k 512 --n 512
    python -m recsdk_b200.utils.microbench kv_transfer --seqs 16 --len 4096 --heads 8             # host tier <-> device pages

``exchange`` and ``allreduce`` run the multi-GPU kernels with a world of one (every "peer" pointer is this GPU's own
buffer): the same code path and memory traffic minus NVLink, which is what a single-GPU ncu capture can show; the
NVLink figures come from the multi-GPU tests (``tests/multi_gpu_worker.py --allreduce``) and the benchmark's phase times.

Prints one JSON line with the measured time and the achieved rate against the measured peaks
(``MEASURED_PEAKS.json`` at the repository root when present, else 6.65 TB/s and 1.59 PFLOP/s).
Small cases of these commands are what the ncu captures under ``profiles/`` were taken on.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0) * 1e9, d.get("bf16_tflops", 1590.0) * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def _time(fn, iters: int, warmup: int = 3) -> float:
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")      # > 126 MB L2
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def host_engines(a) -> dict:
    """Host id-processing engines (no GPU): this package's native ``IdsMapper`` / bucketize against the reference's own,
    unmodified C++ (``baseline/build_ref_host.py`` builds ``baseline/_ref/libhybrid_cpp.so`` from the reference tree) on the
    same ids: Zipf(1.1) ids of one table for the fused unique + lookup, a feature-major KJT for the bucketize."""
    import time

    import numpy as np

    from ..host import host
    from ..utils.data import zipf_ids

    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ref_so = os.path.join(root, "baseline", "_ref", "libhybrid_cpp.so")
    have_ref = os.path.exists(ref_so)
    if have_ref:
        torch.ops.load_library(ref_so)
    g = torch.Generator().manual_seed(0)
    n, rows, world, F = a.batch * 26, a.rows, 8, 26
    ids = zipf_ids(n, rows, 1.1, g)
    ids_np = ids.numpy().astype(np.int64)

    def best(fn, reps=a.iters):
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e3)
        return min(ts)

    out = {"what": "host_engines", "ids": n, "distinct": int(np.unique(ids_np).size), "table_rows": rows,
           "reference_library": ref_so if have_ref else None}
    H = host()
    # ---- fused unique + lookup: a fresh mapper per call measures insertion, a warm one measures the steady state
    def ours_cold():
        H.IdsMapper(rows).ids2indices_unique_out(ids_np)

    warm = H.IdsMapper(rows)
    warm.ids2indices_unique_out(ids_np)
    out["ours_unique_lookup_cold_ms"] = best(ours_cold)
    out["ours_unique_lookup_warm_ms"] = best(lambda: warm.ids2indices_unique_out(ids_np))
    if have_ref:
        def ref_cold():
            torch.classes.hybrid.IdsMapper(rows, True).ids2indices_unique(ids)

        rwarm = torch.classes.hybrid.IdsMapper(rows, True)
        rwarm.ids2indices_unique(ids)
        out["reference_unique_lookup_cold_ms"] = best(ref_cold)
        out["reference_unique_lookup_warm_ms"] = best(lambda: rwarm.ids2indices_unique(ids))
        a_, b_ = warm.ids2indices_unique_out(ids_np), rwarm.ids2indices_unique(ids)
        out["same_distinct_count"] = int(np.asarray(a_[1]).size) == int(b_[1].numel())
    # ---- bucketize of a feature-major KJT (one id per bag) over `world` ranks
    B = a.batch
    lengths = np.ones(F * B, dtype=np.int64)
    out["ours_bucketize_ms"] = best(lambda: H.block_bucketize_sparse_features(lengths, ids_np, None, F, B, world, None, True))
    if have_ref:
        lt, block = torch.from_numpy(lengths), torch.full((F,), (rows + world - 1) // world, dtype=torch.int64)

        def ref_bucketize():
            torch.ops.hybrid.block_bucketize_sparse_features_cpu(lt, ids, False, True, block, world, None, None, None, 0, None,
                                                                 False, False, False, False, None)

        try:
            out["reference_bucketize_ms"] = best(ref_bucketize)
        except Exception as e:  # noqa: BLE001
            out["reference_bucketize_error"] = "%s: %s" % (type(e).__name__, str(e)[:200])
    for k in ("unique_lookup_cold", "unique_lookup_warm", "bucketize"):
        if "reference_%s_ms" % k in out:
            out["speedup_%s" % k] = out["reference_%s_ms" % k] / out["ours_%s_ms" % k]
    out["threads"] = torch.get_num_threads()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "hstu_fwd", "hstu_bwd", "tbe_fwd", "interaction", "ln_mul_bwd", "pooled_bwd",
                                     "exchange", "allreduce", "sampled_softmax", "host_engines", "kv_transfer"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=1024)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--splits", type=int, default=1)
    ap.add_argument("--epi", default="relu", choices=["relu", "none", "mask"])
    ap.add_argument("--colsum", action="store_true")
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--len", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--bias-grads", default="both", choices=["both", "ts", "pos", "none"])
    ap.add_argument("--rows", type=int, default=10_000_000)
    ap.add_argument("--batch", type=int, default=65536)
    ap.add_argument("--tables", type=int, default=26)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    if a.what == "host_engines":
        print(json.dumps(host_engines(a)))
        return
    from ..ops import _lib, gemm

    hbm, flops, src = _peaks()
    dev = torch.device("cuda", 0)
    out = {"what": a.what, "peaks": src}
    if a.what == "gemm":
        A = torch.randn((a.k, a.m) if a.a_mn else (a.m, a.k), device=dev).bfloat16()
        B = torch.randn((a.k, a.n) if a.b_mn else (a.n, a.k), device=dev).bfloat16()
        bias = torch.randn(a.n, device=dev)
        if a.splits > 1:
            C = torch.zeros(a.m, a.n, device=dev)
            fn = lambda: gemm.gemm16(A, B, a_mn=a.a_mn, b_mn=a.b_mn, out=C, epi=gemm.EPI_F32_ATOMIC, splits=a.splits)  # noqa: E731
        elif a.epi == "mask":                                  # input-gradient GEMM of a ReLU layer (+ fused bias gradient)
            C = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
            aux = torch.randn(a.m, a.n, device=dev).bfloat16()
            cs = torch.zeros(a.n, device=dev) if a.colsum else None
            fn = lambda: gemm.gemm16(A, B, a_mn=a.a_mn, b_mn=a.b_mn, out=C, aux=aux, epi=gemm.EPI_RELU_MASK, colsum_out=cs)  # noqa: E731
        else:
            C = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=dev)
            cs = torch.zeros(a.n, device=dev) if a.colsum else None
            fn = lambda: gemm.gemm16(A, B, a_mn=a.a_mn, b_mn=a.b_mn, out=C, bias=bias,  # noqa: E731
                                     epi=gemm.EPI_RELU if a.epi == "relu" else gemm.EPI_NONE, colsum_out=cs)
        ms = _time(fn, a.iters)
        fl = 2.0 * a.m * a.n * a.k
        out.update(ms=ms, tflops=fl / ms / 1e9, frac_of_peak=fl / (ms / 1e3) / flops, shape=[a.m, a.n, a.k])
    elif a.what in ("hstu_fwd", "hstu_bwd"):
        from ..ops import hstu_attention as HA
        from ..ops.hstu_attention_bwd import hstu_attn_bwd

        H, D, L, S = a.heads, 64, a.len, a.seqs
        T = S * L
        q, k, v = [(torch.randn(T, H, D, device=dev) * 0.5).bfloat16() for _ in range(3)]
        off = torch.arange(0, T + 1, L, device=dev)
        kw = dict(ts=None, ts_w=None, ts_divisor=0.301, pos_w=None)
        if a.bias:
            kw = dict(ts=torch.cumsum(torch.rand(T, device=dev) * 3600, 0), ts_w=torch.randn(129, device=dev) * 0.1,
                      ts_divisor=0.301, pos_w=torch.randn(4096, device=dev) * 0.1)
        if a.what == "hstu_fwd":
            o = torch.empty_like(q)
            fn = lambda: HA.hstu_attn_fwd(q, k, v, off, off, L, 0.125, 1.0 / L, True, out=o, **kw)  # noqa: E731
            mm = 2
        else:
            do = torch.randn_like(q)
            fn = lambda: hstu_attn_bwd(do, q, k, v, off, off, 0.125, 1.0 / L, True, None, None, 0, kw["ts"], kw["ts_w"],  # noqa: E731
                                       0.301, kw["pos_w"], max_len_k=L, want_dts=a.bias_grads in ("both", "ts"),
                                       want_dpos=a.bias_grads in ("both", "pos"))
            mm = 5
        ms = _time(fn, a.iters)
        pairs = S * H * (L * (L + 128) / 2)                     # causal (block-granular) score elements
        fl = pairs * D * 2 * mm
        out.update(ms=ms, tflops=fl / ms / 1e9, score_elems_per_s=pairs / (ms / 1e3), shape=[S, L, H, D], bias=a.bias,
                   **({"bias_grads": a.bias_grads} if a.what == "hstu_bwd" and a.bias else {}))
    elif a.what == "tbe_fwd":
        from ..ops import embedding_ops as E

        T, B, D = a.tables, a.batch, 128
        rows = a.rows // T
        lay = E.TbeLayout([D] * T, [rows] * T, [E.SH_LOCAL] * T, [0] * T, 1, 0)
        w = torch.randn(T * rows * D, device=dev).half()
        d = lay.device_tensors(dev, [w.data_ptr()], 2)
        idx = torch.randint(0, rows, (T * B,), device=dev)
        o = torch.empty(B, T * D, dtype=torch.bfloat16, device=dev)
        fn = lambda: E.tbe_forward(lay, d, idx, None, B, E.POOL_SUM, torch.float16, o)  # noqa: E731
        ms = _time(fn, a.iters)
        by = T * B * D * 2 * 2 + T * B * 8
        out.update(ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / (ms / 1e3) / hbm)
    elif a.what == "ln_mul_bwd":
        from ..ops import hstu_ops as H

        rows, C = a.m, a.n
        x = torch.randn(rows, C, device=dev).bfloat16().requires_grad_(True)
        u = torch.randn(rows, C, device=dev).bfloat16().requires_grad_(True)
        ga, be = torch.randn(C, device=dev).requires_grad_(True), torch.randn(C, device=dev).requires_grad_(True)
        y = H.ln_mul(x, u, ga, be)
        dy = torch.randn_like(y)
        fn = lambda: torch.autograd.grad(y, [x, u, ga, be], dy, retain_graph=True)  # noqa: E731
        ms = _time(fn, a.iters)
        by = rows * C * 2 * 5                                   # dy, x, u read; dx, du written
        out.update(ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / (ms / 1e3) / hbm, shape=[rows, C],
                   note="includes the zero-fill of the two [C] parameter-gradient buffers")
    elif a.what == "pooled_bwd":
        # backward of the dynamic pooled lookup: (unique row, bag) pairs -> sorted runs -> per-row gradient sums
        B, F, D = a.batch, a.tables, a.n
        bags = B * F
        g = torch.Generator(device="cpu").manual_seed(0)
        lengths = torch.randint(1, 21, (bags,), generator=g)
        n = int(lengths.sum())
        zipf = torch.distributions.Pareto(torch.tensor(1.0), torch.tensor(0.2)).sample((n,)).long()      # heavy-tailed ids
        uniq, inv = torch.unique(zipf, return_inverse=True)
        U = uniq.numel()
        inv, lengths = inv.to(dev), lengths.to(dev)
        offsets = torch.cat([torch.zeros(1, dtype=torch.long, device=dev), lengths.cumsum(0)])
        grad = torch.randn(B, F * D, device=dev).bfloat16()
        bag_of = torch.repeat_interleave(torch.arange(bags, dtype=torch.int32, device=dev), lengths)
        L = _lib.lib()
        ks, bs = torch.empty_like(inv), torch.empty_like(bag_of)
        tb = int(L.rb_sort_segments_temp_bytes(n))
        temp = torch.empty(tb, dtype=torch.uint8, device=dev)
        red = torch.zeros(U, D, device=dev)
        st = _lib.stream_ptr(dev)

        def fn():
            red.zero_()
            if a.splits > 1:                                    # --splits 2: the one-atomic-per-id kernel, for comparison
                _lib.check(L.rb_pooled_scatter_add(grad.data_ptr(), 2, grad.stride(0), inv.data_ptr(), offsets.data_ptr(), bags, B, D, 0,
                                                   red.data_ptr(), st), "scatter")
                return
            _lib.check(L.rb_sort_pairs_i64_i32(inv.data_ptr(), bag_of.data_ptr(), n, max(1, U.bit_length()), ks.data_ptr(), bs.data_ptr(),
                                               temp.data_ptr(), tb, st), "sort")
            _lib.check(L.rb_pooled_segment_add(grad.data_ptr(), 2, grad.stride(0), ks.data_ptr(), bs.data_ptr(), offsets.data_ptr(), n, B, D,
                                               0, red.data_ptr(), st), "add")
        ms = _time(fn, a.iters)
        by = n * D * 2 + U * D * 4 * 2 + n * 12 * 2             # gradient rows gathered, red zeroed + written, pairs read + written once
        out.update(ms=ms, ids=n, unique=U, gbs=by / ms / 1e6, frac_of_peak=by / (ms / 1e3) / hbm,
                   kernel="scatter_add (atomics)" if a.splits > 1 else "sort + segment_add")
    elif a.what == "exchange":
        from ..modules.embedding_configs import DataType, EmbeddingBagConfig
        from ..ops import embedding_ops as E
        from ..parallel.comm import PeerGroup, ShardingEnv
        from ..parallel.embeddingbag import ShardedEmbeddingBagCollection
        from ..parallel.push_exchange import MODE_ONE_HOT, PH_GRADS, PH_ROWS
        from ..sparse.jagged_tensor import KeyedJaggedTensor

        B, T, D, R = a.batch, a.tables, 128, a.rows
        cfgs = [EmbeddingBagConfig(num_embeddings=R, embedding_dim=D, name="t%d" % i, feature_names=["f%d" % i],
                                   data_type=DataType.FP16) for i in range(T)]
        m = ShardedEmbeddingBagCollection(cfgs, {}, ShardingEnv(1, 0), dev, E.OptimizerSpec(kind=E.OPT_ROWWISE_ADAGRAD),
                                          peer=None, max_local_batch=B, one_hot=True)
        # drive the multi-rank kernels with a world of one: same code, every peer pointer is local
        peer = PeerGroup(None, dev)
        g = torch.Generator().manual_seed(0)
        from ..utils.data import zipf_ids

        ids = torch.cat([zipf_ids(B, R, 1.1, g) for _ in range(T)]).to(dev)
        # build the exchange by hand (``_ensure_capacity`` takes the single-rank shortcut otherwise)
        from ..parallel.push_exchange import PushExchange
        import numpy as np

        L_ = m.layout
        px = PushExchange(peer, dev, B * T, B * T, D, torch.bfloat16, B * L_.total_D * 2)
        i32 = dict(dtype=torch.int32, device=dev)
        f_D = torch.tensor(L_.feature_dims, **i32)
        f_Doff = torch.tensor([int(x) for x in L_.D_offsets[:-1]], **i32)
        tdims = torch.tensor(L_.dims, **i32)
        ftab = torch.tensor(L_.feature_table, **i32)
        kb = torch.from_numpy(np.concatenate([[0], np.cumsum(L_.local_rows[0])[:-1]]).astype(np.int64)).to(dev).view(1, -1).contiguous()
        # world-1 shards are SH_LOCAL: locate_row keeps every id on this rank
        dout = torch.randn(B, L_.total_D, device=dev).bfloat16()
        ws = E.BackwardWorkspace(dev, B * T, D)
        step = [0]

        def fwd():
            px.route_scatter(ids, None, T, B, m.dev["shards"], kb, ftab, L_.n_tables, want_bags=False)
            px.serve_rows(m.dev["key_cumsum"], m.dev["w_offsets"], tdims, f_Doff, L_.n_tables, T, m.weights, torch.bfloat16,
                          L_.total_D, True, B)
            px.wait(PH_ROWS)

        def bwd():
            seg = px.sort_received(L_.key_bits)
            px.push_grads(dout, MODE_ONE_HOT, f_D, f_Doff, T, B)
            px.wait(PH_GRADS)
            step[0] += 1
            E.tbe_backward_update_rows(L_, m.dev, seg, px.grad_recv, px.g_ld, tdims, m.weights, m.state1, m.state2, m.s_offsets,
                                       m.opt, step[0], ws)

        def both():
            fwd()
            bwd()

        fwd()
        ms_f = _time(fwd, a.iters)
        ms = _time(both, a.iters)
        rows_bytes = B * T * D * 2
        out.update(ms_forward=ms_f, ms_forward_backward=ms, entries=B * T,
                   forward_gbs=2 * rows_bytes / ms_f / 1e6, forward_frac_of_peak=2 * rows_bytes / (ms_f / 1e3) / hbm,
                   note="world of one: route + scatter + serve_rows (+ sort + push_grads + update_rows); bytes = rows read + written")
    elif a.what == "allreduce":
        class Flat(torch.nn.Module):
            def __init__(self, n):
                super().__init__()
                self.flat_param = torch.nn.Parameter(torch.zeros(n, device=dev))
                self.register_buffer("flat_grad", torch.randn(n, device=dev), persistent=False)

        n = (a.n + 7) // 8 * 8
        holder = torch.nn.Module()
        holder.a = Flat(n)
        # a world of one short-circuits the reducer class; call the kernel directly with self pointers
        import numpy as np

        L = _lib.lib()
        sb = int(L.rb_allreduce_push_staging_bytes(n, 1, 1))
        staging = torch.zeros(sb, dtype=torch.uint8, device=dev)
        result = torch.zeros(sb, dtype=torch.uint8, device=dev)
        flags = torch.zeros(2 * 16 * int(L.rb_allreduce_push_max_blocks()), dtype=torch.int32, device=dev)
        epoch = torch.zeros(2, dtype=torch.int32, device=dev)
        ps, pr, pf = (np.asarray([t.data_ptr()], dtype=np.uint64) for t in (staging, result, flags))
        st = _lib.stream_ptr(dev)

        def fn():
            _lib.check(L.rb_allreduce_push(holder.a.flat_grad.data_ptr(), n, ps.ctypes.data, pr.ctypes.data, pf.ctypes.data,
                                           epoch.data_ptr(), 1.0, 0, 1, 1, 0, 0, _lib.status_tensor(dev).data_ptr(), 1000, st),
                       "rb_allreduce_push")

        ms = _time(fn, a.iters)
        by = n * 4 * 2 + n * 2 * 4          # fp32 read + write, bf16 staging and result written + read
        out.update(ms=ms, n=n, gbs=by / ms / 1e6, frac_of_peak=by / (ms / 1e3) / hbm,
                   note="two-shot push all-reduce, one rank looped back: local traffic only")
    elif a.what == "kv_transfer":
        # host tier of the paged KV cache: --seqs users of --len tokens, 8 layers, --heads x 64; both engines, both directions
        import numpy as np

        from ..inference.kvcache_manager import NativeKVStorage
        from ..ops import embedding_ops as E

        L, page, chunk, hd = 8, 32, 1024, a.heads * 64
        ppc = chunk // page
        n_chunks = a.seqs * (a.len // chunk)
        row_elems = page * hd
        n_pages = n_chunks * ppc
        st = NativeKVStorage(dev, L, n_chunks, ppc * 2, row_elems, torch.bfloat16, 16 * ppc * 2)
        cache = [torch.randn(n_pages * 2, row_elems, device=dev).bfloat16() for _ in range(L)]
        for layer, c in enumerate(cache):
            st.register_cache(layer, c)
        chunks = np.arange(n_chunks, dtype=np.int64)
        rows = np.random.default_rng(0).permutation(n_pages).astype(np.int64)
        rows = np.stack([rows * 2, rows * 2 + 1], axis=1).reshape(-1)
        by = n_chunks * L * ppc * 2 * row_elems * 2

        def staged(fn):
            def run():
                task, err = fn(chunks, rows)
                assert err == 0
                st.stream_wait(task, L - 1)
                run.tasks.append(task)
            run.tasks = []
            return run

        res = {}
        for name, fn in (("offload", staged(st.offload)), ("onload", staged(st.onload))):
            ts = []
            for _ in range(a.iters + 1):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                for t in fn.tasks:
                    st.release(t)
                fn.tasks.clear()
                ts.append(e0.elapsed_time(e1))
            res["staged_%s_ms" % name] = sorted(ts[1:])[len(ts[1:]) // 2]
            res["staged_%s_gbs" % name] = by / res["staged_%s_ms" % name] / 1e6
        pool_rows = st.pool.view(-1, row_elems)
        per = ppc * 2
        d_rows = torch.from_numpy(rows).to(dev)
        pool_idx = [torch.from_numpy(((chunks[:, None] * L + layer) * per + np.arange(per)[None, :]).reshape(-1)).to(dev)
                    for layer in range(L)]
        for name in ("offload", "onload"):
            def zc():
                for layer in range(L):
                    if name == "offload":
                        E.copy_rows(cache[layer], d_rows, pool_rows, pool_idx[layer], dev)
                    else:
                        E.copy_rows(pool_rows, pool_idx[layer], cache[layer], d_rows, dev)
            ts = []
            for _ in range(a.iters + 1):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                zc()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            res["zero_copy_%s_ms" % name] = sorted(ts[1:])[len(ts[1:]) // 2]
            res["zero_copy_%s_gbs" % name] = by / res["zero_copy_%s_ms" % name] / 1e6
        out.update(res, bytes=by, chunks=n_chunks, layers=L, stats=st.stats(),
                   note="pinned host pool <-> device pages; staged = DMA copies + scatter/gather kernels on four streams, "
                        "zero_copy = one kernel per layer over mapped host memory; the link (PCIe / C2C) is the bound")
        st.close()
    elif a.what == "sampled_softmax":
        from ..ops import model_ops

        M, d, N = a.m, a.k, a.n
        h = torch.randn(M, d, device=dev).bfloat16().requires_grad_()
        ep = torch.randn(M, d, device=dev).bfloat16()
        en = torch.randn(N, d, device=dev).bfloat16()

        def fn():
            model_ops.sampled_softmax_loss(h, ep, en, 1.0 / M)

        ms = _time(fn, a.iters)
        by = M * d * 2 * 4 + M * N * 2 * 3
        out.update(ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / (ms / 1e3) / hbm, note="GEMM + fused loss/gradient pass (forward only timed)")
    else:
        from ..ops import interaction as I

        B, F, D = a.batch, 27, 128
        x0 = torch.randn(B, D, device=dev).bfloat16()
        xs = torch.randn(B, (F - 1) * D, device=dev).bfloat16()
        o = torch.empty(B, 480, dtype=torch.bfloat16, device=dev)
        fn = lambda: I.dot_interaction_fwd(x0, xs, F, o)  # noqa: E731
        ms = _time(fn, a.iters)
        by = B * F * D * 2 + B * 480 * 2
        out.update(ms=ms, gbs=by / ms / 1e6, frac_of_peak=by / (ms / 1e3) / hbm)
    torch.cuda.synchronize()
    _lib.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    sys.exit(main())

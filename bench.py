"""Benchmark of the quantized decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N=1): int4 group-128 decode GEMV at the Llama-3-8B MLP
up-projection shape (A 1x4096 bf16-stored, W 4096x14336).  One step = one pass
of the GEMV over LAYERS distinct quantised weight
matrices (a 32-layer model's worth, 1 GB of packed weights, so the 126 MB L2
cannot serve the traffic).  value = algorithmic bytes moved per second, summed
over ranks.  At N>1 every weight is sharded along N (output columns), each
rank computes its column slab, and the slabs of a step are reassembled with one
NCCL all-gather (strong scaling).

The same JSON line carries: the roofline of the dominant kernel against the
measured HBM copy bandwidth, the end-to-end number through the host-buffer API
(activations in from pinned host memory, outputs back out, every call), the
reference's CPU implementation timed on this box's host cores on a bounded
sample (one thread as shipped, and every core through a harness loop), clocks
sampled during the timed region, per-step percentiles, and the other workloads
(M=8/32, weight-only int8 M=16, paged int8-KV decode attention, W8A8, the
32-layer decode step) as `extra`.  At N>1 `extra` holds the sharded forms: the
tensor-parallel decode step, KV-head-sharded paged decode and N-sharded W8A8
with its outputs pushed to every rank from the GEMM's epilogue.  All inputs are
seeded synthetic data of the stated shapes and distributions.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GRAPHS = os.environ.get("LHB_BENCH_GRAPHS", "1") != "0"
K_DIM, N_DIM, GROUP = 4096, 14336, 128
LAYERS = 32
METRIC = "int4 group-128 decode GEMV effective HBM bandwidth"
UNIT = "TB/s"


def gemv_bytes(M, K, N, G, wbits=4):
    """Algorithmic bytes of one call: packed weights + group/channel scales + A (fp32) + C (fp32)."""
    w = K * N // 2 if wbits == 4 else K * N
    sc = (K // G) * N * 4 if wbits == 4 else N * 4
    return w + sc + 4 * M * K + 4 * M * N


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.001)

    def __enter__(self):
        if self.nv:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr:
            self._thr.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ----------------------------------------------------------------------------- reference arm

def cpu_gemv_baseline(budget_s=12.0, M=1):
    """The reference's gemm_w4a16_groupwise on the host cores: the unmodified
    single-threaded function called on one compact N-shard per thread."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from cpu_checker import best_checker
    chk = best_checker()
    # all the host cores this process may use, whatever OMP_NUM_THREADS a launcher exported
    chk.set_threads(len(os.sched_getaffinity(0)))
    threads = chk.max_threads()
    rng = np.random.default_rng(20242)
    W = (rng.standard_normal((K_DIM, N_DIM)) * 0.02).astype(np.float32)
    p, s = chk.q4_quantize_groupwise(W, GROUP)
    A = chk.round_to_bf16(rng.standard_normal((M, K_DIM)).astype(np.float32))
    shards = threads
    while N_DIM % shards:
        shards -= 1
    ns = N_DIM // shards
    # several copies of the sharded weight, cycled call by call, so that the host
    # caches cannot hold the weights from one call to the next (the GPU arm cycles
    # 32 distinct matrices for the same reason)
    copies = 6
    Bp = [[np.ascontiguousarray(p[:, i * ns:(i + 1) * ns]) for i in range(shards)] for _ in range(copies)]
    Bs = [[np.ascontiguousarray(s[:, i * ns:(i + 1) * ns]) for i in range(shards)] for _ in range(copies)]
    Cs = [np.zeros((M, ns), np.float32) for _ in range(shards)]
    chk.par_gemm_w4a16_shards(A, Bp[0], Bs[0], Cs, GROUP)          # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 400):
        c = len(times) % copies
        t0 = time.perf_counter()
        chk.par_gemm_w4a16_shards(A, Bp[c], Bs[c], Cs, GROUP)
        times.append(time.perf_counter() - t0)
    times.sort()
    p50 = times[len(times) // 2]
    # as shipped: the reference function has no parallel region, one call runs on one thread
    one = []
    Cfull = np.zeros((M, N_DIM), np.float32)
    for _ in range(2):
        t0 = time.perf_counter()
        chk.gemm_w4a16_groupwise(A, p, s, GROUP, Cfull)
        one.append(time.perf_counter() - t0)
    b = gemv_bytes(M, K_DIM, N_DIM, GROUP)
    return {"value": b / p50 / 1e12, "unit": UNIT, "cores": threads,
            "kind": chk.kind, "ms_per_call": p50 * 1e3,
            "one_thread": {"value": b / min(one) / 1e12, "unit": UNIT, "ms_per_call": min(one) * 1e3,
                           "sample": "the unmodified function as shipped (no parallel region): best of 2 calls"},
            "sample": f"{len(times)} calls of one {K_DIM}x{N_DIM} GEMV (M={M}), N split into "
                      f"{shards} compact shards, one per host thread, {copies} weight copies cycled; p50"}


def cpu_other_baselines():
    """The other workloads on the host cores, each on a bounded sample: the reference's functions as
    shipped (one thread) and through the harness loop over independent calls (all cores)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from cpu_checker import AttnCfg, Layout, best_checker
    chk = best_checker()
    chk.set_threads(len(os.sched_getaffinity(0)))
    threads = chk.max_threads()
    rng = np.random.default_rng(20241)
    out = {}

    def best(f, n=2):
        ts = []
        for _ in range(n):
            t0 = time.perf_counter(); f(); ts.append(time.perf_counter() - t0)
        return min(ts)
    # weight-only int8, M=16, K=N=4096: dequantise + fp32 GEMM (the reference has no fused function)
    W = (rng.standard_normal((4096, 4096)) * 0.02).astype(np.float32)
    q, s = chk.q8_quantize_per_col(W)
    A = rng.standard_normal((16, 4096)).astype(np.float32)
    b1 = gemv_bytes(16, 4096, 4096, 0, wbits=8)
    t_one = best(lambda: chk.gemm_w8a16_perchannel(A, q, s))
    shards = threads
    while 4096 % (shards * 16):
        shards -= 1
    ns = 4096 // shards
    Bq = [np.ascontiguousarray(q[:, i * ns:(i + 1) * ns]) for i in range(shards)]
    Bs = [np.ascontiguousarray(s[i * ns:(i + 1) * ns]) for i in range(shards)]
    Cs = [np.zeros((16, ns), np.float32) for _ in range(shards)]
    t_par = best(lambda: chk.par_gemm_w8a16_shards(A, Bq, Bs, Cs), 3)
    out["w8a16_m16"] = {"value": b1 / t_par / 1e12, "unit": "TB/s", "cores": threads, "ms_per_call": t_par * 1e3,
                        "one_thread": {"value": b1 / t_one / 1e12, "ms_per_call": t_one * 1e3},
                        "sample": f"full size (M=16, K=N=4096); harness: {shards} column shards, one per thread"}
    # paged int8-KV decode: 8 of the 64 sequences (requests are independent; tok/s scales with the count)
    n_s, hq, hkv, d, bs, pages = 8, 32, 8, 128, 16, 65536
    lens = rng.integers(512, 4097, size=n_s).astype(np.int32)
    perm = rng.permutation(pages).astype(np.int32)
    tables = np.full((n_s, 4096 // bs), -1, np.int32)
    used = 0
    L = Layout(pages, bs, hkv, d)
    pools = chk.empty_pools_q8(L)
    for r, l in enumerate(lens):
        nb = (int(l) + bs - 1) // bs
        tables[r, :nb] = perm[used:used + nb]; used += nb
        kn = rng.standard_normal((hkv, int(l), d), dtype=np.float32)
        chk.paged_kv_append_q8(pools, kn, kn[:, ::-1].copy(), tables[r], L, 0, int(l))
    Q = rng.standard_normal((n_s, hq, 1, d)).astype(np.float32)
    cfg = AttnCfg(hq, hkv, 1, d, 1, 0.0, 0, 0)
    t_one = best(lambda: chk.paged_attention_q8_batched(Q, pools, tables, lens, cfg, L), 1)
    t_par = best(lambda: chk.paged_attention_q8_batched(Q, pools, tables, lens, cfg, L, parallel=True), 2)
    out["paged_decode_q8"] = {"value": n_s / t_par, "unit": "tok/s", "cores": min(threads, n_s),
                              "one_thread": {"value": n_s / t_one},
                              "sample": f"{n_s} of the 64 sequences ({int(lens.sum())} cached tokens), one request per "
                                        f"thread in the harness loop; requests are independent, so tok/s is per call of this size"}
    del pools
    # W8A8 8192 x 8192 x 28672: one row of M per thread (the function is exactly linear in M), extrapolated
    K5, N5, M5 = 8192, 28672, 8192
    Bq5 = rng.integers(-127, 128, size=(K5, N5), dtype=np.int8)
    rows = max(1, min(threads, 32))
    Aq5 = rng.integers(-127, 128, size=(rows, K5), dtype=np.int8)
    a_s, b_s = np.ones(rows, np.float32), np.ones(N5, np.float32)
    t_one = best(lambda: chk.gemm_w8a8(Aq5[:1], Bq5, a_s[:1], b_s), 1)
    t_par = best(lambda: chk.par_gemm_w8a8_mslabs(Aq5, Bq5, a_s, b_s, 1), 1)
    ops_row = 2.0 * K5 * N5
    out["w8a8_prefill"] = {"value": ops_row * rows / t_par / 1e12, "unit": "TOP/s", "cores": min(threads, rows),
                           "one_thread": {"value": ops_row / t_one / 1e12, "s_per_row": t_one},
                           "extrapolated_s_full_size": t_par / rows * M5,
                           "sample": f"{rows} of the {M5} rows of M, one per thread; time scales linearly with M "
                                     f"(extrapolated, not run at full size)"}
    return {"kind": chk.kind, "cores": threads, "workloads": out}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    budget = max(4.0, min(20.0, 2.0 * (args.steps + args.warmup)))
    cb = cpu_gemv_baseline(budget_s=budget)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": cb["ms_per_call"] * LAYERS, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"cfg2: W4A16 GEMV M=1 K={K_DIM} N={N_DIM} G={GROUP}; "
                                   f"CPU sample = one weight matrix, step time scaled to {LAYERS}"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our arm

# rows of the per-workload table (`--csv`): name, calls per step, operations and bytes per call, step statistics
ROWS = []


def timed(fn, steps, warmup, dist, torch, sampler=None, stats=None, min_region_s=0.0, row=None):
    """W untimed steps, then exactly `steps` steps between CUDA events on the
    launching stream, bracketed by barrier + synchronize; max over ranks.

    With `stats` (a dict) the region is repeated until at least `min_region_s` seconds of
    timed steps have run (each repeat bracketed the same way); the returned time is the median
    region, and `stats` receives the percentiles of the single steps (an event pair per step,
    mirroring bench/bench_util.hpp:98-123 of the reference: p50 / p90 / p99 beside the mean).
    `row` = (name, calls per step, operations per call, bytes per call) adds the workload to the table
    that `--csv` writes in the reference's format (bench/bench_util.hpp:142-154)."""
    if row is not None and stats is None:
        stats = {}
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    regions, step_ms = [], []
    ctx = sampler if sampler is not None else _Null()
    with ctx:
        while True:
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
            ev[0].record()
            for i in range(steps):
                fn()
                ev[i + 1].record()
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            ms = ev[0].elapsed_time(ev[steps])
            if dist is not None:
                t = torch.tensor([ms], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            regions.append(ms)
            if stats is not None:
                step_ms += [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
            # every rank sees the same (max-reduced) times, so every rank stops at the same repeat
            if stats is None or sum(regions) * 1e-3 >= min_region_s or len(regions) >= 200:
                break
    regions.sort()
    ms = regions[len(regions) // 2]
    if stats is not None:
        s = sorted(step_ms)
        pick = lambda q: s[min(len(s) - 1, int(q * len(s)))]
        stats.update({"regions": len(regions), "steps_sampled": len(s), "mean_ms": sum(s) / len(s),
                      "p50_ms": pick(0.50), "p90_ms": pick(0.90), "p99_ms": pick(0.99), "min_ms": s[0], "max_ms": s[-1],
                      "region_ms_min": regions[0], "region_ms_max": regions[-1]})
    if row is not None:
        ROWS.append((row, dict(stats)))
    return ms


def write_csv(path):
    """name,p50_us,p90_us,p99_us,min_us,max_us,mean_us,gflops,gbps per call; throughput from the p50, as the
    reference's harness derives it (bench/bench_util.hpp:119-123, :142-154)."""
    with open(path, "w") as f:
        f.write("name,p50_us,p90_us,p99_us,min_us,max_us,mean_us,gflops,gbps\n")
        for (name, calls, ops, nbytes), s in ROWS:
            us = {k: s[k + "_ms"] * 1e3 / calls for k in ("p50", "p90", "p99", "min", "max", "mean")}
            secs = us["p50"] * 1e-6
            f.write(f"{name},{us['p50']:.3f},{us['p90']:.3f},{us['p99']:.3f},{us['min']:.3f},{us['max']:.3f},{us['mean']:.3f},"
                    f"{(ops / secs / 1e9) if secs > 0 else 0:.2f},{(nbytes / secs / 1e9) if secs > 0 else 0:.2f}\n")


def graphed(fn, torch, enabled=True):
    """Capture `fn` (a fixed sequence of launches on the current stream) into a
    CUDA graph and return its replay; the launches were already run once by the
    caller so that one-time set-up (function attributes, tensor maps) is done."""
    if not enabled:
        return fn, False
    try:
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        torch.cuda.synchronize()
        return g.replay, True
    except Exception as e:          # stay measurable without graphs
        print(f"[bench] graph capture failed ({e!r}); timing eager launches", file=sys.stderr)
        torch.cuda.synchronize()
        return fn, False


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def make_w4_layers(torch, lb, layers, K, n_local, G, seed):
    packed, scales = [], []
    gen = torch.Generator(device="cuda").manual_seed(seed)
    for _ in range(layers):
        W = torch.randn(K, n_local, device="cuda", generator=gen) * 0.02
        p, s = lb.q4_quantize_groupwise(W, G)
        packed.append(p)
        scales.append(s)
        del W
    return packed, scales


def bench_extra(torch, lb, steps, warmup, hbm_peak):
    """The other benchmark workloads on one GPU (kernel-only, inputs resident)."""
    out = {}
    gen = torch.Generator(device="cuda").manual_seed(20241)
    packed, scales = make_w4_layers(torch, lb, 8, K_DIM, N_DIM, GROUP, 20243)
    for M in (8, 32):
        A = torch.randn(M, K_DIM, device="cuda", generator=gen).bfloat16().float()
        C = torch.empty(M, N_DIM, device="cuda")

        def step():
            for p, s in zip(packed, scales):
                lb.gemm_w4a16_groupwise(A, p, s, GROUP, C=C)
        run, _ = graphed(step, torch, GRAPHS)
        b = gemv_bytes(M, K_DIM, N_DIM, GROUP)
        ms = timed(run, steps, warmup, None, torch, row=(f"gemm_w4a16_groupwise_m{M}", len(packed), 2.0 * M * N_DIM * K_DIM, b))
        per = ms / (steps * len(packed)) * 1e-3
        out[f"w4a16_m{M}"] = {"us_per_call": per * 1e6, "GBps": b / per / 1e9,
                              "hbm_frac": b / per / 1e9 / hbm_peak, "bytes": b}
    del packed, scales
    # the same GEMV with asymmetric int4 weights: fp16 scale and zero-point per group
    # (same bytes per group as the reference's fp32 scale), 16 weight sets = 500 MB, M = 1
    asym = []
    for _ in range(16):
        W = torch.randn(K_DIM, N_DIM, device="cuda", generator=gen) * 0.02
        asym.append(lb.q4a_quantize_groupwise(W, GROUP))
        del W
    A = torch.randn(1, K_DIM, device="cuda", generator=gen).bfloat16().float()
    C = torch.empty(1, N_DIM, device="cuda")

    def step_asym():
        for p, s, z in asym:
            lb.gemm_w4a16_asym(A, p, s, z, GROUP, C=C)
    run_a, _ = graphed(step_asym, torch, GRAPHS)
    b = gemv_bytes(1, K_DIM, N_DIM, GROUP)
    ms = timed(run_a, steps, warmup, None, torch, row=("gemm_w4a16_asym_f16_m1", len(asym), 2.0 * N_DIM * K_DIM, b))
    per = ms / (steps * len(asym)) * 1e-3
    out["w4a16_asym_f16_m1"] = {"us_per_call": per * 1e6, "GBps": b / per / 1e9, "hbm_frac": b / per / 1e9 / hbm_peak,
                                "bytes": b,
                                "fast_path": int(lb._cabi.load().lhb_gemm_w4a16_asym_fast_path(1, N_DIM, K_DIM, GROUP))}
    del asym
    # weight-only int8, M=16, K=N=4096, 16 weight sets = 268 MB
    ws = []
    for _ in range(16):
        W = torch.randn(4096, 4096, device="cuda", generator=gen) * 0.02
        ws.append(lb.q8_quantize_per_col(W))
    A = torch.randn(16, 4096, device="cuda", generator=gen)
    C = torch.empty(16, 4096, device="cuda")

    def step8():
        for q, s in ws:
            lb.gemm_w8a16_perchannel(A, q, s, C=C)
    run8, _ = graphed(step8, torch, GRAPHS)
    b = gemv_bytes(16, 4096, 4096, 0, wbits=8)
    ms = timed(run8, steps, warmup, None, torch, row=("gemm_w8a16_perchannel_m16", len(ws), 2.0 * 16 * 4096 * 4096, b))
    per = ms / (steps * len(ws)) * 1e-3
    out["w8a16_m16"] = {"us_per_call": per * 1e6, "GBps": b / per / 1e9, "hbm_frac": b / per / 1e9 / hbm_peak,
                        "bytes": b}
    del ws
    out["paged_decode_q8"] = bench_paged_decode(torch, lb, steps, warmup, hbm_peak)
    torch.cuda.empty_cache()
    out["w8a8_prefill"] = bench_w8a8(torch, lb, min(steps, 5), 3)
    torch.cuda.empty_cache()
    out["fp8_prefill"] = bench_fp8(torch, lb, min(steps, 5), 3)
    torch.cuda.empty_cache()
    out["decode_step_cfg4"] = bench_decode_step(torch, lb, min(steps, 5), 3, hbm_peak)
    torch.cuda.empty_cache()
    return out


def bench_decode_step(torch, lb, steps, warmup, hbm_peak, layers=32, batch=32, ctx_len=2048, seed=20244,
                      rank=0, world=1, dist=None):
    """One decode step of a 32-layer Llama-3-8B-shaped stack (d 4096, 32/8 heads of
    128, FFN 14336, RoPE base 500000, RMSNorm), all seven projections int4 group-128, int8 paged KV holding
    `ctx_len` tokens per sequence, `batch` sequences; the whole step replayed as one CUDA graph.  With
    world > 1 the projections are sharded along N and attention by KV head (decode_step.decode_step_tp):
    every rank generates the same full-size weights from the seed and keeps its column slabs."""
    import numpy as np
    from longhornai_b200 import decode_step as ds
    cfg = ds.StepConfig(4096, 32, 8, 128, 14336, GROUP, 500000.0, False, 1e-5)
    lc = ds.local_config(cfg, world)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    bs = 16
    blocks_per_req = (ctx_len + 1 + bs - 1) // bs
    num_blocks = batch * blocks_per_req
    L = lb.PagedLayout(num_blocks, bs, lc.n_kv_heads, cfg.head_dim)
    acfg = lb.PagedAttnCfg(lc.n_q_heads, lc.n_kv_heads, 1, cfg.head_dim, 1, 0.0, 0, 0)
    rng = np.random.default_rng(seed)
    perm = rng.permutation(num_blocks).astype(np.int32)
    tables = torch.from_numpy(perm.reshape(batch, blocks_per_req).copy()).cuda()
    past = torch.full((batch,), ctx_len, dtype=torch.int32, device="cuda")
    cur = past + 1
    from longhornai_b200 import sharding as sh
    hd, grp = cfg.head_dim, cfg.n_q_heads // cfg.n_kv_heads
    h_lo, h_hi = sh.kv_head_range(cfg.n_kv_heads, rank, world)
    f_lo, f_hi = sh.column_range(cfg.ffn, rank, world)
    d_lo, d_hi = sh.column_range(cfg.dim, rank, world)

    def rnd(k, n, lo, hi):
        """Columns [lo, hi) of a seeded full [k, n] matrix (every rank draws the same full matrix)."""
        w = torch.randn(k, n, device="cuda", generator=gen) * 0.02
        return w[:, lo:hi].contiguous()
    lw, pools = [], []
    ones = torch.ones(4096, device="cuda")
    for _ in range(layers):
        wq = rnd(4096, 4096, h_lo * grp * hd, h_hi * grp * hd)
        wk = rnd(4096, 1024, h_lo * hd, h_hi * hd)
        wv = rnd(4096, 1024, h_lo * hd, h_hi * hd)
        wo = rnd(4096, 4096, d_lo, d_hi)
        full_gu = torch.randn(4096, 2 * 14336, device="cuda", generator=gen) * 0.02
        wgu = torch.cat([full_gu[:, f_lo:f_hi], full_gu[:, 14336 + f_lo:14336 + f_hi]], dim=1).contiguous()
        del full_gu
        wdown = rnd(14336, 4096, d_lo, d_hi)
        lw.append(ds.LayerWeights.quantize(lc, wq, wk, wv, wo, wgu, wdown, ones, ones))
        del wq, wk, wv, wo, wgu, wdown
        shape = (num_blocks, lc.n_kv_heads, bs, cfg.head_dim)
        pools.append(ds.KVPools(
            torch.randint(-127, 128, shape, dtype=torch.int8, device="cuda", generator=gen),
            torch.randint(-127, 128, shape, dtype=torch.int8, device="cuda", generator=gen),
            torch.rand(shape[:3], device="cuda", generator=gen) * 0.02 + 0.005,
            torch.rand(shape[:3], device="cuda", generator=gen) * 0.02 + 0.005))
    x0 = torch.randn(batch, 4096, device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed + 1))
    x = x0.clone()
    if world == 1:
        buf = ds.StepBuffers.allocate(cfg, batch, x.device)

        def step():
            x.copy_(x0)                  # every replay starts from the same hidden state
            ds.decode_step(x, lw, pools, tables, past, cur, cfg, L, acfg, buf)
    else:
        # exchanges: this library's push all-gather over peer memory; the NCCL composition is timed
        # beside it (and is the fallback when the processes cannot map each other's memory)
        from longhornai_b200 import peer as lpeer
        nccl_buf = ds.TPBuffers.allocate(cfg, world, batch, x.device)

        def nccl_step():
            x.copy_(x0)
            ds.decode_step_tp(x, lw, pools, tables, past, cur, cfg, L, acfg, nccl_buf, rank, world, dist)
        pg, why = None, ""
        if os.environ.get("LHB_TP_EXCHANGE", "peer") == "peer":
            try:
                pg = lpeer.PeerGather(ds.TPBuffers.peer_shapes(cfg, batch), rank, world, dist)
            except Exception as e:      # noqa: BLE001 - reported in the JSON line
                why = f"{type(e).__name__}: {e}"[:200]
            ok = torch.tensor([1 if pg is not None else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0 and pg is not None:
                pg = None
                why = "a peer could not map the buffers"
        if pg is not None:
            buf = ds.TPBuffers.allocate(cfg, world, batch, x.device, peer=pg)
            buf.fused_push = os.environ.get("LHB_TP_FUSED", "0") == "1"
            x = buf.x

            def step():
                x.copy_(x0)
                ds.decode_step_tp(x, lw, pools, tables, past, cur, cfg, L, acfg, buf, rank, world, dist)
            run_n, _ = graphed(nccl_step, torch, GRAPHS)
            nccl_ms = timed(run_n, steps, warmup, dist, torch) / steps
            # the two exchanges must give the same hidden state, bit for bit, on every rank
            nccl_step()
            torch.cuda.synchronize()
            x_nccl = x.clone()
        else:
            step, nccl_ms = nccl_step, None
    run, is_graph = graphed(step, torch, GRAPHS)
    ms = timed(run, steps, warmup, dist, torch)
    per = ms / steps * 1e-3
    wbytes = sum(w.weight_bytes() for w in lw) * world
    kvbytes = layers * batch * (ctx_len + 1) * cfg.n_kv_heads * (2 * cfg.head_dim + 8)
    b = wbytes + kvbytes
    finite = bool(torch.isfinite(x).all().item())
    out = {"ms_per_step": per * 1e3, "tok_per_s": batch / per, "GBps": b / per / 1e9,
           "hbm_frac_per_gpu": b / per / 1e9 / hbm_peak / world, "bytes": b, "layers": layers, "batch": batch,
           "ctx_len": ctx_len, "launches_per_step": layers * ds.launches_per_layer(batch) + 1,
           "graph": int(is_graph), "finite": int(finite), "n_gpus": world}
    if world > 1:
        out["sharding"] = (f"projections N/{world}, attention {cfg.n_kv_heads // world} KV heads per rank, "
                           f"4 all-gathers per layer")
        out["exchange"] = "peer-memory push (own kernel)" if pg is not None else "nccl"
        if pg is not None:
            pg.check()                                  # raises if any bounded wait gave up
            out["ms_per_step_nccl_exchange"] = nccl_ms
            step()
            torch.cuda.synchronize()
            same = torch.tensor([1 if torch.equal(x, x_nccl) else 0], device="cuda")
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            out["tp_parity"] = ("bit-identical" if int(same.item()) == 1 else "MISMATCH") + \
                               " (hidden state after the step: peer-memory exchange against NCCL all-gathers, every rank)"
            out["launches_per_step"] += layers * 5 + 1        # four exchanges and a separate SwiGLU per layer, one slab copy
            pg.close(dist)
        elif why:
            out["peer_exchange_unavailable"] = why
    return out


def bench_fp8(torch, lb, steps, warmup, M=8192, K=8192, N=28672):
    """The prefill-sized GEMM shape (8192 x 8192 x 28672) with E4M3 operands and per-tensor scales (lh::gemm_fp8_e4m3) on tcgen05."""
    gen = torch.Generator(device="cuda").manual_seed(20246)
    A, sa = lb.fp8_quantize_per_tensor(torch.randn(M, K, device="cuda", generator=gen))
    B, sb = lb.fp8_quantize_per_tensor(torch.randn(K, N, device="cuda", generator=gen) * 0.02)
    sa, sb = float(sa.item()), float(sb.item())
    Cout = torch.empty(M, N, device="cuda")

    def step():
        lb.gemm_fp8_e4m3(A, B, sa, sb, C=Cout)
    ms = timed(step, steps, warmup, None, torch, row=(f"gemm_fp8_e4m3_{M}x{N}x{K}", 1, 2.0 * M * N * K, M * K + K * N + 4.0 * M * N))
    per = ms / steps * 1e-3
    ops = 2.0 * M * N * K
    _, bf16_peak, kind = measured_peaks()
    return {"ms_per_call": per * 1e3, "TFLOPs": ops / per / 1e12,
            "frac_of_2x_bf16_" + kind: ops / per / 1e12 / (2 * bf16_peak),
            "frac_of_nominal_4500": ops / per / 1e12 / 4500.0,
            "fast_path": int(lb._cabi.load().lhb_gemm_fp8_fast_path(M, N, K))}


def bench_w8a8(torch, lb, steps, warmup, M=8192, K=8192, N=28672):
    """Prefill-sized W8A8 GEMM: per-token int8 activations x per-channel int8 weights,
    int32 accumulate, fp32 rescale (Llama-3-70B MLP shape)."""
    import ctypes as C
    gen = torch.Generator(device="cuda").manual_seed(20245)
    X = torch.randn(M, K, device="cuda", generator=gen)
    Aq, a_s = lb.q8_quantize_per_row(X)
    del X
    Wt = torch.randn(K, N, device="cuda", generator=gen) * 0.02
    Bq, b_s = lb.q8_quantize_per_col(Wt)
    del Wt
    Cout = torch.empty(M, N, device="cuda")

    def step():
        lb.gemm_w8a8(Aq, Bq, a_s, b_s, C=Cout)
    ms = timed(step, steps, warmup, None, torch, row=(f"gemm_w8a8_{M}x{N}x{K}", 1, 2.0 * M * N * K, M * K + K * N + 4.0 * M * N))
    per = ms / steps * 1e-3
    ops = 2.0 * M * N * K
    _, bf16_peak, kind = measured_peaks()
    return {"ms_per_call": per * 1e3, "TOPs": ops / per / 1e12,
            "frac_of_2x_bf16_" + kind: ops / per / 1e12 / (2 * bf16_peak),
            "frac_of_nominal_4500": ops / per / 1e12 / 4500.0,
            "fast_path": int(lb._cabi.load().lhb_gemm_w8a8_fast_path(M, N, K)),
            "bytes": M * K + K * N + 4 * M * N + 4 * (M + N)}


def bench_paged_decode(torch, lb, steps, warmup, hbm_peak, n_req=64, hq=32, hkv=8, d=128, bs=16,
                       pool_pages=65536, seed=20243):
    """Paged int8-KV decode attention: 64 sequences, lengths U[512,4096], page 16, random
    block tables over a 64k-page pool, int8 KV with per-row fp32 scales."""
    import numpy as np
    rng = np.random.default_rng(seed)
    lens = rng.integers(512, 4097, size=n_req).astype(np.int32)
    perm = rng.permutation(pool_pages).astype(np.int32)
    max_blocks = 4096 // bs
    tables = np.full((n_req, max_blocks), -1, np.int32)
    used = 0
    for r, l in enumerate(lens):
        nb = (int(l) + bs - 1) // bs
        tables[r, :nb] = perm[used:used + nb]
        used += nb
    L = lb.PagedLayout(pool_pages, bs, hkv, d)
    shp = (pool_pages, hkv, bs, d)
    k = torch.zeros(shp, dtype=torch.int8, device="cuda")
    v = torch.zeros_like(k)
    ks = torch.zeros(shp[:3], device="cuda")
    vs = torch.zeros_like(ks)
    td = torch.from_numpy(tables).cuda()
    gen = torch.Generator(device="cuda").manual_seed(seed)
    for r, l in enumerate(lens):
        kn = torch.randn(hkv, int(l), d, device="cuda", generator=gen)
        vn = torch.randn(hkv, int(l), d, device="cuda", generator=gen)
        lb.paged_kv_append_q8(k, v, ks, vs, kn, vn, td[r], L, 0, int(l))
    Q = torch.randn(n_req, hq, 1, d, device="cuda", generator=gen)
    O = torch.empty_like(Q)
    sl = torch.from_numpy(lens).cuda()
    cfg = lb.PagedAttnCfg(hq, hkv, 1, d, 1, 0.0, 0, 0)

    def step():
        lb.paged_attention_q8_batched(Q, k, v, ks, vs, td, sl, cfg, L, O=O)
    run, _ = graphed(step, torch, GRAPHS)
    total = int(lens.sum())
    pages = int(sum((int(l) + bs - 1) // bs for l in lens))
    b = total * hkv * (2 * d + 8) + 2 * Q.numel() * 4 + 4 * pages + 4 * n_req
    ms = timed(run, steps, warmup, None, torch, row=("paged_attention_q8_batched_decode", 1, 4.0 * total * hq * d, b))
    per = ms / steps * 1e-3
    import ctypes as C
    fast = lb._cabi.load().lhb_paged_attention_q8_fast_path(C.byref(cfg), C.byref(L))
    return {"tok_per_s": n_req / per, "us_per_step": per * 1e6, "GBps": b / per / 1e9,
            "hbm_frac": b / per / 1e9 / hbm_peak, "bytes": b, "sum_len": total, "fast_path": int(fast),
            "note": "KV working set 313 MB > L2; one kernel launch per step"}


def bench_paged_decode_sharded(torch, lb, steps, warmup, hbm_peak, rank, world, dist, n_req=64, hq=32, hkv=8, d=128,
                               bs=16, pool_pages=65536, seed=20243):
    """Paged int8-KV decode attention sharded by KV head: rank r holds the pools of heads
    [r * Hkv/g, (r + 1) * Hkv/g) (a GQA group stays on one rank), the replicated block tables and the
    query heads of its KV heads; there is no exchange inside the op.  Timed alone and with the
    all-gather that reassembles O [n_req, Hq, d] on every rank."""
    import numpy as np
    from longhornai_b200 import sharding as sh
    rng = np.random.default_rng(seed)
    lens = rng.integers(512, 4097, size=n_req).astype(np.int32)
    perm = rng.permutation(pool_pages).astype(np.int32)
    max_blocks = 4096 // bs
    tables = np.full((n_req, max_blocks), -1, np.int32)
    used = 0
    for r, l in enumerate(lens):
        nb = (int(l) + bs - 1) // bs
        tables[r, :nb] = perm[used:used + nb]
        used += nb
    h_lo, h_hi = sh.kv_head_range(hkv, rank, world)
    hk, grp = h_hi - h_lo, hq // hkv
    L = lb.PagedLayout(pool_pages, bs, hk, d)
    shp = (pool_pages, hk, bs, d)
    k = torch.zeros(shp, dtype=torch.int8, device="cuda")
    v = torch.zeros_like(k)
    ks = torch.zeros(shp[:3], device="cuda")
    vs = torch.zeros_like(ks)
    td = torch.from_numpy(tables).cuda()
    gen = torch.Generator(device="cuda").manual_seed(seed)         # every rank draws the same full tensors
    for r, l in enumerate(lens):
        kn = torch.randn(hkv, int(l), d, device="cuda", generator=gen)
        vn = torch.randn(hkv, int(l), d, device="cuda", generator=gen)
        lb.paged_kv_append_q8(k, v, ks, vs, kn[h_lo:h_hi].contiguous(), vn[h_lo:h_hi].contiguous(), td[r], L, 0, int(l))
    Qfull = torch.randn(n_req, hq, 1, d, device="cuda", generator=gen)
    Q = Qfull[:, h_lo * grp:h_hi * grp].contiguous()
    O = torch.empty_like(Q)
    sl = torch.from_numpy(lens).cuda()
    cfg = lb.PagedAttnCfg(hk * grp, hk, 1, d, 1, 0.0, 0, 0)

    def op():
        lb.paged_attention_q8_batched(Q, k, v, ks, vs, td, sl, cfg, L, O=O)
    run, _ = graphed(op, torch, GRAPHS)
    gathered = torch.empty((world,) + tuple(O.shape), device="cuda")

    def op_gather():
        run()
        dist.all_gather_into_tensor(gathered, O)
    ms_op = timed(run, steps, warmup, dist, torch)
    ms_g = timed(op_gather, steps, warmup, dist, torch)
    per, per_g = ms_op / steps * 1e-3, ms_g / steps * 1e-3
    total = int(lens.sum())
    pages = int(sum((int(l) + bs - 1) // bs for l in lens))
    b_rank = total * hk * (2 * d + 8) + 2 * Q.numel() * 4 + 4 * pages + 4 * n_req
    # parity across the sharding: rank 0 also runs the unsharded problem and compares the reassembled heads
    parity = None
    op_gather()
    torch.cuda.synchronize()
    if rank == 0:
        Lf = lb.PagedLayout(pool_pages, bs, hkv, d)
        shf = (pool_pages, hkv, bs, d)
        kf = torch.zeros(shf, dtype=torch.int8, device="cuda"); vf = torch.zeros_like(kf)
        ksf = torch.zeros(shf[:3], device="cuda"); vsf = torch.zeros_like(ksf)
        gen = torch.Generator(device="cuda").manual_seed(seed)
        for r, l in enumerate(lens):
            kn = torch.randn(hkv, int(l), d, device="cuda", generator=gen)
            vn = torch.randn(hkv, int(l), d, device="cuda", generator=gen)
            lb.paged_kv_append_q8(kf, vf, ksf, vsf, kn, vn, td[r], Lf, 0, int(l))
        cf = lb.PagedAttnCfg(hq, hkv, 1, d, 1, 0.0, 0, 0)
        Of = lb.paged_attention_q8_batched(Qfull, kf, vf, ksf, vsf, td, sl, cf, Lf)
        whole = sh.assemble_heads(gathered)
        err = (whole - Of).abs()
        tol = 1e-4 + 1e-3 * Of.abs()
        parity = {"max_abs_err_vs_one_gpu": float(err.max().item()), "within_1e-3_1e-4": bool((err <= tol).all().item())}
        del kf, vf, ksf, vsf
    return {"tok_per_s": n_req / per, "us_per_step": per * 1e6, "tok_per_s_with_gather": n_req / per_g,
            "us_per_step_with_gather": per_g * 1e6, "GBps_per_rank": b_rank / per / 1e9,
            "hbm_frac_per_rank": b_rank / per / 1e9 / hbm_peak, "bytes_per_rank": b_rank, "sum_len": total,
            "kv_heads_per_rank": hk, "gather_bytes_per_rank": O.numel() * 4, "n_gpus": world, "parity": parity,
            "sharding": f"{hk} of {hkv} KV heads (and their {hk * grp} query heads) per rank, tables replicated, "
                        f"no exchange inside the op; optional NCCL all-gather of O"}


def bench_w8a8_sharded(torch, lb, steps, warmup, rank, world, dist, M=8192, K=8192, N=28672):
    """W8A8 8192 x 8192 x 28672 with N sharded over the ranks.  Three forms of the same step:
    the GEMM on the local slab alone (no exchange); the GEMM whose epilogue stores every finished
    tile into every rank's full-width C over NVLink while the main loop runs on (this library's
    kernel, lhb_gemm_w8a8_sharded), followed by a one-element all-reduce as the completion signal;
    and the composition local GEMM + NCCL all-gather of the [M, N/g] slabs."""
    from longhornai_b200 import peer as lpeer
    from longhornai_b200 import sharding as sh
    gen = torch.Generator(device="cuda").manual_seed(20245)       # the same full tensors on every rank
    X = torch.randn(M, K, device="cuda", generator=gen)
    Aq, a_s = lb.q8_quantize_per_row(X)
    del X
    Wt = torch.randn(K, N, device="cuda", generator=gen) * 0.02
    Bq_full, bs_full = lb.q8_quantize_per_col(Wt)
    del Wt
    Bq, b_s = sh.shard_w8(Bq_full, bs_full, rank, world)
    del Bq_full, bs_full
    w = N // world
    C_local = torch.empty(M, w, device="cuda")
    ops = 2.0 * M * N * K
    _, bf16_peak, kind = measured_peaks()
    out = {"n_gpus": world, "sharding": f"N/{world} = {w} columns of B per rank, A replicated"}

    def gemm_only():
        lb.gemm_w8a8(Aq, Bq, a_s, b_s, C=C_local)
    ms = timed(gemm_only, steps, warmup, dist, torch)
    t_gemm = ms / steps * 1e-3
    out["gemm_only"] = {"ms_per_call": t_gemm * 1e3, "TOPs": ops / t_gemm / 1e12}
    gathered = torch.empty(world, M, w, device="cuda")

    def gemm_nccl():
        lb.gemm_w8a8(Aq, Bq, a_s, b_s, C=C_local)
        dist.all_gather_into_tensor(gathered, C_local)
    ms = timed(gemm_nccl, steps, warmup, dist, torch)
    t_nccl = ms / steps * 1e-3
    out["gemm_then_nccl_allgather"] = {"ms_per_call": t_nccl * 1e3, "TOPs": ops / t_nccl / 1e12,
                                       "layout": "[g, M, N/g] (a re-layout would still be needed for row-major C)"}
    nvlink_s = (world - 1) / world * M * N * 4 / 770e9            # bytes every rank must receive / measured peer-copy rate
    out["nvlink_floor_ms"] = nvlink_s * 1e3
    pg, why = None, ""
    try:
        pg = lpeer.PeerGather({"C": (M, N)}, rank, world, dist)
    except Exception as e:      # noqa: BLE001 - reported in the JSON line
        why = f"{type(e).__name__}: {e}"[:200]
    ok = torch.tensor([1 if pg is not None else 0], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0:
        if pg is not None:
            pg.close(dist)
        out["fused_push_unavailable"] = why or "a peer could not map the buffers"
        return out
    token = torch.zeros(1, device="cuda")

    def fused():
        pg.gemm_w8a8_sharded(Aq, Bq, a_s, b_s, "C")
        dist.all_reduce(token)                                      # every rank's stream has passed its GEMM
    ms = timed(fused, steps, warmup, dist, torch)
    t_fused = ms / steps * 1e-3
    roof = max(t_gemm, nvlink_s)
    out["gemm_with_epilogue_push"] = {"ms_per_call": t_fused * 1e3, "TOPs": ops / t_fused / 1e12,
                                      "exposed_exchange_ms": (t_fused - t_gemm) * 1e3,
                                      "frac_of_roof": roof / t_fused,
                                      "roof": "max(local GEMM time, (g-1)/g * M*N*4 B / 770 GB/s measured peer-copy rate)",
                                      "layout": "row-major [M, N] on every rank, no re-layout",
                                      "peer_mapping": pg.mapping}
    if pg.mapping_note:
        out["gemm_with_epilogue_push"]["peer_mapping_note"] = pg.mapping_note[:300]
    out["TOPs"] = ops / min(t_fused, t_nccl) / 1e12
    out["ms_per_call"] = min(t_fused, t_nccl) * 1e3
    out["frac_of_2x_bf16_" + kind + "_per_gpu"] = ops / min(t_fused, t_nccl) / 1e12 / (2 * bf16_peak) / world
    # parity: this rank's columns of the pushed matrix are the local GEMM's bits; every other slab matches
    # its producer's checksum
    fused()
    torch.cuda.synchronize()
    dist.barrier()
    full = pg.tensor("C")
    gemm_only()
    own = torch.equal(full[:, rank * w:(rank + 1) * w], C_local)
    sums = torch.stack([full[:, r * w:(r + 1) * w].double().sum() for r in range(world)])
    mine = C_local.double().sum().reshape(1)
    theirs = torch.empty(world, dtype=torch.float64, device="cuda")
    dist.all_gather_into_tensor(theirs, mine)
    good = torch.tensor([1 if (own and bool(torch.equal(sums, theirs))) else 0], device="cuda")
    dist.all_reduce(good, op=dist.ReduceOp.MIN)
    out["parity"] = "bit-identical" if int(good.item()) == 1 else "MISMATCH"
    pg.check()
    pg.close(dist)
    return out


def profile_traffic(name):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch, read from the committed ncu summary
    of that kernel (the markdown table under the repository's profile summaries); None when the summary is absent or has no such rows."""
    import re
    path = os.path.join(ROOT, "profiles", name + ".md")
    try:
        text = open(path).read()
    except OSError:
        return None
    unit = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    total, seen = 0.0, 0
    for metric in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
        m = re.search(r"\|\s*" + re.escape(metric) + r"\s*\|\s*([0-9.eE+-]+)\s*\|\s*(\w+)\s*\|", text)
        if m and m.group(2) in unit:
            total += float(m.group(1)) * unit[m.group(2)]
            seen += 1
    return int(total) if seen == 2 else None


def run_ours(args):
    import torch
    import longhornai_b200 as lb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    g = world
    if N_DIM % (g * 16):
        raise SystemExit("N must divide into 16-column-aligned shards")
    n_local = N_DIM // g
    hbm_peak, _, peak_kind = measured_peaks()
    M = 1

    packed, scales = make_w4_layers(torch, lb, LAYERS, K_DIM, n_local, GROUP, 20242 + rank)
    gen = torch.Generator(device="cuda").manual_seed(7)
    acts = [torch.randn(M, K_DIM, device="cuda", generator=gen).bfloat16().float() for _ in range(LAYERS)]
    outs = torch.empty(LAYERS, M, n_local, device="cuda")
    from longhornai_b200 import sharding

    def gemvs():
        for i in range(LAYERS):
            lb.gemm_w4a16_groupwise(acts[i], packed[i], scales[i], GROUP, C=outs[i])
    run_gemvs, is_graph = graphed(gemvs, torch, GRAPHS)

    def step():
        run_gemvs()
        if g > 1:
            sharding.all_gather_columns(outs, g, dist)     # [g, layers, M, N/g]

    sampler = ClockSampler(physical_gpu_index(local)) if rank == 0 else None
    stats = {}
    ms = timed(step, args.steps, args.warmup, dist, torch, sampler, stats=stats, min_region_s=0.5,
               row=("gemm_w4a16_groupwise_m1 (headline, per launch)", LAYERS, 2.0 * M * N_DIM * K_DIM,
                    g * (gemv_bytes(M, K_DIM, n_local, GROUP) - 4 * M * K_DIM) + 4 * M * K_DIM))
    launches = args.steps * LAYERS
    bytes_call_local = gemv_bytes(M, K_DIM, n_local, GROUP)
    bytes_step_total = LAYERS * (g * (bytes_call_local - 4 * M * K_DIM) + 4 * M * K_DIM)
    value = bytes_step_total * args.steps / (ms * 1e-3) / 1e12

    # end to end through the host-buffer path: activations come from pinned host
    # memory and results go back to pinned host memory on every call
    h_act_all = torch.stack([a.cpu() for a in acts]).pin_memory()       # the step's activations, one pinned buffer
    h_act = [h_act_all[i] for i in range(LAYERS)]
    h_out = torch.empty(LAYERS, M, n_local).pin_memory()
    d_act_all = torch.empty(LAYERS, M, K_DIM, device="cuda")
    d_acts = [d_act_all[i] for i in range(LAYERS)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    e2e_mode = os.environ.get("LHB_BENCH_E2E", "batched")

    def e2e_body():
        # As a serving loop would run it.  "batched": the step's activations arrive in one copy, the GEMVs
        # follow back to back on the launching stream (programmatic dependent launch between them stays
        # intact), each call's result copy trails on a second stream.  "percall": one input copy per
        # call on a third stream, every GEMV waiting for its own.  Either way every call's activations
        # come from the host and its result returns to the host inside the step.
        main = torch.cuda.current_stream()
        s_out.wait_stream(main)
        if e2e_mode == "batched":
            d_act_all.copy_(h_act_all, non_blocking=True)
        else:
            s_in.wait_stream(main)
        for i in range(LAYERS):
            if e2e_mode != "batched":
                with torch.cuda.stream(s_in):
                    d_acts[i].copy_(h_act[i], non_blocking=True)
                    landed = torch.cuda.Event()
                    landed.record(s_in)
                main.wait_event(landed)
            lb.gemm_w4a16_groupwise(d_acts[i], packed[i], scales[i], GROUP, C=outs[i])
            done = torch.cuda.Event()
            done.record(main)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                h_out[i].copy_(outs[i], non_blocking=True)
        if e2e_mode != "batched":
            main.wait_stream(s_in)
        main.wait_stream(s_out)
    run_e2e, e2e_graph = graphed(e2e_body, torch, GRAPHS)

    def step_e2e():
        run_e2e()
        if g > 1:
            sharding.all_gather_columns(outs, g, dist)     # [g, layers, M, N/g]
        torch.cuda.current_stream().synchronize()      # the caller reads the results on the host
    stats_e2e = {}
    ms_e2e = timed(step_e2e, args.steps, args.warmup, dist, torch, stats=stats_e2e, min_region_s=0.3,
                   row=("gemm_w4a16_groupwise_m1 from host buffers (per launch)", LAYERS, 2.0 * M * N_DIM * K_DIM,
                        g * (gemv_bytes(M, K_DIM, n_local, GROUP) - 4 * M * K_DIM) + 4 * M * K_DIM))
    e2e_value = bytes_step_total * args.steps / (ms_e2e * 1e-3) / 1e12

    status = lb.default_context().poll()
    if status != 0:
        raise SystemExit(f"device status word = {status}")

    tp_step, sharded = None, {}
    if g > 1 and not args.no_extra:
        # the sharded forms of the other workloads: every rank takes part, rank 0 reports
        del packed, scales, run_gemvs, run_e2e
        torch.cuda.empty_cache()
        try:
            tp_step = bench_decode_step(torch, lb, min(args.steps, 5), 3, hbm_peak, rank=rank, world=g, dist=dist)
        except Exception as e:
            tp_step = {"error": repr(e)}
        torch.cuda.empty_cache()
        try:
            sharded["paged_decode_q8"] = bench_paged_decode_sharded(torch, lb, args.steps, args.warmup, hbm_peak, rank, g, dist)
        except Exception as e:
            sharded["paged_decode_q8"] = {"error": repr(e)}
        torch.cuda.empty_cache()
        try:
            sharded["w8a8_prefill"] = bench_w8a8_sharded(torch, lb, min(args.steps, 5), 3, rank, g, dist)
        except Exception as e:
            sharded["w8a8_prefill"] = {"error": repr(e)}
        torch.cuda.empty_cache()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    per_launch_s = ms * 1e-3 / launches
    achieved = bytes_call_local / per_launch_s / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": g, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"cfg2: W4A16 group-{GROUP} decode GEMV, A {M}x{K_DIM} (bf16-stored, fp32 in the API), "
                               f"W {K_DIM}x{N_DIM} int4 packed [K/2,N] + fp32 scales; {LAYERS} distinct weight "
                               f"matrices per step",
                   "M": M, "K": K_DIM, "N": N_DIM, "group": GROUP, "layers_per_step": LAYERS,
                   "sharding": f"N/{g} columns per rank" + (", one all-gather of the outputs per step" if g > 1 else ""),
                   "l2": f"inputs larger than L2: {LAYERS * bytes_call_local / 1e6:.0f} MB of weights per rank "
                         f"cycled every step" + ("" if LAYERS * bytes_call_local > 2 * 126e6 else
                                                 " (NOT larger than L2 at this shard size)"),
                   "launch": "CUDA graph replay of the step" if is_graph else "eager launches",
                   "fast_path": int(lb._cabi.load().lhb_gemm_w4a16_fast_path(M, n_local, K_DIM, GROUP))},
        "step_stats": dict(stats, note="per-step CUDA-event times over all timed regions; ms_per_step and value "
                                       "come from the median region of exactly `steps` steps"),
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps, "step_stats": stats_e2e,
                "h2d_bytes_per_step": LAYERS * M * K_DIM * 4, "d2h_bytes_per_step": LAYERS * M * n_local * 4,
                "mode": e2e_mode,
                "note": ("the step's activations H2D from one pinned buffer at the start of the step, the GEMVs back to back, "
                         "every call's output D2H to pinned memory on a second stream, host sync every step; "
                         if e2e_mode == "batched" else
                         "every call's activations H2D from pinned memory and its outputs D2H to pinned memory, "
                         "input copies / GEMVs / result copies on three streams, host sync every step; ") +
                        "weights resident" + ("; the step replayed as one CUDA graph" if e2e_graph else "")},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": "gemv_mma_kernel<4,1>", "achieved": achieved, "peak": hbm_peak,
                     "unit": "GB/s", "frac": achieved / hbm_peak, "peak_kind": f"of {peak_kind}",
                     "frac_of_nominal_8TBps": achieved / 8000.0, "bytes_per_launch": bytes_call_local,
                     "us_per_launch": per_launch_s * 1e6,
                     # dram bytes of one launch of this kernel at the full N, read from the committed
                     # profiler summary of the kernel; scaled by the shard width
                     "traffic": (lambda tr: int(tr * (n_local / N_DIM)) if tr else None)(profile_traffic("gemv_w4a16_m1_cfg2"))},
        "clocks": sampler.summary() if sampler else None,
    }
    if g == 1 and not args.no_extra:
        try:
            line["extra"] = bench_extra(torch, lb, args.steps, args.warmup, hbm_peak)
        except Exception as e:      # the headline must still be printed
            line["extra"] = {"error": repr(e)}
    if tp_step is not None:
        line["extra"] = dict({"decode_step_cfg4": tp_step}, **sharded)
    if g == 1 and not args.no_cpu:
        try:
            line["cpu_baseline"] = cpu_gemv_baseline(budget_s=8.0)
        except Exception as e:
            line["cpu_baseline"] = {"error": repr(e)}
        try:
            line["cpu_baseline"]["other_workloads"] = cpu_other_baselines()
        except Exception as e:
            line["cpu_baseline"]["other_workloads"] = {"error": repr(e)}
    if args.csv:
        write_csv(args.csv)
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--csv", default=None, metavar="PATH",
                    help="also write the per-workload table (p50/p90/p99/min/max/mean per call, GFLOP/s and GB/s "
                         "from the p50) in the reference harness's CSV format")
    ap.add_argument("--only", default=None, choices=["paged_decode", "w8a8", "decode_step", "sharded"],
                    help="run one secondary workload alone on one GPU (for profiling) and print its numbers")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.only == "paged_decode":
        import torch
        import longhornai_b200 as lb
        torch.cuda.set_device(0)
        print(json.dumps({"paged_decode_q8": bench_paged_decode(torch, lb, args.steps, args.warmup,
                                                                 measured_peaks()[0])}), flush=True)
    elif args.only == "w8a8":
        import torch
        import longhornai_b200 as lb
        torch.cuda.set_device(0)
        print(json.dumps({"w8a8_prefill": bench_w8a8(torch, lb, args.steps, args.warmup, M=2048)}), flush=True)
    elif args.only == "sharded":
        # under torch.distributed.run: the KV-head-sharded paged decode and the N-sharded W8A8 alone
        import torch
        import torch.distributed as dist
        import longhornai_b200 as lb
        world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        res = {"paged_decode_q8": bench_paged_decode_sharded(torch, lb, args.steps, args.warmup, measured_peaks()[0],
                                                             rank, world, dist)}
        torch.cuda.empty_cache()
        res["w8a8_prefill"] = bench_w8a8_sharded(torch, lb, min(args.steps, 5), 3, rank, world, dist)
        if rank == 0:
            print(json.dumps(res), flush=True)
        dist.barrier()
        dist.destroy_process_group()
    elif args.only == "decode_step":
        import torch
        import longhornai_b200 as lb
        world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist = None
        if world > 1:                       # under torch.distributed.run: the tensor-parallel step
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        layers = int(os.environ.get("LHB_BENCH_LAYERS", "32"))
        res = bench_decode_step(torch, lb, args.steps, args.warmup, measured_peaks()[0], layers=layers,
                                rank=rank, world=world, dist=dist)
        if rank == 0:
            print(json.dumps({"decode_step_cfg4": res}), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
    if args.csv and args.only and int(os.environ.get("RANK", "0")) == 0:
        write_csv(args.csv)


if __name__ == "__main__":
    main()

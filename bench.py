"""Benchmark of the Q4_K / Q6_K matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens M]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload (the configuration the headline metric is quoted on): the Q6_K decode GEMV shaped like
a Llama-3-8B output projection, K=4096 -> N=128256, M tokens (default 1), synthetic seeded
blocks and N(0,1) activations (llm_rs_b200/synth.py).  A step is one `Backend::matmul` call on
that weight.  With N GPUs the weight rows are split N ways and the output slices are
all-gathered, inside the kernel over peer stores up to four tokens, over NCCL otherwise (strong
scaling: the total work is fixed).  The K steps are timed twice, launched one by one and as
replays of a CUDA graph of sixteen or more steps, and the faster figure is `value` (`config.timing`
names the method and gives the other figure): with several GPUs a step is shorter than the
Python call that launches it.

One JSON line on stdout (rank 0).  `value` is algorithmic GB/s (GGUF weight bytes + input +
output, per step) with everything resident in HBM; `e2e` is the same metric through the public
API with host buffers (activations copied in and the output copied out inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

K_IN, N_OUT = 4096, 128256
Q6K, Q4K = 14, 12
BLOCK_BYTES = {Q4K: 144, Q6K: 210}
L2_BYTES = 126e6
# values one rank receives from its peers per matmul, above which NCCL moves them (LLMRS_BENCH_FUSED_WORDS overrides)
FUSED_GATHER_MAX_WORDS = int(os.environ.get("LLMRS_BENCH_FUSED_WORDS", 1 << 18))


def algorithmic_bytes(dtype: int, K: int, N: int, M: int, in_bytes: int = 4, out_bytes: int = 4) -> int:
    """GGUF weight bytes + activations in + outputs out (the figure the roofline uses)."""
    return N * (K // 256) * BLOCK_BYTES[dtype] + M * K * in_bytes + M * N * out_bytes


def ncu_dram_bytes_per_launch() -> tuple[int | None, str | None]:
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel (Q6_K 4096 ->
    128256, one token), from the ncu capture recorded in profiles/traffic.json together with the commit
    of the kernel it was taken on; None when the record is missing."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            rec = json.load(f)["q6k_gemv_k4096_n128256_m1"]
        return int(rec["dram_bytes_read"]) + int(rec["dram_bytes_write"]), str(rec.get("kernel_commit"))
    except Exception:  # noqa: BLE001
        return None, None


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the GPU is busy."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80, "sw_power_cap": 0x4}
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    r = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                except Exception:
                    r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self._nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread:
            self._thread.join(1.0)
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# CPU baseline: the CPU restatement of the reference's op, on the host cores.
# ------------------------------------------------------------------------------------------------
def cpu_baseline(dtype: int, K: int, N: int, M: int, budget_s: float, rows: int | None = None):
    """Times the oracle's all-cores matmul on `rows` output rows (default: all N) for about
    budget_s seconds.  Returns (GB/s scaled to the algorithmic bytes of the sample, info)."""
    from llm_rs_b200 import synth
    from oracle import oracle as O
    rows = min(rows or N, N)
    w = synth.weight(dtype, K, rows, tid=2)
    x = synth.activations(M, K, tid=3)
    threads = len(os.sched_getaffinity(0))
    O.matmul(dtype, w, K, rows, x, fast=True, threads=threads)          # warm-up
    t0 = time.perf_counter()
    reps = 0
    while True:
        O.matmul(dtype, w, K, rows, x, fast=True, threads=threads)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s or reps >= 200:
            break
    per = dt / reps
    gbs = algorithmic_bytes(dtype, K, rows, M) / per / 1e9
    return gbs, per, {"cores": threads, "kind": "port",
                      "sample": f"{rows} of {N} output rows x K={K}, M={M}; {reps} passes in {dt:.1f} s; "
                                f"dequantise-then-dot over all rows, OpenMP over rows, -O2 -march=native"}


def cpu_baselines_other_configs():
    """The same CPU path on config 1 (the case the reference's own CPU code runs: Q4_K 4096 x 4096, one
    token; once as its test computes it -- one thread, dequantise the row, sequential float sum,
    tests/ops.rs:116-136 -- and once on all cores) and on the smallest case of config 3 (Q4_K
    4096 -> 14336 at 128 tokens, a sample of 1024 output rows, scaled linearly to all rows)."""
    from llm_rs_b200 import synth
    from oracle import oracle as O
    threads = len(os.sched_getaffinity(0))
    out = {}
    K, N = 4096, 4096
    w, x = synth.weight(Q4K, K, N, tid=2), synth.activations(1, K, tid=3)

    def time_it(fn, budget):
        fn()
        t0, reps = time.perf_counter(), 0
        while time.perf_counter() - t0 < budget and reps < 500:
            fn()
            reps += 1
        return (time.perf_counter() - t0) / reps

    t = time_it(lambda: O.matmul(Q4K, w, K, N, x, acc="f32", threads=1), 1.5)
    out["config1_q4k_4096x4096_m1_one_thread_as_the_reference_test"] = {
        "ms": round(t * 1e3, 3), "GBps": round(algorithmic_bytes(Q4K, K, N, 1) / t / 1e9, 3), "cores": 1}
    t = time_it(lambda: O.matmul(Q4K, w, K, N, x, fast=True, threads=threads), 1.5)
    out["config1_q4k_4096x4096_m1_all_cores"] = {
        "ms": round(t * 1e3, 3), "GBps": round(algorithmic_bytes(Q4K, K, N, 1) / t / 1e9, 3), "cores": threads}
    K, N, M, rows = 4096, 14336, 128, 1024
    w, x = synth.weight(Q4K, K, rows, tid=4), synth.activations(M, K, tid=5)
    t = time_it(lambda: O.matmul(Q4K, w, K, rows, x, fast=True, threads=threads), 2.0) * (N / rows)
    out["config3_q4k_4096x14336_m128_all_cores"] = {
        "ms": round(t * 1e3, 2), "TFLOPs": round(2.0 * M * K * N / t / 1e12, 4), "cores": threads,
        "sample": f"{rows} of {N} rows, scaled linearly"}
    return out


def run_reference(args, rank: int, world: int):
    """--impl reference: the reference's CPU implementation of the op (its Rust test code, restated in
    C: oracle/llmrs_oracle.c; the Rust/Metal original cannot be built on this box) on the host cores."""
    if rank != 0:
        return
    M = args.tokens
    rows = min(N_OUT, 32064)          # a quarter of the rows per step keeps K steps within minutes
    from llm_rs_b200 import synth
    from oracle import oracle as O
    w = synth.weight(Q6K, K_IN, rows, tid=2)
    x = synth.activations(M, K_IN, tid=3)
    threads = len(os.sched_getaffinity(0))      # all host cores (torchrun sets OMP_NUM_THREADS=1)
    for _ in range(max(args.warmup, 1)):
        O.matmul(Q6K, w, K_IN, rows, x, fast=True, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.matmul(Q6K, w, K_IN, rows, x, fast=True, threads=threads)
    per = (time.perf_counter() - t0) / args.steps
    gbs = algorithmic_bytes(Q6K, K_IN, rows, M) / per / 1e9
    line = {
        "impl": "reference", "metric": "q6k_gemv_algorithmic_GBps", "value": round(gbs, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(per * 1e3 * N_OUT / rows, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"configs[1]: Q6_K GEMV K={K_IN} N={N_OUT} M={M}", "sampled_rows": rows,
                   "note": "ms_per_step is scaled from the row sample to all N rows"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{rows} of {N_OUT} rows per step"},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# Our arm
# ------------------------------------------------------------------------------------------------
def allgather_check(be, stream, dev, world, fused, weight, xbuf, N, M, out_torch_dtype):
    """Product against product: the matmul with the all-gather fused into the kernel (FusedGather: one eager
    call and one replay of a captured CUDA graph) beside the plain matmul of the same weight shard followed
    by NCCL's all-gather, on the same inputs.  The caller passes activations that differ from those of the
    calls before, so a mailbox word left over from an earlier call cannot pass for this call's.  Returns
    the differences; `ok` is what the bench fails on."""
    import torch
    import torch.distributed as dist

    from llm_rs_b200 import DType
    per = N // world
    ldt = DType.F32 if out_torch_dtype == torch.float32 else DType.BF16
    local = torch.empty(M, per, device=dev, dtype=out_torch_dtype)
    lbuf = be.wrap(local.data_ptr(), [per] if M == 1 else [per, M], ldt, keepalive=local)
    gathered = torch.empty(world, M, per, device=dev, dtype=out_torch_dtype)
    be.matmul(lbuf, weight, xbuf)
    dist.all_gather_into_tensor(gathered.view(-1), local.view(-1))
    stream.synchronize()
    ref = gathered.permute(1, 0, 2).reshape(M, N).float()
    fused.out.zero_()
    stream.synchronize()
    dist.barrier()
    eager = fused(weight, xbuf).clone()
    stream.synchronize()
    dist.barrier()
    res = {}
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fused(weight, xbuf)
        fused.out.zero_()
        stream.synchronize()
        dist.barrier()
        g.replay()
        stream.synchronize()
        replay = fused.out.clone()
    except Exception as e:  # noqa: BLE001
        replay = None
        res["graph"] = f"not captured: {e!r}"
    scale = float(ref.abs().max())
    lim = 2.0 ** -7 if out_torch_dtype == torch.bfloat16 else (2e-4 if M <= 64 else 4e-3)
    ok = True
    for name, got in (("eager", eager), ("graph_replay", replay)):
        if got is None:
            continue
        d = (got.float() - ref).abs()
        res[name] = {"bit_equal": bool(torch.equal(got.float(), ref)), "max_diff_over_max": float(d.max()) / max(scale, 1e-30),
                     "rel_l2": float(d.norm() / ref.norm().clamp_min(1e-30))}
        ok = ok and res[name]["max_diff_over_max"] <= lim and bool(torch.isfinite(got.float()).all())
    res["limit_max_diff_over_max"] = lim
    res["ok"] = ok
    t = torch.tensor([0.0 if ok else 1.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)                  # every rank checked its own copy
    res["ok_all_ranks"] = float(t.item()) == 0.0
    lbuf.free()
    return res


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    from llm_rs_b200 import CudaBackend, DType, TensorView, synth
    from llm_rs_b200.shard import row_range

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    stream = torch.cuda.Stream(device=dev)
    M = args.tokens
    a, b = row_range(N_OUT, rank, world)
    n_local = b - a
    peak_gbs, peak_kind = measured_peaks()

    with torch.cuda.stream(stream):
        be = CudaBackend(local_rank, stream=stream.cuda_stream)
        w_host = synth.weight(Q6K, K_IN, N_OUT, tid=2, rows=(a, b))
        shard_bytes = w_host.nbytes
        # Distinct copies of the shard, rotated per step, keep the working set above L2.
        copies = max(1, int(np.ceil(3.2 * L2_BYTES / shard_bytes))) if shard_bytes < 3.2 * L2_BYTES else 1
        weights = [be.upload_tensor(TensorView("output.weight", DType.Q6K, [K_IN, n_local], w_host))
                   for _ in range(copies)]
        x_host = synth.activations(M, K_IN, tid=3)
        x_pinned = torch.from_numpy(x_host.copy()).pin_memory()
        x_dev = torch.from_numpy(x_host).to(dev)
        xbuf = be.wrap(x_dev.data_ptr(), [K_IN] if M == 1 else [K_IN, M], DType.F32, keepalive=x_dev)

        per = N_OUT // world
        full = torch.zeros(M, N_OUT, device=dev, dtype=torch.float32)
        if M == 1 or world == 1:
            local = full[:, a:b] if world > 1 else full
            gathered = None
        else:
            local = torch.empty(M, per, device=dev, dtype=torch.float32)
            gathered = torch.empty(world, M, per, device=dev, dtype=torch.float32)
        obuf = be.wrap(local.data_ptr(), [n_local] if M == 1 else [n_local, M], DType.F32, keepalive=local)
        out_pinned = torch.empty(M, N_OUT, dtype=torch.float32).pin_memory()

        # With more than one GPU and a decode batch the all-gather is fused into the kernel (peer stores
        # over NVLink, llm_rs_b200/shard.py: FusedGather); NCCL remains the fallback.
        fused = None
        exchange = "none"
        if world > 1:
            exchange = "NCCL all-gather of output slices"
            if M <= 4 and not args.nccl:
                try:
                    from llm_rs_b200.shard import FusedGather
                    fused = FusedGather(be, N_OUT, M)
                    full = None
                    exchange = "all-gather fused into the kernel (peer stores over NVLink)"
                except Exception as e:  # noqa: BLE001
                    print(f"[bench] fused all-gather unavailable ({e!r}); using NCCL", file=sys.stderr)
                    fused = None

        def gather():
            if world == 1:
                return
            if M == 1:
                dist.all_gather_into_tensor(full.view(-1), local.reshape(-1))
            else:
                dist.all_gather_into_tensor(gathered.view(-1), local.reshape(-1))
                full.view(M, world, -1).copy_(gathered.permute(1, 0, 2))

        last = {"out": full}

        def step(i):
            if fused is not None:
                last["out"] = fused(weights[i % copies], xbuf)
            else:
                be.matmul(obuf, weights[i % copies], xbuf)
                gather()

        def step_e2e(i):
            be.write(xbuf, x_pinned.numpy())                       # H2D of this step's activations
            step(i)
            out_pinned.copy_(last["out"], non_blocking=True)       # D2H of the step's result
            stream.synchronize()

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(dev)

        def timed(fn, steps, warmup):
            for i in range(warmup):
                fn(i)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(steps):
                fn(warmup + i)
            e1.record(stream)
            barrier()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms / steps

        def timed_in_graphs(fn, steps, warmup):
            """The same K steps, enqueued as replays of one CUDA graph that holds sixteen or more of them (whole
            rotations of the weight copies) plus an eager remainder: with several GPUs a step is 20-40 us
            of device time and the Python call that launches it is no shorter, so eager timing measures
            the host.  Returns (ms per step, steps per graph)."""
            for i in range(warmup):
                fn(i)
            per_graph = copies * max(1, -(-16 // copies))   # whole rotations, sixteen steps at least
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(per_graph):
                    fn(i)
            graph.replay()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps // per_graph):
                graph.replay()
            for i in range(steps % per_graph):
                fn(i)
            e1.record(stream)
            barrier()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms / steps, per_graph

        sampler = ClockSampler(local_rank)
        sampler.start()
        n0 = be.launch_count()
        ms_step = timed(step, args.steps, max(args.warmup, 3))
        launches = be.launch_count() - n0 - max(args.warmup, 3)
        timing = "eager launches"
        try:
            ms_graph, per_graph = timed_in_graphs(step, args.steps, max(args.warmup, 3))
            if ms_graph < ms_step:
                timing = (f"{args.steps // per_graph} replays of a CUDA graph of {per_graph} steps"
                          f" + {args.steps % per_graph} eager steps (eager launches: {ms_step * 1e3:.1f} us per step)")
                ms_step = ms_graph
            else:
                timing = f"eager launches (in CUDA graphs of {per_graph} steps: {ms_graph * 1e3:.1f} us per step)"
        except Exception as e:  # noqa: BLE001
            print(f"[bench] graph timing unavailable ({e!r}); keeping the eager figure", file=sys.stderr)
        # the dominant kernel alone (no collective), same rotation: its launch duration
        ms_kernel = timed(lambda i: be.matmul(obuf, weights[i % copies], xbuf), args.steps, 3)
        ms_e2e = timed(step_e2e, args.steps, max(args.warmup, 3))
        # keep the GPU busy long enough for the clock sampler to see it under this load
        t_end = time.perf_counter() + 1.0
        i = 0
        while time.perf_counter() < t_end:
            for _ in range(200):
                step(i)
                i += 1
            stream.synchronize()
        clocks = sampler.stop()
        be.sync()

        # correctness guard: a sample of rows against the CPU checker would import the oracle,
        # which only the cpu_baseline leg may do; here make sure the output is live, and on several
        # GPUs hold the fused exchange against matmul + NCCL all-gather on fresh activations.
        final = last["out"]
        assert bool(torch.isfinite(final).all()) and float(final.abs().sum()) > 0.0
        gather_check = None
        if fused is not None:
            x_dev.copy_(torch.from_numpy(synth.activations(M, K_IN, tid=77)).to(dev))
            gather_check = allgather_check(be, stream, dev, world, fused, weights[0], xbuf, N_OUT, M, torch.float32)
            x_dev.copy_(torch.from_numpy(x_host).to(dev))
            stream.synchronize()

        multi = None
        if world > 1 and not args.no_extra:
            for b in weights:
                b.free()
            multi = multi_gpu_stacks(be, stream, dev, rank, world, peak_gbs)

    alg = algorithmic_bytes(Q6K, K_IN, N_OUT, M)
    alg_local = algorithmic_bytes(Q6K, K_IN, n_local, M)
    value = alg / (ms_step * 1e-3) / 1e9
    e2e_value = alg / (ms_e2e * 1e-3) / 1e9
    achieved = alg_local / (ms_kernel * 1e-3) / 1e9

    # DRAM bytes of one launch of the headline kernel (dram__bytes_read.sum + dram__bytes_write.sum of
    # the ncu capture summarised under profiles/), scaled by the rows this GPU holds
    ncu_bytes, ncu_commit = ncu_dram_bytes_per_launch()
    traffic = int(ncu_bytes * n_local / N_OUT) if (M == 1 and ncu_bytes) else None

    checks_ok = (gather_check is None or gather_check["ok_all_ranks"]) and (multi is None or multi.get("allgather_checks_ok", True))
    if rank != 0:
        if not checks_ok:
            sys.exit(3)
        return
    line = {
        "metric": "q6k_gemv_algorithmic_GBps", "value": round(value, 2), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int32+f32",
        "data": "synthetic",
        "config": {"workload": f"configs[1]: Q6_K GEMV K={K_IN} N={N_OUT} M={M} (Llama-3-8B output projection)",
                   "parallelism": f"N-split x{world}" + (f" + {exchange}" if world > 1 else ""),
                   "rows_per_gpu": n_local,
                   "l2": (f"inputs larger than L2: the {shard_bytes / 1e6:.0f} MB weight shard is streamed every step "
                          f"(L2 is 126 MB)" if copies == 1 else
                          f"inputs larger than L2: {copies} distinct copies of the {shard_bytes / 1e6:.0f} MB weight "
                          f"shard per GPU, rotated per step (L2 is 126 MB)"),
                   "algorithmic_bytes_per_step": alg, "timing": timing},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak_gbs, "unit": "GB/s",
                     "frac": round(achieved / peak_gbs, 4), "traffic": traffic,
                     "kernel": "gemv_kernel (Q6_K, 1 token)", "ms_per_launch": round(ms_kernel, 5),
                     "peak_kind": f"of {peak_kind}", "bytes_per_launch": alg_local,
                     "traffic_source": f"profiles/traffic.json (ncu capture of the kernel at commit {ncu_commit})" if traffic else None},
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": int(x_host.nbytes),
                "d2h_bytes_per_step": int(M * N_OUT * 4), "ms_per_step": round(ms_e2e, 5),
                "note": ("one public-API call per step with host buffers: a 16 KB host-to-device write of the activations, the "
                         "kernel, a 513 KB device-to-host read of the logits and a stream synchronisation; at one token the "
                         "copies and the synchronisation are ~40 % of the step, so this is a host-interface figure, not a kernel one")},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        gbs, per_s, info = cpu_baseline(Q6K, K_IN, N_OUT, M, budget_s=10.0)
        line["cpu_baseline"] = {"value": round(gbs, 3), "unit": "GB/s", **info}
        line["cpu_baseline"]["other_configs"] = cpu_baselines_other_configs()
    if gather_check is not None:
        line["allgather_check"] = gather_check
    if multi is not None:
        line["extra"] = multi
    if world == 1 and not args.no_extra:
        line["extra"] = extra_measurements(be_factory=lambda: CudaBackend(local_rank, stream=stream.cuda_stream),
                                           stream=stream, peak_gbs=peak_gbs)
    print(json.dumps(line), flush=True)
    if not checks_ok:
        print("[bench] the fused all-gather disagrees with matmul + NCCL all-gather: see allgather_check", file=sys.stderr)
        sys.exit(3)


def multi_gpu_stacks(be, stream, dev, rank, world, peak_gbs):
    """Configs 4 and 5 on `world` GPUs: the linear stack of one decode / prefill step of an 8B- and a
    70B-shaped model, every weight N-sharded (rank g keeps rows [g N/G, (g+1) N/G)), activations
    replicated, each matmul followed by the all-gather of its output slices -- fused into the decode
    kernel up to 4 tokens, NCCL above.  One CUDA graph per step where capture works.  All ranks run
    this; the caller prints rank 0's result.  Times are CUDA events on the stream, max over ranks."""
    import torch
    import torch.distributed as dist

    from llm_rs_b200 import DType, TensorView, synth
    from llm_rs_b200.shard import FusedGather, row_range
    tf_peak = 1658.7
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tf_peak = float(json.load(f).get("bf16_tflops", tf_peak))
    except Exception:  # noqa: BLE001
        pass
    models = {
        "config4_llama8b": dict(hidden=4096, kv=1024, ffn=14336, vocab=128256, layers=32, Ms=(1, 4, 16, 64)),
        "config5_llama70b": dict(hidden=8192, kv=1024, ffn=28672, vocab=128256, layers=80, Ms=(1, 64, 512, 4096)),
    }
    out = {"n_gpus": world, "note": ("linear stack only (7 matmuls per layer + output projection, bf16 activations); "
                                      "weights N-sharded, activations replicated, all-gather of every output: fused "
                                      "into the kernel (peer mailboxes) where a rank receives <= 256 K values per matmul "
                                      "and M <= 128, NCCL elsewhere; no_exchange = the same matmuls without the "
                                      "all-gather")}
    for name, cfg in models.items():
        H, KV, F, V, L = cfg["hidden"], cfg["kv"], cfg["ffn"], cfg["vocab"], cfg["layers"]
        layer = [(Q4K, H, H), (Q4K, H, KV), (Q4K, H, KV), (Q4K, H, H), (Q4K, H, F), (Q4K, H, F), (Q6K, F, H)]
        per_gpu = sum((N // world) * (K // 256) * BLOCK_BYTES[dt] for dt, K, N in layer)
        n_sets = int(min(8, max(2, np.ceil(4 * L2_BYTES / per_gpu))))        # rotated so weights come from HBM
        host = []
        for i, (dt, K, N) in enumerate(layer):
            a, b = row_range(N, rank, world)
            host.append(synth.weight(dt, K, N, tid=400 + i, rows=(a, b)))
        sets = [[be.upload_tensor(TensorView("w", DType(dt), [K, N // world], h)) for (dt, K, N), h in zip(layer, host)]
                for _ in range(n_sets)]
        a, b = row_range(V, rank, world)
        wout = be.upload_tensor(TensorView("w", DType.Q6K, [H, V // world], synth.weight(Q6K, H, V, tid=450, rows=(a, b))))
        del host
        weight_bytes = L * sum(N * (K // 256) * BLOCK_BYTES[dt] for dt, K, N in layer) + V * (H // 256) * 210
        flops_per_token = 2.0 * (L * sum(K * N for _, K, N in layer) + H * V)
        res = {}
        for M in cfg["Ms"]:
            shp = (lambda d: [d] if M == 1 else [d, M])
            xs = {K: be.upload_tensor(TensorView("x", DType.BF16, shp(K), synth.bf16_bits(synth.activations(M, K, tid=K))))
                  for K in (H, F)}
            dims = sorted({N for _, _, N in layer} | {V})
            locals_ = {N: torch.empty(M, N // world, device=dev, dtype=torch.bfloat16) for N in dims}
            lbufs = {N: be.wrap(t.data_ptr(), shp(N // world), DType.BF16, keepalive=t) for N, t in locals_.items()}
            # the fused exchange where one launch holds all tokens' staged activations, NCCL elsewhere
            # fused where the exchange is latency (few words per peer), NCCL where it is volume
            kinds = {(dt, K, N) for dt, K, N in layer + [(Q6K, H, V)]}
            fits = {(dt, K, N) for dt, K, N in kinds
                    if be.allgather_max_tokens(DType(dt), K) >= M and (world - 1) * M * (N // world) <= FUSED_GATHER_MAX_WORDS}
            fused = {N: FusedGather(be, N, M, out_dtype=torch.bfloat16) for N in dims} if fits else None
            fulls = {N: torch.empty(world, M, N // world, device=dev, dtype=torch.bfloat16) for N in dims}

            def step(exchange=True):
                for l in range(L):
                    for (dt, K, N), w in zip(layer, sets[l % n_sets]):
                        run_one(w, dt, K, N, exchange)
                run_one(wout, Q6K, H, V, exchange)

            def run_one(w, dt, K, N, exchange):
                if exchange and (dt, K, N) in fits:
                    fused[N](w, xs[K])
                else:
                    be.matmul(lbufs[N], w, xs[K])
                    if exchange:
                        dist.all_gather_into_tensor(fulls[N].view(-1), locals_[N].view(-1))

            def timed(exchange, reps):
                step(exchange)
                stream.synchronize()
                runner = lambda: step(exchange)
                graph = None
                try:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        step(exchange)
                    runner = graph.replay
                except Exception as e:  # noqa: BLE001
                    graph = None
                    if rank == 0:
                        print(f"[bench] no CUDA graph for {name} M={M} ({e!r}); timing eager launches", file=sys.stderr)
                    torch.cuda.synchronize(dev)
                runner()
                dist.barrier()
                torch.cuda.synchronize(dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(reps):
                    runner()
                e1.record(stream)
                e1.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return float(t.item()) * 1e-3, graph is not None

            reps = 10 if M <= 64 else (3 if M <= 512 else 2)
            t, graphed = timed(True, reps)
            t0, _ = timed(False, reps)
            # the fused exchange against matmul + NCCL all-gather, once per kind of matrix, on other activations
            checks = {}
            if fits:
                xs2 = {K: be.upload_tensor(TensorView("x", DType.BF16, shp(K), synth.bf16_bits(synth.activations(M, K, tid=7000 + K))))
                       for K in (H, F)}
                for (dt, K, N) in sorted(fits):
                    w = wout if N == V else sets[0][[i for i, k in enumerate(layer) if k == (dt, K, N)][0]]
                    c = allgather_check(be, stream, dev, world, fused[N], w, xs2[K], N, M, torch.bfloat16)
                    checks[f"{'q4k' if dt == Q4K else 'q6k'}_{K}x{N}"] = c
                    out["allgather_checks_ok"] = out.get("allgather_checks_ok", True) and c["ok_all_ranks"]
                for bfr in xs2.values():
                    bfr.free()
            res[f"m{M}"] = {"ms_per_step": round(t * 1e3, 4), "ms_no_exchange": round(t0 * 1e3, 4),
                            "tok_per_s": round(M / t, 1),
                            "weight_GBps": round(weight_bytes / t / 1e9, 1),
                            "frac_of_hbm_peak_x_gpus": round(weight_bytes / t / 1e9 / (peak_gbs * world), 4),
                            "TFLOPs": round(flops_per_token * M / t / 1e12, 1),
                            "frac_of_tensor_peak_x_gpus": round(flops_per_token * M / t / 1e12 / (tf_peak * world), 4),
                            "exchange": ("fused peer stores" if fits == kinds else
                                         "fused peer stores where a rank receives <= 256 K values per matmul, NCCL all-gather elsewhere" if fits
                                         else "NCCL all-gather"),
                            "cuda_graph": graphed, "allgather_check": checks}
            for bfr in list(xs.values()) + list(lbufs.values()):
                bfr.free()
            del fused, fulls, locals_
            torch.cuda.synchronize(dev)
        for st in sets:
            for bfr in st:
                bfr.free()
        wout.free()
        out[name] = res
    return out


def extra_measurements(be_factory, stream, peak_gbs):
    """The other parts of the headline metric, kernel-only (device-resident inputs, CUDA-event time
    from the context, weights rotated so every launch reads them from HBM, not L2):
    decode GEMV at the reference bench's shapes, config 2 at M in {8, 32, 64}, the prefill GEMMs of
    config 3, and the linear stack of one 8B decode step (config 4)."""
    import torch

    from llm_rs_b200 import DType, TensorView, synth
    tf_peak = 1658.7
    ppath = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(ppath):
        with open(ppath) as f:
            tf_peak = float(json.load(f).get("bf16_tflops", tf_peak))
    out = {"gemv": {}, "gemm": {}, "decode_stack": {}, "peaks": {"hbm_gbs": peak_gbs, "dense_16bit_tflops": tf_peak}}
    with torch.cuda.stream(stream):
        be = be_factory()

        def time_matmul(dt, K, N, M, in_dt, out_dt, iters):
            w = synth.weight(dt, K, N, tid=5)
            copies = min(48, max(1, int(np.ceil(3.2 * L2_BYTES / w.nbytes))))
            ws = [be.upload_tensor(TensorView("w", DType(dt), [K, N], w)) for _ in range(copies)]
            xh = synth.activations(M, K)
            x = be.upload_tensor(TensorView("x", in_dt, [K] if M == 1 else [K, M],
                                            synth.bf16_bits(xh) if in_dt == DType.BF16 else xh))
            o = be.alloc([N] if M == 1 else [N, M], out_dt)
            for i in range(5):
                be.matmul(o, ws[i % copies], x)
            be.sync()
            be.reset_gpu_secs()
            n0 = be.launch_count()
            for i in range(iters):
                be.matmul(o, ws[i % copies], x)
            be.sync()
            t = be.gpu_secs_total() / iters
            time_matmul.launches_per_call = (be.launch_count() - n0) / iters
            for b in ws + [x, o]:
                b.free()
            return t

        for name, dt, K, N, Ms in (("q4k_4096x4096", Q4K, 4096, 4096, (1,)),
                                   ("q4k_4096x1024", Q4K, 4096, 1024, (1,)),
                                   ("q4k_4096x14336", Q4K, 4096, 14336, (1,)),
                                   ("q6k_14336x4096", Q6K, 14336, 4096, (1,)),
                                   ("q4k_4096x128256", Q4K, 4096, 128256, (1,)),
                                   ("q4k_4096x4096", Q4K, 4096, 4096, (16, 64)),
                                   ("q4k_4096x14336", Q4K, 4096, 14336, (16, 64)),
                                   ("q6k_14336x4096", Q6K, 14336, 4096, (16, 64)),
                                   ("q4k_4096x128256", Q4K, 4096, 128256, (8, 32, 64)),
                                   ("q6k_4096x128256", Q6K, 4096, 128256, (1, 2, 4, 8, 16, 32, 64))):
            for M in Ms:
                t = time_matmul(dt, K, N, M, DType.F32, DType.F32, 50 if N >= 100000 else 200)
                alg = algorithmic_bytes(dt, K, N, M)
                out["gemv"][f"{name}_m{M}"] = {"us": round(t * 1e6, 2), "GBps": round(alg / t / 1e9, 1),
                                               "frac_of_hbm_peak": round(alg / t / 1e9 / peak_gbs, 4),
                                               # one launch per call: the decode kernel; two: conversion + tensor-core kernel
                                               "kernel": "decode kernel (dp4a, fixed-point activations)"
                                               if time_matmul.launches_per_call < 1.5
                                               else "small-batch tensor-core kernel (exact integer operands, 1e-4 class)"}
        # the same output projection on the one-term tensor-core kernel (2e-3 class; LLMRS_TC_TWO_TERM=0)
        os.environ["LLMRS_TC_TWO_TERM"] = "0"
        try:
            be_two, be = be, be_factory()
        finally:
            del os.environ["LLMRS_TC_TWO_TERM"]
        for M in (8, 32, 64):
            t = time_matmul(Q6K, 4096, 128256, M, DType.F32, DType.F32, 50)
            alg = algorithmic_bytes(Q6K, 4096, 128256, M)
            out["gemv"][f"q6k_4096x128256_m{M}_one_term"] = {
                "us": round(t * 1e6, 2), "GBps": round(alg / t / 1e9, 1),
                "frac_of_hbm_peak": round(alg / t / 1e9 / peak_gbs, 4), "kernel": "tensor-core f16, one term (2e-3 class)"}
        be.close()
        be = be_two
        # config 3: Q4_K 4096 -> 14336 then Q6_K 14336 -> 4096, bf16 activations in and out
        for M in (128, 512, 2048):
            for name, dt, K, N in (("q4k_4096x14336", Q4K, 4096, 14336), ("q6k_14336x4096", Q6K, 14336, 4096)):
                t = time_matmul(dt, K, N, M, DType.BF16, DType.BF16, 30)
                fl = 2.0 * M * K * N
                out["gemm"][f"{name}_m{M}"] = {"us": round(t * 1e6, 1), "TFLOPs": round(fl / t / 1e12, 1),
                                               "frac_of_tensor_peak": round(fl / t / 1e12 / tf_peak, 4)}
        # next rows: the feed-forward front as one call, and the embedding lookup
        out["ffn_front"], out["embed"] = {}, {}
        wg = [be.upload_tensor(TensorView("w", DType.Q4K, [4096, 14336], synth.weight(Q4K, 4096, 14336, tid=60 + i)))
              for i in range(8)]                      # 4 gate/up pairs, 264 MB: rotated, so they come from HBM
        for M in (1, 4):
            x = be.upload_tensor(TensorView("x", DType.BF16, [4096] if M == 1 else [4096, M],
                                            synth.bf16_bits(synth.activations(M, 4096))))
            o = be.alloc([14336] if M == 1 else [14336, M], DType.BF16)
            g = be.alloc([14336] if M == 1 else [14336, M], DType.BF16)
            for fused in (True, False):
                def run(i):
                    a, b = wg[2 * (i % 4)], wg[2 * (i % 4) + 1]
                    if fused:
                        be.matmul_gate_up(o, a, b, x)
                    else:                             # the two matmuls alone: silu and mul would come on top
                        be.matmul(g, a, x)
                        be.matmul(o, b, x)
                for i in range(5):
                    run(i)
                be.sync()
                be.reset_gpu_secs()
                for i in range(100):
                    run(i)
                be.sync()
                t = be.gpu_secs_total() / 100
                wbytes = 2 * 14336 * 16 * 144
                out["ffn_front"][f"q4k_4096x14336_m{M}_{'one_call' if fused else 'two_matmuls'}"] = {
                    "us": round(t * 1e6, 2), "weight_GBps": round(wbytes / t / 1e9, 1),
                    "frac_of_hbm_peak": round(wbytes / t / 1e9 / peak_gbs, 4)}
            for b in (x, o, g):
                b.free()
        for b in wg:
            b.free()
        rng = np.random.default_rng(5)
        for name, dt, bb in (("q4k", Q4K, 144), ("q6k", Q6K, 210)):
            vocab, dim, ntok = 128256, 4096, 2048
            table = be.upload_tensor(TensorView("t", DType(dt), [dim, vocab], synth.weight(dt, dim, vocab, tid=70)))
            toks = rng.integers(0, vocab, ntok).astype(np.uint32)
            o = be.alloc([dim, ntok], DType.BF16)
            for _ in range(3):
                be.embed(o, table, toks)
            be.sync()
            be.reset_gpu_secs()
            for _ in range(20):
                be.embed(o, table, toks)
            be.sync()
            t = be.gpu_secs_total() / 20
            nbytes = ntok * (dim // 256) * bb + ntok * dim * 2
            out["embed"][f"{name}_dim4096_tokens2048"] = {"us": round(t * 1e6, 2), "GBps": round(nbytes / t / 1e9, 1),
                                                          "frac_of_hbm_peak": round(nbytes / t / 1e9 / peak_gbs, 4)}
            table.free()
            o.free()
        # the other ops of a decode step (8B shapes): time per call, and attention's KV bytes per second
        out["other_ops"] = {}

        def time_call(fn, iters=50):
            for _ in range(3):
                fn()
            be.sync()
            be.reset_gpu_secs()
            for _ in range(iters):
                fn()
            be.sync()
            return be.gpu_secs_total() / iters

        hd, nh, nkv, blk = 128, 32, 8, 256
        xa = be.upload_tensor(TensorView("x", DType.BF16, [4096], synth.bf16_bits(synth.activations(1, 4096, tid=9))))
        xo = be.alloc([4096], DType.BF16)
        nw = be.upload_tensor(TensorView("w", DType.F32, [4096], np.ones(4096, np.float32)))
        out["other_ops"]["rms_norm_4096_us"] = round(time_call(lambda: be.rms_norm(xo, xa, nw, 1e-5)) * 1e6, 2)
        out["other_ops"]["add_4096_us"] = round(time_call(lambda: be.add(xo, xa, xa)) * 1e6, 2)
        kx = be.upload_tensor(TensorView("k", DType.BF16, [1024], synth.bf16_bits(synth.activations(1, 1024, tid=8))))
        pos = be.upload_u32([4095])
        out["other_ops"]["rope_q4096_k1024_us"] = round(time_call(lambda: be.rope(xa, kx, pos, hd, 500000.0)) * 1e6, 2)
        for name, n_req, ctx_len, q_per in (("decode_8x4096", 8, 4096, 1), ("prefill_1x512", 1, 512, 512),
                                             ("prefill_1x2048", 1, 2048, 2048)):
            pages_per = (ctx_len + blk - 1) // blk
            n_slots = n_req * pages_per * blk
            kp = be.upload_tensor(TensorView("k", DType.BF16, [nkv * hd, n_slots],
                                             synth.bf16_bits(synth.activations(n_slots, nkv * hd, tid=11))))
            vp = be.upload_tensor(TensorView("v", DType.BF16, [nkv * hd, n_slots],
                                             synth.bf16_bits(synth.activations(n_slots, nkv * hd, tid=12))))
            tq = n_req * q_per
            qb = be.upload_tensor(TensorView("q", DType.BF16, [nh * hd] if tq == 1 else [nh * hd, tq],
                                             synth.bf16_bits(synth.activations(tq, nh * hd, tid=13))))
            ob = be.alloc([nh * hd] if tq == 1 else [nh * hd, tq], DType.BF16)
            bt = be.upload_u32(np.arange(n_req * pages_per, dtype=np.uint32))
            qs = be.upload_u32([i * q_per for i in range(n_req + 1)])
            sl = be.upload_u32([ctx_len] * n_req)
            t = time_call(lambda: be.attention(ob, qb, kp, vp, bt, qs, sl, nh, nkv, hd, blk, pages_per), 10)
            kv_bytes = 2 * n_req * ctx_len * nkv * hd * 2
            out["other_ops"][f"attention_{name}"] = {"us": round(t * 1e6, 1), "kv_GBps": round(kv_bytes / t / 1e9, 1)}
            if q_per > 1:       # causal: query token i of the request sees ctx_len - q_per + i + 1 positions
                pairs = n_req * (q_per * (ctx_len - q_per) + q_per * (q_per + 1) // 2)
                out["other_ops"][f"attention_{name}"]["TFLOPs"] = round(4.0 * nh * hd * pairs / t / 1e12, 1)
            for b in (kp, vp, qb, ob, bt, qs, sl):
                b.free()
        # config 4: the 225 matmuls of one Llama-3-8B decode step (32 x {wq, wk, wv, wo, gate, up: Q4_K;
        # down: Q6_K} + output: Q6_K), back to back; norms, rope and attention are outside this path.
        layer = [(Q4K, 4096, 4096), (Q4K, 4096, 1024), (Q4K, 4096, 1024), (Q4K, 4096, 4096),
                 (Q4K, 4096, 14336), (Q4K, 4096, 14336), (Q6K, 14336, 4096)]
        lw = [be.upload_tensor(TensorView("w", DType(dt), [K, N], synth.weight(dt, K, N, tid=100 + i)))
              for i, (dt, K, N) in enumerate(layer)]
        n_layer_sets = 4            # 4 distinct layers (551 MB) rotated: > 4x L2, like 32 distinct ones
        sets = [lw] + [[be.upload_tensor(TensorView("w", DType(dt), [K, N], synth.weight(dt, K, N, tid=200 + 10 * j + i)))
                        for i, (dt, K, N) in enumerate(layer)] for j in range(n_layer_sets - 1)]
        wout = be.upload_tensor(TensorView("w", DType.Q6K, [4096, 128256], synth.weight(Q6K, 4096, 128256, tid=300)))
        weight_bytes = 32 * sum(N * (K // 256) * BLOCK_BYTES[dt] for dt, K, N in layer) + 128256 * 16 * 210
        for M in (1, 4, 16, 64):
            shp = (lambda d: [d] if M == 1 else [d, M])
            xs = {4096: be.upload_tensor(TensorView("x", DType.BF16, shp(4096), synth.bf16_bits(synth.activations(M, 4096)))),
                  14336: be.upload_tensor(TensorView("x", DType.BF16, shp(14336), synth.bf16_bits(synth.activations(M, 14336))))}
            outs = {n: be.alloc(shp(n), DType.BF16) for n in (4096, 1024, 14336, 128256)}
            outs_v = be.alloc(shp(1024), DType.BF16)
            norm_w = be.upload_tensor(TensorView("g", DType.F32, [4096], np.ones(4096, np.float32)))

            def step(one_call_ffn=False, one_call_qkv=False):
                for l in range(32):
                    ws = sets[l % n_layer_sets]
                    for i, ((dt, K, N), wb) in enumerate(zip(layer, ws)):
                        if one_call_qkv and i == 0:          # norm + q, k, v projections as one call
                            be.rms_norm_matmul_qkv(outs[4096], outs[1024], outs_v, ws[0], ws[1], ws[2], xs[K], norm_w, 1e-5)
                        elif one_call_qkv and i in (1, 2):
                            pass
                        elif one_call_ffn and i == 4:        # gate and up (and silu, mul) as one call
                            be.matmul_gate_up(outs[N], ws[4], ws[5], xs[K])
                        elif not (one_call_ffn and i == 5):
                            be.matmul(outs[N], wb, xs[K])
                be.matmul(outs[128256], wout, xs[4096])

            def timed_graph(fn):
                for _ in range(2):
                    fn()
                be.sync()
                # the launches are captured once in a CUDA graph and replayed (matmul only enqueues)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    fn()
                graph.replay()
                stream.synchronize()
                reps = 10
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(reps):
                    graph.replay()
                e1.record(stream)
                stream.synchronize()
                return e0.elapsed_time(e1) * 1e-3 / reps

            t = timed_graph(step)
            t_ffn = timed_graph(lambda: step(True))
            t_both = timed_graph(lambda: step(True, True))
            out["decode_stack"][f"m{M}"] = {"ms_per_step": round(t * 1e3, 4), "tok_per_s": round(M / t, 1),
                                            "weight_GBps": round(weight_bytes / t / 1e9, 1),
                                            "frac_of_hbm_peak": round(weight_bytes / t / 1e9 / peak_gbs, 4),
                                            "matmuls_per_step": 225,
                                            "with_gate_up_as_one_call": {
                                                "ms_per_step": round(t_ffn * 1e3, 4), "tok_per_s": round(M / t_ffn, 1),
                                                "frac_of_hbm_peak": round(weight_bytes / t_ffn / 1e9 / peak_gbs, 4),
                                                "calls_per_step": 193},
                                            "with_norm_qkv_and_gate_up_as_one_call_each": {
                                                "ms_per_step": round(t_both * 1e3, 4), "tok_per_s": round(M / t_both, 1),
                                                "frac_of_hbm_peak": round(weight_bytes / t_both / 1e9 / peak_gbs, 4),
                                                "calls_per_step": 129,
                                                "note": "the q/k/v call also computes the rms_norm in front of them"}}
            for b in list(xs.values()) + list(outs.values()) + [outs_v, norm_w]:
                b.free()
        # A whole decode step of the 8B shape through the trait: per layer rms_norm, q/k/v matmuls, rope,
        # scatter_kv, paged attention, wo matmul, add, rms_norm, gate/up + silu * mul as one call, down
        # matmul, add; then the final norm and the output projection.  One CUDA graph; the embedding
        # lookup before it and the argmax after it move host data and are timed as they are.
        out["decode_step_full"] = {}
        hd, nh, nkv, blk, ctx_len = 128, 32, 8, 256, 1024
        ones = be.upload_tensor(TensorView("n", DType.F32, [4096], np.ones(4096, np.float32)))
        emb = be.upload_tensor(TensorView("e", DType.Q4K, [4096, 32000], synth.weight(Q4K, 4096, 32000, tid=500)))
        for M in (1, 8):
            shp = (lambda d: [d] if M == 1 else [d, M])
            pages_per = (ctx_len + blk) // blk + 1
            n_slots = M * pages_per * blk
            pools = [(be.alloc([nkv * hd, n_slots], DType.BF16), be.alloc([nkv * hd, n_slots], DType.BF16)) for _ in range(32)]
            kv_init = synth.bf16_bits(synth.activations(n_slots, nkv * hd, tid=501) * np.float32(0.3))
            for kp, vp in pools:
                be.write(kp, kv_init)
                be.write(vp, kv_init)
            bt = be.upload_u32(np.arange(M * pages_per, dtype=np.uint32))
            qs = be.upload_u32(list(range(M + 1)))
            sl = be.upload_u32([ctx_len + 1] * M)
            pos = be.upload_u32([ctx_len] * M)
            slots = be.upload_u32([r * pages_per * blk + ctx_len for r in range(M)])
            x, x2, xn = (be.alloc(shp(4096), DType.BF16) for _ in range(3))
            qb, ao, wo_o, ffn_o = (be.alloc(shp(4096), DType.BF16) for _ in range(4))
            kb, vb = be.alloc(shp(1024), DType.BF16), be.alloc(shp(1024), DType.BF16)
            gu, gu2 = be.alloc(shp(14336), DType.BF16), be.alloc(shp(14336), DType.BF16)
            logits = be.alloc(shp(128256), DType.BF16)
            toks = np.arange(M, dtype=np.uint32) + 17

            def layers(fuse=True):
                for l in range(32):
                    wq, wk, wv, wo, w1, w3, w2 = sets[l % n_layer_sets]
                    kp, vp = pools[l]
                    if fuse:                             # the norm inside the decode kernel's staging, q/k/v in one launch
                        be.rms_norm_matmul_qkv(qb, kb, vb, wq, wk, wv, x, ones, 1e-5)
                    else:
                        be.rms_norm(xn, x, ones, 1e-5)
                        be.matmul(qb, wq, xn)
                        be.matmul(kb, wk, xn)
                        be.matmul(vb, wv, xn)
                    if fuse:
                        be.rope_scatter_kv(qb, kb, vb, pos, hd, 500000.0, kp, vp, slots)
                    else:
                        be.rope(qb, kb, pos, hd, 500000.0)
                        be.scatter_kv(kp, kb, slots, nkv * hd, M)
                        be.scatter_kv(vp, vb, slots, nkv * hd, M)
                    be.attention(ao, qb, kp, vp, bt, qs, sl, nh, nkv, hd, blk, pages_per)
                    if fuse:                             # residual adds in the matmul's epilogue, gate/up as one call
                        be.matmul_add(x2, wo, ao, x)
                        be.rms_norm_matmul_gate_up(gu, w1, w3, x2, ones, 1e-5)
                        be.matmul_add(x, w2, gu, x2)
                    else:                                # call for call what src/arch/llama.rs:152-169 makes
                        be.matmul(wo_o, wo, ao)
                        be.add(x2, x, wo_o)
                        be.rms_norm(xn, x2, ones, 1e-5)
                        be.matmul(gu, w1, xn)
                        be.matmul(gu2, w3, xn)
                        be.silu(gu)
                        be.mul(gu, gu, gu2)
                        be.matmul(ffn_o, w2, gu)
                        be.add(x, x2, ffn_o)
                be.rms_norm(xn, x, ones, 1e-5)
                be.matmul(logits, wout, xn)

            be.embed(x, emb, toks)
            t_plain = timed_graph(lambda: layers(False))
            be.embed(x, emb, toks)                       # fresh activations: 32 random layers blow the scale up
            # the one-call forms: inside the decode kernel up to 4 tokens, fewer launches (one norm, one rope + scatter) above
            t_graph = timed_graph(layers)
            be.embed(x, emb, toks)
            be.sync()
            t0 = time.perf_counter()
            for _ in range(5):
                be.embed(x, emb, toks)
                be.argmax(logits) if M == 1 else be.sync()
            t_edges = (time.perf_counter() - t0) / 5
            out["decode_step_full"][f"m{M}_ctx{ctx_len}"] = {
                "ms_graph": round(t_graph * 1e3, 4), "ms_embed_and_argmax_host_timed": round(t_edges * 1e3, 4),
                "tok_per_s": round(M / (t_graph + t_edges), 1), "calls_per_layer": 6,
                "call_for_call_as_the_reference": {"ms_graph": round(t_plain * 1e3, 4), "calls_per_layer": 16,
                                                   "tok_per_s": round(M / (t_plain + t_edges), 1)}}
            for b in [bt, qs, sl, pos, slots, x, x2, xn, qb, ao, wo_o, ffn_o, kb, vb, gu, gu2, logits] + [p for kv in pools for p in kv]:
                b.free()
        out["decode_step_full"]["note"] = ("random weights: the numbers in the activations are meaningless, the work is that "
                                           "of a Llama-3-8B decode step at the stated context; argmax only at one token")
        # a whole prefill pass through the trait: one request of T prompt tokens, call for call as
        # src/arch/llama.rs:150-170 makes them (the logits of the last token only, as a server needs them)
        out["prefill_step_full"] = {}
        for T in (512, 2048):
            pages_per = (T + blk - 1) // blk
            n_slots = pages_per * blk
            pools = [(be.alloc([nkv * hd, n_slots], DType.BF16), be.alloc([nkv * hd, n_slots], DType.BF16)) for _ in range(32)]
            bt = be.upload_u32(np.arange(pages_per, dtype=np.uint32))
            qs, sl = be.upload_u32([0, T]), be.upload_u32([T])
            pos = be.upload_u32(np.arange(T, dtype=np.uint32))
            x, x2, xn, qb, ao, wo_o, ffn_o = (be.alloc([4096, T], DType.BF16) for _ in range(7))
            kb, vb = be.alloc([1024, T], DType.BF16), be.alloc([1024, T], DType.BF16)
            gu, gu2 = be.alloc([14336, T], DType.BF16), be.alloc([14336, T], DType.BF16)
            last, lastn = be.alloc([4096], DType.BF16), be.alloc([4096], DType.BF16)
            last_idx = be.upload_u32([T - 1])
            logits = be.alloc([128256], DType.BF16)
            toks = (np.arange(T, dtype=np.uint32) * 7 + 3) % 32000

            def prefill():
                for l in range(32):
                    wq, wk, wv, wo, w1, w3, w2 = sets[l % n_layer_sets]
                    kp, vp = pools[l]
                    be.rms_norm(xn, x, ones, 1e-5)
                    be.matmul(qb, wq, xn)
                    be.matmul(kb, wk, xn)
                    be.matmul(vb, wv, xn)
                    be.rope_scatter_kv(qb, kb, vb, pos, hd, 500000.0, kp, vp, pos)
                    be.attention(ao, qb, kp, vp, bt, qs, sl, nh, nkv, hd, blk, pages_per)
                    be.matmul(wo_o, wo, ao)
                    be.add(x2, x, wo_o)
                    be.rms_norm(xn, x2, ones, 1e-5)
                    be.matmul_gate_up(gu, w1, w3, xn)
                    be.matmul(ffn_o, w2, gu)
                    be.add(x, x2, ffn_o)
                be.gather(last, x, last_idx, 1)
                be.rms_norm(lastn, last, ones, 1e-5)
                be.matmul(logits, wout, lastn)

            be.embed(x, emb, toks)
            t = timed_graph(prefill)
            out["prefill_step_full"][f"t{T}"] = {"ms_graph": round(t * 1e3, 3), "tok_per_s": round(T / t, 1)}
            for b in [bt, qs, sl, pos, x, x2, xn, qb, ao, wo_o, ffn_o, kb, vb, gu, gu2, last, lastn, last_idx, logits] + [p for kv in pools for p in kv]:
                b.free()
        out["prefill_step_full"]["note"] = ("one request, 8B shapes, random weights, 32 layers in one CUDA graph: norms, q/k/v, "
                                            "rope + KV scatter, causal attention, wo, residuals, gate/up, down; last token's logits")
        out["decode_stack"]["note"] = ("linear stack only (225 matmuls, bf16 activations), one CUDA graph per step; "
                                       "weight bytes per step 4 841 250 816")
        out["gguf_upload"] = gguf_upload_measurement(be)
        be.close()
    return out


def gguf_upload_measurement(be):
    """File -> device through Loader (pinned staging pieces, eight readers) beside upload_tensor from a
    pageable array, on one layer's worth of an 8B model written as a GGUF file to the temp directory
    (so the reads come from the page cache: this times the pipeline, not a disk)."""
    import struct
    import tempfile
    import time

    from llm_rs_b200 import DType, TensorView, synth
    from llm_rs_b200.gguf import GgufFile, Loader

    def s(x):
        return struct.pack("<Q", len(x)) + x

    tensors = [(b"blk.0.ffn_gate.weight", Q4K, 4096, 14336), (b"blk.0.ffn_up.weight", Q4K, 4096, 14336),
               (b"blk.0.ffn_down.weight", Q6K, 14336, 4096), (b"blk.0.attn_q.weight", Q4K, 4096, 4096),
               (b"blk.0.attn_output.weight", Q4K, 4096, 4096), (b"blk.0.attn_v.weight", Q6K, 4096, 1024)]
    blobs = [np.ascontiguousarray(synth.weight(dt, K, N, tid=300 + i)) for i, (_n, dt, K, N) in enumerate(tensors)]
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), 1) + s(b"general.architecture") + struct.pack("<I", 8) + s(b"llama")
    off = 0
    for (name, dt, K, N), blob in zip(tensors, blobs):
        head += s(name) + struct.pack("<IQQIQ", 2, K, N, dt, off)
        off += (blob.nbytes + 31) // 32 * 32
    head += b"\0" * (-len(head) % 32)
    res = {}
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "layer.gguf")
        with open(path, "wb") as f:
            f.write(head)
            for blob in blobs:
                f.write(blob.tobytes())
                f.write(b"\0" * (-blob.nbytes % 32))
        total = sum(b.nbytes for b in blobs)
        with GgufFile.open(path) as g:
            for rep in range(2):                       # the first pass allocates the staging buffers
                ld = Loader(g, be)
                t0 = time.perf_counter()
                bufs = [ld.req(name.decode()) for name, *_ in tensors]
                dt_s = time.perf_counter() - t0
                for b in bufs:
                    b.free()
            res["file_to_device"] = {"MB": round(total / 1e6, 1), "ms": round(dt_s * 1e3, 2), "GBps": round(total / dt_s / 1e9, 2)}
        t0 = time.perf_counter()
        bufs = [be.upload_tensor(TensorView(name.decode(), DType(dt), [K, N], blob)) for (name, dt, K, N), blob in zip(tensors, blobs)]
        dt_s = time.perf_counter() - t0
        for b in bufs:
            b.free()
        res["upload_tensor_from_pageable_host"] = {"ms": round(dt_s * 1e3, 2), "GBps": round(total / dt_s / 1e9, 2)}
    res["note"] = "wall clock, file in the page cache; Q6_K re-laid out on the device in both"
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=1, help="M, decode batch (1..64)")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the other parts of the metric (other GEMV shapes, prefill GEMM TFLOP/s, decode stack)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--nccl", action="store_true", help="N>1: use the NCCL all-gather instead of the fused one")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()

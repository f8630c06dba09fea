#!/usr/bin/env python
"""Benchmark of the B200 backend for the Wave GEMM / flash-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemm|fa|skinny]
                    [--impl ours|reference] [--gather]

One "step" is one pass of the hot path over one batch of synthetic input.  The
headline workload (default) is the bf16 GEMM M=N=K=8192 with f32 accumulation
and bf16 output; with N GPUs every rank owns one 8192-column block of a C that
is N times wider (weak scaling, no collective in the timed region; --gather
adds and separately times the NCCL all-gather of C).  `--workload fa` is the
causal flash-attention forward B=16 H=32 S=4096 D=128 (batch x head sharded),
`--workload skinny` the M=16, N=28672, K=8192 decode-shaped GEMM.  The default
run also measures the other two workloads briefly and reports them under
"also".  Prints ONE JSON line on rank 0.

`--impl reference` times the reference's own CPU implementation of the same
path (its calibrate runner's host code compiled as a shared object, else the
restated oracle) on a bounded sample of the workload, using all host threads.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "TFLOP/s + % tensor roofline: GEMM 8192^3 bf16, FA-fwd S=4096 d=128 @1/2/4/8 B200"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch from one ncu capture of
# the same kernel (summaries under profiles/): gemm and skinny at full size; fa
# captured at B=2 (250.58 MB) and scaled by the 8x heads of the B=16 workload,
# since every head moves the same bytes; fa_published at full size.
NCU_TRAFFIC_BYTES = {"gemm": 1203.57e6, "fa": 8 * 251.89e6, "skinny": 477.11e6, "fa_published": 1055.49e6}

WORKLOADS = {
    "gemm": dict(name="gemm_bf16_8192x8192x8192_f32acc_bf16out", M=8192, N=8192, K=8192),
    "skinny": dict(name="gemm_bf16_16x28672x8192_f32acc_bf16out_streamk", M=16, N=28672, K=8192),
    "fa": dict(name="fa_fwd_causal_bf16_b16_h32_s4096_d128", B=16, H=32, S=4096, D=128),
    # The configuration the reference's own attention number is published on
    # (docs/PerfReferences/WaveGfx950FlashAttention.md:39-44): non-causal, fixed
    # softmax reference for |Q|,|K| <= 1, inputs of its runner's range.
    "fa_published": dict(name="fa_fwd_noncausal_bf16_b2_h64_s8192_d128_qk_max_abs_1", B=2, H=64, S=8192, D=128,
                         causal=False, qk_max_abs=1.0, published_tflops=1115.6),
}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


# ----------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed
    region runs (reading only; no setting is changed)."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, t_begin: float | None = None, t_end: float | None = None) -> dict:
        """Summarises the samples whose timestamp falls inside [t_begin, t_end]
        (host wall-clock seconds); all samples if no window is given or none
        fell inside it."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime
        rows = []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[1]), float(parts[2]),
                             [n for n, v in zip(names, parts[3:7]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if t_begin is not None and t_begin <= r[0] <= t_end]
        window = "timed region" if inside else "whole run"
        use = inside or rows
        reasons = sorted({n for r in use for n in r[3]})
        return {"sm_mhz": statistics.median([r[1] for r in use]) if use else None,
                "sm_max_mhz": max([r[2] for r in use]) if use else None,
                "reasons": reasons, "samples": len(use), "window": window}


# ----------------------------------------------------------------------------
# workloads on the GPU
# ----------------------------------------------------------------------------
class GemmWork:
    def __init__(self, torch, wc, M, N, K, rank, world, seed=0, streamk=1):
        self.torch, self.wc = torch, wc
        self.M, self.N, self.K = M, N, K
        g = torch.Generator(device="cuda")
        g.manual_seed(1234 + seed)
        # A is replicated across ranks (same seed); each rank has its own B block.
        self.a = (torch.randn(M, K, device="cuda", generator=g) * (K ** -0.5 if M > 16 else 1.0)).to(torch.bfloat16)
        g.manual_seed(4321 + seed + 977 * rank)
        self.b = (torch.randn(N, K, device="cuda", generator=g) * K ** -0.5).to(torch.bfloat16)
        self.c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        knobs = dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4) if M % 256 == 0 else dict(bn=1)
        self.desc = wc.gemm_desc(M, N, K, in_type=wc.BF16, out_type=wc.BF16, streamk_workers=streamk, **knobs)
        s, c = wc.gemm_workspace_bytes(self.desc)
        self.ws = torch.zeros(s + c, dtype=torch.uint8, device="cuda") if s + c else None
        self.flops = 2.0 * M * N * K
        self.alg_bytes = 2.0 * (M * K + N * K + M * N)
        self.launches_per_step = 1
        self.h2d = 2 * (M * K + N * K)
        self.d2h = 2 * M * N
        self.host = None

    def step(self, stream):
        self.wc.gemm(self.desc, self.a.data_ptr(), self.b.data_ptr(), self.c.data_ptr(),
                     self.ws.data_ptr() if self.ws is not None else 0, stream)

    def prepare_host(self):
        t = self.torch
        self.host = (self.a.cpu().pin_memory(), self.b.cpu().pin_memory(),
                     t.empty(self.M, self.N, dtype=t.bfloat16).pin_memory())

    def step_host(self, stream):
        a, b, c = self.host
        self.wc.gemm_host(self.desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream)

    def check(self, oracle) -> float:
        """Sampled parity check outside the timed region: a few rows against the
        CPU oracle (f32 accumulate, k ascending)."""
        rows = np.unique(np.linspace(0, self.M - 1, 8).astype(np.int32))
        a = self.a.cpu().view(self.torch.int16).numpy().view(np.uint16)
        b = self.b.cpu().view(self.torch.int16).numpy().view(np.uint16)
        want = oracle.round_output(oracle.gemm_ref(a, b, oracle.BF16, rows=rows), "bf16")
        got = self.c.float().cpu().numpy()[rows]
        return float(np.max(np.abs(got - want) / (1.0e-2 + 2.0 ** -7 * np.abs(want))))


class FaWork:
    def __init__(self, torch, wc, B, H, S, D, rank, world, seed=0, causal=True, qk_max_abs=0.0):
        self.torch, self.wc = torch, wc
        self.B, self.H, self.S, self.D, self.causal = B, H, S, D, causal
        g = torch.Generator(device="cuda")
        g.manual_seed(99 + seed + 131 * rank)
        if qk_max_abs > 0.0:
            # the value set of the reference runner's generator (17 buckets, Q/K x0.125, V x0.25;
            # wave-fa-gfx950-runner.cpp:188-202), drawn from torch's generator
            mk = lambda scale: (torch.randint(-8, 9, (B * H, S, D), device="cuda", generator=g).float()
                                * scale).to(torch.bfloat16)
            self.q, self.k, self.v = mk(0.125), mk(0.125), mk(0.25)
        else:
            mk = lambda: torch.randn(B * H, S, D, device="cuda", generator=g).to(torch.bfloat16)
            self.q, self.k, self.v = mk(), mk(), mk()
        self.o = torch.empty_like(self.q)
        self.desc = wc.fa_desc(B, H, S, S, D, causal=causal, io_type=wc.BF16, qk_max_abs=qk_max_abs)
        # unmasked pairs only for the causal case; the reference's own formula
        # (4*B*H*S^2*D, wave-fa-gfx950-runner.cpp:465-466) counts the full square
        pairs = S * (S + 1) / 2 if causal else float(S) * S
        self.flops = 4.0 * B * H * D * pairs
        self.flops_full_square = 4.0 * B * H * D * float(S) * S
        self.alg_bytes = 4.0 * B * H * S * D * 2
        self.launches_per_step = 1
        self.h2d = 3 * B * H * S * D * 2
        self.d2h = B * H * S * D * 2
        self.host = None

    def step(self, stream):
        self.wc.flash_attention_fwd(self.desc, self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(),
                                    self.o.data_ptr(), 0, stream)

    def prepare_host(self):
        t = self.torch
        self.host = tuple(x.cpu().pin_memory() for x in (self.q, self.k, self.v)) + (
            t.empty(self.q.shape, dtype=t.bfloat16).pin_memory(),)

    def step_host(self, stream):
        q, k, v, o = self.host
        self.wc.flash_attention_fwd_host(self.desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), stream)

    def check(self, oracle) -> float:
        BH = self.B * self.H
        heads = oracle.fa_sample_heads(BH)
        rows = oracle.fa_sample_rows(self.S)
        bits = lambda x: x[heads.tolist()].cpu().view(self.torch.int16).numpy().view(np.uint16)
        want = oracle.fa_ref(bits(self.q), bits(self.k), bits(self.v), oracle.BF16, 1.0 / np.sqrt(self.D),
                             causal=self.causal, rows=rows)
        got = self.o[heads.tolist()].float().cpu().numpy()[:, rows]
        return float(np.max(np.abs(got - want)) / 3.0e-2)


def time_steps(torch, work, steps, warmup, stream, dist=None, host=False):
    """W untimed warm-up steps, then exactly K steps between two CUDA events on
    the launching stream, bracketed by barrier + synchronize; returns the
    maximum over ranks of the elapsed milliseconds."""
    fn = work.step_host if host else work.step
    for _ in range(warmup):
        fn(stream.cuda_stream)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    work.t_begin = time.time()
    e0.record(stream)
    for _ in range(steps):
        fn(stream.cuda_stream)
    e1.record(stream)
    torch.cuda.synchronize()
    work.t_end = time.time()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def make_work(torch, wc, workload, rank, world):
    w = WORKLOADS[workload]
    if workload.startswith("fa"):
        return FaWork(torch, wc, w["B"], w["H"], w["S"], w["D"], rank, world, causal=w.get("causal", True),
                      qk_max_abs=w.get("qk_max_abs", 0.0))
    return GemmWork(torch, wc, w["M"], w["N"], w["K"], rank, world, streamk=0 if workload == "skinny" else 1)


# ----------------------------------------------------------------------------
# CPU baseline (checker code used as the reported baseline, never as the product)
# ----------------------------------------------------------------------------
def cpu_baseline(workload: str, budget_s: float = 12.0) -> dict:
    """Times the reference's CPU implementation of the path on a bounded sample
    of the workload with all host threads."""
    from oracle import oracle
    oracle.build()
    cores = host_threads()
    ref = oracle.ref_lib()
    w = WORKLOADS[workload]
    if workload in ("gemm", "skinny"):
        M, N, K = w["M"], w["N"], w["K"]
        rng = np.random.default_rng(0)
        a = oracle.to_bits(rng.standard_normal((M, K), dtype=np.float32) * np.float32(K ** -0.5), oracle.BF16)
        b = oracle.to_bits(rng.standard_normal((N, K), dtype=np.float32) * np.float32(K ** -0.5), oracle.BF16)
        run = (lambda rows: oracle.ref_gemm_rows(a, b, oracle.BF16, rows=rows, threads=cores)) if ref is not None \
            else (lambda rows: oracle.gemm_ref(a, b, oracle.BF16, rows=rows, threads=cores))
        # probe, then size the sample for the budget
        probe = np.arange(min(M, cores), dtype=np.int32)
        t0 = time.perf_counter()
        run(probe)
        per_row = (time.perf_counter() - t0) / probe.size
        nrows = int(max(probe.size, min(M, budget_s / max(per_row, 1e-9))))
        nrows = max(cores, nrows // cores * cores) if nrows >= cores else nrows
        nrows = min(nrows, M)
        rows = np.arange(nrows, dtype=np.int32)
        t0 = time.perf_counter()
        run(rows)
        dt = time.perf_counter() - t0
        flops = 2.0 * nrows * N * K
        sample = f"{nrows} of {M} output rows x all {N} columns, K={K}"
    else:
        B, H, S, D = w["B"], w["H"], w["S"], w["D"]
        causal = w.get("causal", True)
        heads = 2
        if causal:
            q = oracle.baseline_inputs((heads, S, D), "normal", 1, 0, oracle.BF16)
            k = oracle.baseline_inputs((heads, S, D), "normal", 1, 1, oracle.BF16)
            v = oracle.baseline_inputs((heads, S, D), "normal", 1, 2, oracle.BF16)
        else:  # the reference runner's own inputs
            q = oracle.fa_input_bits(heads * S * D, oracle.BF16, 1, 0, 0.125).reshape(heads, S, D)
            k = oracle.fa_input_bits(heads * S * D, oracle.BF16, 1, 1, 0.125).reshape(heads, S, D)
            v = oracle.fa_input_bits(heads * S * D, oracle.BF16, 1, 2, 0.25).reshape(heads, S, D)
        nrows = 64 * cores

        def run(rows):
            return oracle.fa_ref(q, k, v, oracle.BF16, 1.0 / np.sqrt(D), causal=causal, rows=rows, threads=cores)
        rows = np.linspace(0, S - 1, nrows).astype(np.int32)
        t0 = time.perf_counter()
        run(rows)
        dt = time.perf_counter() - t0
        scale = int(max(1, min(S // nrows, budget_s / max(dt, 1e-9))))
        if scale > 1:
            rows = np.linspace(0, S - 1, nrows * scale).astype(np.int32)
            t0 = time.perf_counter()
            run(rows)
            dt = time.perf_counter() - t0
        flops = float(sum(4.0 * D * ((r + 1) if causal else S) for r in rows.tolist()) * heads)
        ref = None  # the port: the compiled runner's row function has no causal mask and no thread pool
        sample = f"{rows.size} query rows x {heads} heads of S={S}, {'causal' if causal else 'non-causal'}, f64"
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": cores,
            "kind": "reference" if ref is not None else "port", "sample": sample, "seconds": dt}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t_all = time.perf_counter()
    # Each step is a bounded sample of the workload (about 8 s of CPU work), so the
    # counts are capped to keep the run within minutes; the line says what ran.
    warm = min(max(args.warmup, 0), 1)
    for _ in range(warm):
        cpu_baseline(args.workload, budget_s=2.0)
    results = []
    for _ in range(max(1, min(args.steps, 3))):
        results.append(cpu_baseline(args.workload, budget_s=8.0))
    best = max(results, key=lambda r: r["value"])
    w = WORKLOADS[args.workload]
    line = {
        "impl": "reference", "metric": METRIC, "value": best["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": len(results), "warmup": warm, "steps_requested": args.steps, "warmup_requested": args.warmup,
        "ms_per_step": best["seconds"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"], "sample": best["sample"]},
        "cpu_baseline": {k: best[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": best["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t_all,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", choices=["fa", "fa_published", "gemm", "skinny"], default="gemm")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--gather", action="store_true", help="also time the NCCL all-gather of the output shards")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--shape", default=None,
                    help="override the workload's size for profiling smaller cases: M,N,K (gemm, skinny) or B,H,S (fa)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    if args.shape:
        dims = [int(x) for x in args.shape.split(",")]
        w = WORKLOADS[args.workload]
        keys = ("B", "H", "S") if args.workload.startswith("fa") else ("M", "N", "K")
        w.update(dict(zip(keys, dims)))
        w["name"] += "_shape_override_" + "x".join(str(d) for d in dims)

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the backend has no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    wc = importlib.import_module("7_b200").wave_cuda
    wc.lib()
    pk, pk_kind = peaks()
    stream = torch.cuda.current_stream()

    work = make_work(torch, wc, args.workload, rank, world)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.5)  # let nvidia-smi come up so that samples fall inside the timed region
    ms = time_steps(torch, work, args.steps, args.warmup, stream, dist)
    clocks = sampler.stop(work.t_begin, work.t_end) if rank == 0 else None
    wc.check_device_status()
    ms_per_step = ms / args.steps
    value = work.flops * world / (ms_per_step * 1e-3) / 1e12

    gather = None
    if args.gather and world > 1:
        from importlib import import_module
        sh = import_module("7_b200.sharding")
        local = work.c if not args.workload.startswith("fa") else work.o
        for _ in range(3):
            sh.all_gather_shards(local, dist)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(10):
            sh.all_gather_shards(local, dist)
        e1.record(stream)
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 10], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gather = {"ms": float(t.item()), "bytes_per_rank": local.numel() * local.element_size()}

    # end-to-end: host buffers in, host buffers out, through the C-ABI host call
    work.prepare_host()
    e2e_ms = time_steps(torch, work, args.e2e_steps, 3, stream, dist, host=True) / args.e2e_steps
    wc.check_device_status()
    e2e_value = work.flops * world / (e2e_ms * 1e-3) / 1e12
    launches = (args.steps + args.warmup) * work.launches_per_step + (args.e2e_steps + 3) * work.launches_per_step

    parity = None
    also = {}
    cpu = None
    if rank == 0:
        from oracle import oracle
        oracle.build()
        work.step(stream.cuda_stream)
        torch.cuda.synchronize()
        parity = work.check(oracle)
    if not args.no_also and args.workload == "gemm":
        del work.host
        for other in ("fa", "fa_published", "skinny"):
            w2 = make_work(torch, wc, other, rank, world)
            steps2 = 10 if other.startswith("fa") else 50
            ms2 = time_steps(torch, w2, steps2, 3, stream, dist) / steps2
            wc.check_device_status()
            launches += (steps2 + 3) * w2.launches_per_step
            entry = {"workload": WORKLOADS[other]["name"], "ms_per_step": ms2,
                     "tflops": w2.flops * world / (ms2 * 1e-3) / 1e12}
            if other.startswith("fa"):
                entry["tflops_full_square_formula"] = w2.flops_full_square * world / (ms2 * 1e-3) / 1e12
                entry["frac_of_peak"] = entry["tflops"] / world / pk["bf16_tflops"]
                if "published_tflops" in WORKLOADS[other]:  # one GPU's rate against the reference's one-GPU number
                    entry["reference_published_tflops_gfx950"] = WORKLOADS[other]["published_tflops"]
                    entry["vs_published"] = entry["tflops"] / world / WORKLOADS[other]["published_tflops"]
            else:
                entry["gbs"] = w2.alg_bytes / (ms2 * 1e-3) / 1e9
                entry["frac_of_hbm_peak"] = entry["gbs"] / pk["hbm_gbs"]
            if rank == 0:
                from oracle import oracle
                w2.step(stream.cuda_stream)
                torch.cuda.synchronize()
                entry["parity_worst_over_tolerance"] = w2.check(oracle)
            also[other] = entry
            del w2
            torch.cuda.empty_cache()
    if rank == 0 and not args.no_cpu_baseline:
        cpu = cpu_baseline(args.workload)
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        # Under a long back-to-back loop the part runs into its power cap and
        # the SM clock drops; the matching denominator is then the sustained
        # cuBLAS figure, otherwise the burst one.
        capped = bool(clocks and clocks.get("sm_mhz") and "sw_power_cap" in clocks.get("reasons", [])
                      and clocks["sm_mhz"] < 0.85 * clocks["sm_max_mhz"])
        timed_alone = not capped
        if args.workload == "skinny":
            roof = {"bound": "hbm", "achieved": work.alg_bytes / (ms_per_step * 1e-3) / 1e9, "peak": pk["hbm_gbs"],
                    "unit": "GB/s"}
        else:
            peak = pk["bf16_tflops"] if timed_alone else pk["bf16_tflops_sustained"]
            roof = {"bound": "tensor", "achieved": work.flops / (ms_per_step * 1e-3) / 1e12, "peak": peak,
                    "unit": "TFLOP/s", "peak_kind": ("burst" if timed_alone else "sustained, power-capped clocks")
                    + f" ({pk_kind})", "frac_of_burst_peak": work.flops / (ms_per_step * 1e-3) / 1e12 / pk["bf16_tflops"],
                    "frac_of_nominal_2250": work.flops / (ms_per_step * 1e-3) / 1e12 / 2250.0}
        roof["frac"] = roof["achieved"] / roof["peak"]
        roof["traffic"] = NCU_TRAFFIC_BYTES.get(args.workload)
        roof["kernel_ms"] = ms_per_step
        w = WORKLOADS[args.workload]
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "per_gpu": {k: v for k, v in w.items() if k != "name"},
                       "sharding": ("N-column blocks, one 8192-column block per GPU" if not args.workload.startswith("fa")
                                    else "batch x head slabs, 512 heads per GPU") if world > 1 else "single GPU",
                       "l2": "inputs and output larger than L2 (no flush needed)",
                       "accumulate": "f32", "plan": wc.gemm_plan(work.desc) if not args.workload.startswith("fa") else
                       {"tile_m": 256, "tile_n": 128, "grid": [w["S"] // 256, w["B"] * w["H"]]}},
            "roofline": roof,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": work.h2d,
                    "d2h_bytes_per_step": work.d2h, "ms_per_step": e2e_ms},
            "cpu_baseline": cpu, "gpu_launches": launches, "clocks": clocks,
            "parity_worst_over_tolerance": parity, "also": also or None, "gather": gather,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def _keep_stdout_for_the_result() -> None:
    """stdout carries the one JSON line.  Libraries write there too (NCCL prints
    its version banner with printf when NCCL_DEBUG is set on the host), so file
    descriptor 1 is pointed at stderr for the run and `print` keeps the original."""
    sys.stdout.flush()
    result = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = result


if __name__ == "__main__":
    _keep_stdout_for_the_result()
    main()

#!/usr/bin/env python
"""Benchmark of the B200 backend for the Wave GEMM / flash-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemm|fa|fa_published|skinny]
                    [--impl ours|reference] [--scaling strong|weak] [--no-gather]

One "step" is one pass of the hot path over one batch of synthetic input.  The
headline workload (default) is the bf16 GEMM M=N=K=8192 with f32 accumulation
and bf16 output.  With N GPUs it stays ONE 8192^3 problem (strong scaling):
rank r computes the N-column block `column_shard(8192, N, r)` of C from the
replicated A and its rows of B, into the reference's column-major layout
(offset n*M + m, python/mlir/dialects/wave_matmul.py:1040) in which the block
is contiguous; `value` is the whole problem's FLOP over the slowest rank's
compute time.  The NCCL all-gather that gives every rank the whole C is timed
separately (`gather`), and rows of the GATHERED matrix are checked against the
CPU oracle, so that columns computed by every rank are compared.
`--workload fa` is the causal flash-attention forward B=16 H=32 S=4096 D=128,
its 512 (batch, head) slabs split over the ranks the same way; `--workload
skinny` the M=16, N=28672, K=8192 decode-shaped GEMM (single-GPU by
definition: N independent replicas).  `--scaling weak` gives every rank the
whole single-GPU problem instead.  The default run also measures the other
workloads briefly and reports them under "also".  Prints ONE JSON line on rank 0.

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
NVLINK_PEER_GBS = 770.0  # measured peer copy per direction on this pool (nominal 900)
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the single-GPU
# workload from one ncu capture of the same kernel (summaries under
# profiles/, each captured at the workload's full size).
NCU_TRAFFIC_BYTES = {"gemm": 1167.68e6, "fa": 2137.99e6, "skinny": 477.11e6, "fa_published": 1059.24e6}

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
    """Samples SM clocks and throttle reasons with nvidia-smi while timed
    regions run (reading only; no setting is changed).  One sampler runs for
    the whole benchmark; each timed region is summarised from the samples whose
    timestamps fall inside it."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap,power.draw")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

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

    def _rows(self):
        import datetime
        rows = []
        for line in list(self.lines):
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                power = float(parts[7]) if len(parts) > 7 else None
                rows.append((ts, float(parts[1]), float(parts[2]),
                             [n for n, v in zip(self.NAMES, parts[3:7]) if v.lower().startswith("active")], power))
            except ValueError:
                continue
        return rows

    def window(self, t_begin: float | None = None, t_end: float | None = None) -> dict:
        """Summary of the samples inside [t_begin, t_end] (host wall-clock
        seconds); of all samples if no window is given or none fell inside it."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        rows = self._rows()
        inside = [r for r in rows if t_begin is not None and t_begin <= r[0] <= t_end]
        use = inside or rows
        powers = [r[4] for r in use if r[4] is not None]
        return {"sm_mhz": statistics.median([r[1] for r in use]) if use else None,
                "sm_max_mhz": max([r[2] for r in use]) if use else None,
                "reasons": sorted({n for r in use for n in r[3]}), "samples": len(use),
                "window": "timed region" if inside else "whole run",
                "power_w_max": max(powers) if powers else None}

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()


# ----------------------------------------------------------------------------
# workloads on the GPU
# ----------------------------------------------------------------------------
class GemmWork:
    """C = A * B^T, bf16 in, f32 accumulate, bf16 out.  strong: one M x N x K
    problem, this rank owns the columns column_shard(N, world, rank); weak: the
    whole problem on every rank (its own B).  C is column-major (this rank's
    block [n_local][M] is contiguous and gathers in place)."""

    kind = "gemm"

    def __init__(self, torch, wc, sh, M, N, K, rank, world, strong, seed=0, streamk=0):
        self.torch, self.wc, self.sh = torch, wc, sh
        self.M, self.N, self.K, self.rank, self.world, self.strong = M, N, K, rank, world, strong
        g = torch.Generator(device="cuda")
        g.manual_seed(1234 + seed)
        # A is replicated across ranks (same seed).
        self.a = (torch.randn(M, K, device="cuda", generator=g) * (K ** -0.5 if M > 16 else 1.0)).to(torch.bfloat16)
        g.manual_seed(4321 + seed + (0 if strong else 977 * rank))
        b_full = (torch.randn(N, K, device="cuda", generator=g) * K ** -0.5).to(torch.bfloat16)
        self.skinny = M % 256 != 0
        if strong and world > 1:
            self.n0, self.n1 = sh.column_shard(N, world, rank, 256)
        else:
            self.n0, self.n1 = 0, N
        self.b_full = b_full if (strong and rank == 0) else None  # rank 0 checks the gathered C against all of B
        self.b = b_full[self.n0:self.n1].contiguous() if strong and world > 1 else b_full
        self.nl = self.n1 - self.n0
        knobs = dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4) if not self.skinny else dict(bn=1)
        layout = wc.ROW_MAJOR if self.skinny else wc.COL_MAJOR
        self.col_major = layout == wc.COL_MAJOR
        self.c = torch.empty((self.nl, M) if self.col_major else (M, self.nl), device="cuda", dtype=torch.bfloat16)
        self.desc = wc.gemm_desc(M, self.nl, K, in_type=wc.BF16, out_type=wc.BF16, out_layout=layout,
                                 streamk_workers=streamk, **knobs)
        s, c = wc.gemm_workspace_bytes(self.desc)
        self.ws = torch.zeros(s + c, dtype=torch.uint8, device="cuda") if s + c else None
        total_n = N if strong else N * world
        self.flops = 2.0 * M * total_n * K                 # whole job, all ranks
        self.flops_rank = 2.0 * M * self.nl * K
        self.alg_bytes = 2.0 * (M * K + self.nl * K + M * self.nl)  # this rank's launch
        self.launches_per_step = 1
        self.host = None

    def step(self, stream):
        self.wc.gemm(self.desc, self.a.data_ptr(), self.b.data_ptr(), self.c.data_ptr(),
                     self.ws.data_ptr() if self.ws is not None else 0, stream)

    # ---- end to end: every operand starts and ends in pinned host memory
    def prepare_host(self):
        t = self.torch
        self.host = (self.a.cpu().pin_memory(), self.b.cpu().pin_memory(), t.empty_like(self.c, device="cpu").pin_memory())
        sharded = self.strong and self.world > 1
        self.a_stage = t.empty_like(self.a) if sharded else None
        a_rows = self.M // self.world if sharded else self.M
        self.h2d = 2 * (a_rows * self.K + self.nl * self.K)
        self.d2h = 2 * self.M * self.nl

    def step_host(self, stream, dist=None):
        a, b, c = self.host
        if self.a_stage is not None:
            self.sh.sharded_gemm_host(self.wc, self.desc, self.a_stage, a, b, c, dist, self.rank, self.world, stream)
        else:
            self.wc.gemm_host(self.desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream)

    def host_result(self):
        return self.host[2]

    # ---- the all-gather that gives every rank the whole output
    def local_output(self):
        return self.c

    def check(self, oracle, gathered=None) -> dict:
        """Sampled parity outside the timed region: 8 rows of C (all columns, so
        every rank's block of a gathered C is compared) against the CPU oracle
        (f32 accumulate, k ascending)."""
        t = self.torch
        rows = np.unique(np.linspace(0, self.M - 1, 8).astype(np.int32))
        a = self.a.cpu().view(t.int16).numpy().view(np.uint16)
        if gathered is not None:
            b_src, c_src, what = self.b_full, gathered.reshape(self.N, self.M), f"gathered C, columns of all {self.world} ranks"
        else:
            b_src, c_src, what = self.b, self.c, "this rank's C"
        b = b_src.cpu().view(t.int16).numpy().view(np.uint16)
        want = oracle.round_output(oracle.gemm_ref(a, b, oracle.BF16, rows=rows), "bf16")
        got = (c_src[:, rows.tolist()].float().cpu().numpy().T if self.col_major
               else c_src[rows.tolist()].float().cpu().numpy())
        worst = float(np.max(np.abs(got - want) / (1.0e-2 + 2.0 ** -7 * np.abs(want))))
        return {"worst_over_tolerance": worst, "checked": what, "rows": int(rows.size), "columns": int(want.shape[1]),
                "tolerance": "|d| <= 1e-2 + 2^-7*|exp| (bf16 output: one ulp in place of the runner's 1e-3 term)"}

    def check_host(self, oracle) -> float:
        """Elements of the end-to-end call's host result that are more than one
        bf16 unit in the last place away from the device-resident run's (the
        host call computes C by column blocks, which may group the f32 sums
        differently: one rounding step of the bf16 result, plus the runner's
        absolute 1e-3 for sums that cancel towards zero; anything beyond would
        be an error)."""
        got, ref = self.host_result().float(), self.c.cpu().float()
        return float(((got - ref).abs() > 2.0 ** -7 * ref.abs() + 1e-3).sum().item())


class FaWork:
    """Flash-attention forward; strong: B*H slabs split by head_shard."""

    kind = "fa"

    def __init__(self, torch, wc, sh, B, H, S, D, rank, world, strong, seed=0, causal=True, qk_max_abs=0.0):
        self.torch, self.wc, self.sh = torch, wc, sh
        self.B, self.H, self.S, self.D, self.causal = B, H, S, D, causal
        self.rank, self.world, self.strong = rank, world, strong
        BH = B * H
        g = torch.Generator(device="cuda")
        g.manual_seed(99 + seed + (0 if strong else 131 * rank))
        if qk_max_abs > 0.0:
            # the value set of the reference runner's generator (17 buckets, Q/K x0.125, V x0.25;
            # wave-fa-gfx950-runner.cpp:188-202), drawn from torch's generator
            mk = lambda scale: (torch.randint(-8, 9, (BH, S, D), device="cuda", generator=g).float()
                                * scale).to(torch.bfloat16)
            q, k, v = mk(0.125), mk(0.125), mk(0.25)
        else:
            mk = lambda: torch.randn(BH, S, D, device="cuda", generator=g).to(torch.bfloat16)
            q, k, v = mk(), mk(), mk()
        if strong and world > 1:
            self.h0, self.h1 = sh.head_shard(BH, world, rank)
            self.full = (q, k, v) if rank == 0 else None  # rank 0 checks heads of every rank's slab
            q, k, v = (x[self.h0:self.h1] for x in (q, k, v))
        else:
            self.h0, self.h1 = 0, BH
            self.full = None
        self.q, self.k, self.v = q, k, v
        self.hl = self.h1 - self.h0
        self.o = torch.empty_like(self.q)
        self.desc = wc.fa_desc(1, self.hl, S, S, D, causal=causal, io_type=wc.BF16, qk_max_abs=qk_max_abs)
        # unmasked pairs only for the causal case; the reference's own formula
        # (4*B*H*S^2*D, wave-fa-gfx950-runner.cpp:465-466) counts the full square
        pairs = S * (S + 1) / 2 if causal else float(S) * S
        total_bh = BH if strong else BH * world
        self.flops = 4.0 * total_bh * D * pairs
        self.flops_rank = 4.0 * self.hl * D * pairs
        self.flops_full_square = 4.0 * total_bh * D * float(S) * S
        self.alg_bytes = 4.0 * self.hl * S * D * 2
        self.launches_per_step = 1
        self.host = None

    def step(self, stream):
        self.wc.flash_attention_fwd(self.desc, self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(),
                                    self.o.data_ptr(), 0, stream)

    def prepare_host(self):
        t = self.torch
        self.host = tuple(x.cpu().pin_memory() for x in (self.q, self.k, self.v)) + (
            t.empty(self.q.shape, dtype=t.bfloat16).pin_memory(),)
        self.h2d = 3 * self.hl * self.S * self.D * 2
        self.d2h = self.hl * self.S * self.D * 2

    def step_host(self, stream, dist=None):
        q, k, v, o = self.host
        self.wc.flash_attention_fwd_host(self.desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), stream)

    def host_result(self):
        return self.host[3]

    def local_output(self):
        return self.o

    def check(self, oracle, gathered=None) -> dict:
        if gathered is not None:
            q, k, v = self.full
            o, what = gathered.reshape(q.shape), f"gathered O, heads of the first, middle and last rank of {self.world}"
        else:
            q, k, v, o, what = self.q, self.k, self.v, self.o, "this rank's O"
        heads = oracle.fa_sample_heads(q.shape[0])
        rows = oracle.fa_sample_rows(self.S)
        bits = lambda x: x[heads.tolist()].cpu().view(self.torch.int16).numpy().view(np.uint16)
        want = oracle.fa_ref(bits(q), bits(k), bits(v), oracle.BF16, 1.0 / np.sqrt(self.D), causal=self.causal, rows=rows)
        got = o[heads.tolist()].float().cpu().numpy()[:, rows]
        return {"worst_over_tolerance": float(np.max(np.abs(got - want)) / 3.0e-2), "checked": what,
                "heads": [int(h) for h in heads], "rows": int(rows.size),
                "tolerance": "max abs <= 3e-2 (wave-fa-gfx950-runner.cpp:388) on the runner's head/row sample"}

    def check_host(self, oracle) -> float:
        return float((self.host_result().view(self.torch.int16) != self.o.cpu().view(self.torch.int16)).sum().item())


def time_steps(torch, work, steps, warmup, stream, dist=None, host=False):
    """W untimed warm-up steps, then exactly K steps between two CUDA events on
    the launching stream, bracketed by barrier + synchronize; returns the
    maximum over ranks of the elapsed milliseconds."""
    fn = (lambda s: work.step_host(s, dist)) if host else work.step
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


def make_work(torch, wc, sh, workload, rank, world, strong):
    w = WORKLOADS[workload]
    if workload.startswith("fa"):
        return FaWork(torch, wc, sh, w["B"], w["H"], w["S"], w["D"], rank, world, strong, causal=w.get("causal", True),
                      qk_max_abs=w.get("qk_max_abs", 0.0))
    # the skinny GEMM is a single-GPU configuration: N independent replicas
    return GemmWork(torch, wc, sh, w["M"], w["N"], w["K"], rank, world, strong and workload != "skinny")


def time_gather(torch, sh, work, dist, stream, world) -> tuple[dict, object]:
    """The NCCL all-gather of the ranks' output blocks (column-major C blocks /
    O slabs, contiguous and equally sized), timed by itself, max over ranks."""
    local = work.local_output()
    full = None
    for _ in range(3):
        full = sh.all_gather_shards(local, dist)
    torch.cuda.synchronize()
    dist.barrier()
    iters = 10
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
        full = sh.all_gather_shards(local, dist)
    e1.record(stream)
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    nbytes = local.numel() * local.element_size()
    recv_gbs = (world - 1) * nbytes / (ms * 1e-3) / 1e9
    return {"collective": "ncclAllGather over NVLink (torch.distributed all_gather_into_tensor)", "ms": ms,
            "bytes_per_rank": nbytes, "received_gbs_per_rank": recv_gbs,
            "frac_of_nvlink_peer_copy": recv_gbs / NVLINK_PEER_GBS, "nvlink_peer_copy_gbs": NVLINK_PEER_GBS}, full


def time_fused_gather(torch, wc, sh, work, dist, stream, rank, world, oracle) -> dict:
    """The all-gather fused into the kernel: every rank writes its block (GEMM:
    N-column block of C; attention: (batch, head) slab of O) straight into every
    rank's copy of the full output -- peer-mapped memory, TMA / bulk stores out of
    the epilogue while the kernel computes on, or one multimem.st per 16 bytes to
    an NVLink multicast address -- followed by a one-element all-reduce as the
    barrier after which the copies may be read.  Timed as one step, max over
    ranks; rank 0's copy is then checked against the oracle on a sample that
    spans every rank's part."""
    gemm = work.kind == "gemm"
    shape = (work.N, work.M) if gemm else (work.B * work.H, work.S, work.D)
    try:
        out = sh.PeerMappedOutput(shape, torch.bfloat16, dist, rank, world)
    except Exception as err:  # no symmetric memory on this system: say so, the NCCL gather stands
        return {"unavailable": f"{type(err).__name__}: {err}"[:300]}
    if gemm:
        offset = work.n0 * work.M * 2
        block_bytes = work.nl * work.M * 2
        desc = wc.gemm_desc(work.M, work.nl, work.K, in_type=wc.BF16, out_type=wc.BF16, out_layout=wc.COL_MAJOR,
                            streamk_workers=1, bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)
    else:
        offset = work.h0 * work.S * work.D * 2
        block_bytes = work.hl * work.S * work.D * 2
        desc = work.desc
    targets = out.block_targets(offset)
    iters = 20 if gemm else 10

    def timed(step):
        out.local.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            step()
        e1.record(stream)
        torch.cuda.synchronize()
        wc.check_device_status()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        entry = {"ms_per_step": ms, "tflops": work.flops / (ms * 1e-3) / 1e12}
        if rank == 0:
            entry["parity"] = work.check(oracle, out.local)
        dist.barrier()
        return entry

    def unicast():
        if gemm:
            wc.gemm_multi_output(desc, work.a.data_ptr(), work.b.data_ptr(), targets, stream.cuda_stream)
        else:
            wc.flash_attention_fwd_multi_output(desc, work.q.data_ptr(), work.k.data_ptr(), work.v.data_ptr(), targets,
                                                0, stream.cuda_stream)
        out.settle()

    def multicast():
        if gemm:
            wc.gemm_multicast_output(desc, work.a.data_ptr(), work.b.data_ptr(), out.ptrs[rank] + offset,
                                     out.multicast_ptr + offset, stream.cuda_stream)
        else:
            wc.flash_attention_fwd_multicast_output(desc, work.q.data_ptr(), work.k.data_ptr(), work.v.data_ptr(),
                                                    out.ptrs[rank] + offset, out.multicast_ptr + offset, 0,
                                                    stream.cuda_stream)
        out.settle()
    res = timed(unicast)
    entry = "wave_cuda_gemm_multi_output" if gemm else "wave_cuda_flash_attention_fwd_multi_output"
    res.update({"kernel": f"{entry}: this rank's block written to every rank's copy of the output from the kernel's "
                          "epilogue over NVLink (peer-mapped memory, TMA / bulk stores from shared memory), then a one-element all-reduce as barrier",
                "launches": 2 * (iters + 3), "bytes_sent_per_rank": (world - 1) * block_bytes,
                "sent_gbs_per_rank": (world - 1) * block_bytes / (res["ms_per_step"] * 1e-3) / 1e9})
    if out.multicast_ptr:
        res["multicast"] = timed(multicast)
        res["multicast"]["kernel"] = (entry.replace("multi_output", "multicast_output") + ": every 16 bytes stored once "
                                      "to an NVLink multicast address (multimem.st), replicated to all ranks in the switch")
        res["multicast"]["bytes_sent_per_rank"] = block_bytes
    else:
        res["multicast"] = {"unavailable": "the symmetric-memory handle has no multicast address (no NVLS for this group)"}
    del out
    return res


def optional_leg(fn, *args, **kwargs) -> dict:
    """Runs one of the legs that explain the headline number (fused gather,
    sustained loop, cuBLAS comparison).  If it raises, the JSON line still
    comes out, with the error in the leg's place."""
    try:
        return fn(*args, **kwargs)
    except Exception as err:  # noqa: BLE001 - whatever it is, it must not cost the headline line
        return {"error": f"{type(err).__name__}: {err}"[:300]}


def sustained_leg(torch, work, stream, sampler, seconds, pk) -> dict:
    """Back-to-back launches for about `seconds` (the power-capped regime a
    short burst never reaches), with the SM clock sampled meanwhile."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        work.step(stream.cuda_stream)
    torch.cuda.synchronize()
    probe = 10
    e0.record(stream)
    for _ in range(probe):
        work.step(stream.cuda_stream)
    e1.record(stream)
    torch.cuda.synchronize()
    per = max(e0.elapsed_time(e1) / probe, 1e-3)
    n = int(min(max(seconds * 1e3 / per, 20), 20000))
    t0 = time.time()
    e0.record(stream)
    for _ in range(n):
        work.step(stream.cuda_stream)
    e1.record(stream)
    torch.cuda.synchronize()
    t1 = time.time()
    ms = e0.elapsed_time(e1) / n
    clk = sampler.window(t0 + 0.3 * (t1 - t0), t1) if sampler is not None else {}
    tflops = work.flops_rank / (ms * 1e-3) / 1e12
    out = {"launches": n, "seconds": (t1 - t0), "ms_per_launch": ms, "tflops": tflops,
           "frac_of_sustained_peak": tflops / pk["bf16_tflops_sustained"], "sm_mhz_median": clk.get("sm_mhz"),
           "reasons": clk.get("reasons"), "power_w_max": clk.get("power_w_max")}
    if clk.get("sm_mhz"):
        out["ms_x_mhz"] = ms * clk["sm_mhz"]  # clock-independent cost: milliseconds at 1 MHz
    return out


def cublas_comparison(torch, work, stream, seconds=2.5) -> dict:
    """This library's GEMM against torch.matmul (cuBLAS) on the same operands,
    interleaved in one loop so that both run under the same power cap and
    clocks: blocks of launches take turns, each block timed with CUDA events."""
    a, b = work.a, work.b
    out = torch.empty(a.shape[0], b.shape[0], device="cuda", dtype=torch.bfloat16)
    bt = b.t()
    ours = lambda: work.step(stream.cuda_stream)
    theirs = lambda: torch.matmul(a, bt, out=out)
    for _ in range(3):
        ours()
        theirs()
    torch.cuda.synchronize()

    def block(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        return e0, e1, n
    # burst: a short block each after an idle moment
    burst = {}
    for name, fn in (("ours", ours), ("cublas", theirs)):
        time.sleep(0.5)
        e0, e1, n = block(fn, 10)
        torch.cuda.synchronize()
        burst[name] = work.flops_rank / (e0.elapsed_time(e1) / n * 1e-3) / 1e12
    # sustained: alternate blocks of 40 launches until the time is up; the first third is warm-up
    blocks = []
    t_end = time.time() + seconds
    while time.time() < t_end:
        blocks.append(("ours",) + block(ours, 40))
        blocks.append(("cublas",) + block(theirs, 40))
        torch.cuda.synchronize()
    keep = blocks[len(blocks) // 3:]
    rate = {}
    for name in ("ours", "cublas"):
        ms = [e0.elapsed_time(e1) / n for nm, e0, e1, n in keep if nm == name]
        rate[name] = work.flops_rank / (statistics.median(ms) * 1e-3) / 1e12
    return {"ours_tflops_sustained": rate["ours"], "cublas_tflops_sustained": rate["cublas"],
            "ratio_sustained": rate["ours"] / rate["cublas"], "ours_tflops_burst": burst["ours"],
            "cublas_tflops_burst": burst["cublas"], "ratio_burst": burst["ours"] / burst["cublas"],
            "how": "torch.matmul(A, B^T) on the same bf16 operands; blocks of 40 launches taking turns for "
                   f"{seconds} s (median of the last two thirds), and 10-launch bursts after 0.5 s idle",
            "launches": 20 + 40 * len(blocks) // 2}


def roofline_for(workload, work, ms_per_step, clocks, pk, pk_kind) -> dict:
    """Roofline of this rank's launch: algorithmic FLOP (or bytes) over the
    measured launch duration against the measured peak."""
    if workload == "skinny":
        roof = {"bound": "hbm", "achieved": work.alg_bytes / (ms_per_step * 1e-3) / 1e9, "peak": pk["hbm_gbs"],
                "unit": "GB/s", "peak_kind": f"copy bandwidth ({pk_kind})"}
    else:
        # Under a long back-to-back loop the part runs into its power cap and the
        # SM clock drops; the matching denominator is then the sustained cuBLAS
        # figure, otherwise the burst one.
        capped = bool(clocks and clocks.get("sm_mhz") and "sw_power_cap" in (clocks.get("reasons") or [])
                      and clocks["sm_mhz"] < 0.85 * clocks["sm_max_mhz"])
        achieved = work.flops_rank / (ms_per_step * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved,
                "peak": pk["bf16_tflops_sustained"] if capped else pk["bf16_tflops"], "unit": "TFLOP/s",
                "peak_kind": ("sustained, power-capped clocks" if capped else "burst") + f" ({pk_kind})",
                "frac_of_burst_peak": achieved / pk["bf16_tflops"], "frac_of_nominal_2250": achieved / 2250.0}
    roof["frac"] = roof["achieved"] / roof["peak"]
    single_gpu_problem = work.world == 1 or not work.strong
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(workload) if single_gpu_problem else None
    roof["algorithmic_bytes"] = work.alg_bytes
    roof["kernel_ms"] = ms_per_step
    return roof


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
        "scaling": "strong" if args.scaling == "strong" and args.workload != "skinny" else "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"], "sample": best["sample"]},
        "cpu_baseline": {k: best[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": best["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t_all,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
def measure_workload(torch, wc, sh, workload, rank, world, strong, steps, warmup, e2e_steps, stream, dist, sampler,
                     pk, pk_kind, want_gather, want_cpu, want_sustained, counters) -> dict:
    """Everything reported for one workload: device-timed rate, roofline, the
    separately timed all-gather with parity of the gathered output, the
    end-to-end rate through the host-buffer calls, the CPU baseline and the
    sustained leg."""
    from oracle import oracle
    work = make_work(torch, wc, sh, workload, rank, world, strong)
    sharded = work.strong and world > 1
    # Every workload starts its timed loop from an idle GPU, like the first one: the legs that ran
    # before it (sustained loops, the cuBLAS comparison) leave the part at a power-capped clock.
    torch.cuda.synchronize()
    time.sleep(1.5)
    ms = time_steps(torch, work, steps, warmup, stream, dist) / steps
    clocks = sampler.window(work.t_begin, work.t_end) if sampler is not None else None
    wc.check_device_status()
    counters["launches"] += (steps + warmup) * work.launches_per_step
    res = {"workload": WORKLOADS[workload]["name"], "ms_per_step": ms, "tflops": work.flops / (ms * 1e-3) / 1e12,
           "scaling": "strong" if work.strong else "weak"}
    if workload.startswith("fa"):
        res["tflops_full_square_formula"] = work.flops_full_square / (ms * 1e-3) / 1e12
        if "published_tflops" in WORKLOADS[workload]:  # one GPU's rate against the reference's one-GPU number
            res["reference_published_tflops_gfx950"] = WORKLOADS[workload]["published_tflops"]
            res["vs_published_per_gpu"] = work.flops_rank / (ms * 1e-3) / 1e12 / WORKLOADS[workload]["published_tflops"]
    if workload == "skinny":
        res["gbs_per_gpu"] = work.alg_bytes / (ms * 1e-3) / 1e9
    if rank == 0:
        res["roofline"] = roofline_for(workload, work, ms, clocks, pk, pk_kind)
        res["clocks"] = clocks

    # parity of the device-resident result (this rank), then of the gathered output (all ranks)
    work.step(stream.cuda_stream)
    torch.cuda.synchronize()
    counters["launches"] += 1
    gathered = None
    if sharded and want_gather:
        res["gather"], gathered = time_gather(torch, sh, work, dist, stream, world)
        res["ms_per_step_with_gather"] = ms + res["gather"]["ms"]
        res["tflops_with_gather"] = work.flops / ((ms + res["gather"]["ms"]) * 1e-3) / 1e12
    else:
        res["gather"] = None
    if rank == 0:
        oracle.build()
        res["parity"] = work.check(oracle, gathered)
    del gathered
    if sharded and want_gather:
        res["fused_gather"] = optional_leg(time_fused_gather, torch, wc, sh, work, dist, stream, rank, world, oracle)
        counters["launches"] += res["fused_gather"].get("launches", 0)
        if "ms_per_step" in res["fused_gather"]:  # compute + NCCL gather against the fused kernels
            fg = res["fused_gather"]
            fg["speedup_over_compute_plus_nccl_gather"] = res["ms_per_step_with_gather"] / fg["ms_per_step"]
            if "ms_per_step" in fg.get("multicast", {}):
                fg["multicast"]["speedup_over_compute_plus_nccl_gather"] = \
                    res["ms_per_step_with_gather"] / fg["multicast"]["ms_per_step"]

    # end to end: host buffers in, host buffers out
    work.prepare_host()
    e2e_ms = time_steps(torch, work, e2e_steps, 3, stream, dist, host=True) / e2e_steps
    wc.check_device_status()
    counters["launches"] += (e2e_steps + 3) * work.launches_per_step
    mismatched = work.check_host(oracle)
    res["e2e"] = {"value": work.flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": work.h2d,
                  "d2h_bytes_per_step": work.d2h, "ms_per_step": e2e_ms,
                  "h2d_gbs_per_rank": work.h2d / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": work.d2h / (e2e_ms * 1e-3) / 1e9,
                  "host_link_gbs_all_ranks": (work.h2d + work.d2h) * world / (e2e_ms * 1e-3) / 1e9,
                  "elements_beyond_one_ulp_of_device_run": mismatched,
                  "path": ("each rank copies M/N rows of A and its B block from pinned host memory, the ranks "
                           "all-gather A over NVLink, wave_cuda_gemm_host_a_resident computes and returns the C block"
                           if sharded and work.kind == "gemm" else
                           "wave_cuda_gemm_host" if work.kind == "gemm" else "wave_cuda_flash_attention_fwd_host")
                          + "; copies inside the timed region"}
    work.host = None

    if want_sustained:
        res["sustained"] = optional_leg(sustained_leg, torch, work, stream, sampler if rank == 0 else None, want_sustained, pk)
        counters["launches"] += res["sustained"].get("launches", 0) + 13
    if workload == "gemm" and want_sustained and not work.skinny:
        res["vs_cublas"] = optional_leg(cublas_comparison, torch, work, stream)
        counters["launches"] += res["vs_cublas"].get("launches", 0)
    if want_cpu and rank == 0:
        cpu = cpu_baseline(workload)
        res["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    res["plan"] = wc.gemm_plan(work.desc) if work.kind == "gemm" else {
        "work_item_rows": 256, "keys_per_block": 80, "heads_per_gpu": work.hl}
    del work
    torch.cuda.empty_cache()
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", choices=["fa", "fa_published", "gemm", "skinny"], default="gemm")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong",
                    help="strong: one fixed problem split over the GPUs (default); weak: the whole problem on every GPU")
    ap.add_argument("--no-gather", action="store_true", help="skip the NCCL all-gather of the output shards")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true")
    ap.add_argument("--no-sustained", action="store_true")
    ap.add_argument("--sustained-seconds", type=float, default=2.0)
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
        NCU_TRAFFIC_BYTES[args.workload] = None

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
    pkg = importlib.import_module("7_b200")
    wc, sh = pkg.wave_cuda, importlib.import_module("7_b200.sharding")
    wc.lib()
    pk, pk_kind = peaks()
    stream = torch.cuda.current_stream()
    strong = args.scaling == "strong"

    sampler = None
    if rank == 0:
        sampler = ClockSampler(local_rank)
        sampler.start()
        time.sleep(0.5)  # let nvidia-smi come up so that samples fall inside the timed region
    counters = {"launches": 0}
    sustained = 0.0 if args.no_sustained else args.sustained_seconds
    main_res = measure_workload(torch, wc, sh, args.workload, rank, world, strong, args.steps, args.warmup,
                                args.e2e_steps, stream, dist, sampler, pk, pk_kind, not args.no_gather,
                                not args.no_cpu_baseline, sustained, counters)
    also = {}
    if not args.no_also and args.workload == "gemm":
        for other in ("fa", "fa_published", "skinny"):
            steps2 = 10 if other.startswith("fa") else 50
            also[other] = measure_workload(torch, wc, sh, other, rank, world, strong, steps2, 3,
                                           3 if other != "skinny" else 5, stream, dist, sampler, pk, pk_kind,
                                           not args.no_gather, (not args.no_cpu_baseline) and other == "fa",
                                           sustained if other == "fa" else 0.0, counters)
    if sampler is not None:
        sampler.stop()

    if rank == 0:
        w = WORKLOADS[args.workload]
        is_strong = main_res["scaling"] == "strong"
        per = {k: v for k, v in w.items() if k != "name"}
        line = {
            "metric": METRIC, "value": main_res["tflops"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": main_res["ms_per_step"], "higher_is_better": True,
            "scaling": main_res["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "problem": per,
                       "sharding": ("single GPU" if world == 1 else
                                    ("one problem: " if is_strong else "one problem per GPU: ") +
                                    ("N-column blocks of B and C (A replicated), column-major C blocks"
                                     if not args.workload.startswith("fa") else "contiguous (batch x head) slabs of Q, K, V, O")),
                       "l2": "inputs and output larger than L2 (no flush needed)" if world == 1 or not is_strong else
                             "replicated operand larger than L2 (no flush needed)",
                       "accumulate": "f32", "plan": main_res.pop("plan")},
            "roofline": main_res.get("roofline"), "e2e": main_res["e2e"], "cpu_baseline": main_res.get("cpu_baseline"),
            "gpu_launches": counters["launches"], "clocks": main_res.get("clocks"),
            "parity_worst_over_tolerance": main_res["parity"]["worst_over_tolerance"], "parity": main_res["parity"],
            "gather": main_res.get("gather"), "value_with_gather": main_res.get("tflops_with_gather"),
            "fused_gather": main_res.get("fused_gather"),
            "sustained": main_res.get("sustained"), "vs_cublas": main_res.get("vs_cublas"), "also": also or None,
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

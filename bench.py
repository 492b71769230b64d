"""Benchmark of the ternary expert-GEMM path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One "step" is one MoE routed-expert layer pass over one batch of synthetic tokens (BASELINE config 4:
16384 tokens per step over all ranks, hidden 4096, 384 experts each a SwiGLU FFN 4096->2048->4096 in
TQ1 with one fp16 scale per 128 K-elements, top-6 softmax routing from seeded N(0,1) logits, bf16
activations). With N > 1 (launched by torch.distributed.run, one rank per GPU) the experts are sharded
evenly over the ranks and the tokens split evenly, with NCCL all-to-all dispatch and combine: the
total work is fixed, so scaling is "strong". Rank 0 prints ONE JSON line.

Keys beyond the base contract:
  roofline      the dominant kernel (the grouped expert GEMM): algorithmic FLOPs per launch / mean
                launch time measured with CUDA events on the launching stream, against the measured
                dense bf16 peak in MEASURED_PEAKS.json (fallback 1590 TFLOP/s).
  cpu_baseline  the reference's C++ CPU ternary kernel (oracle/_ref, "reference") or the C oracle
                ("port") timed on this host's cores on a bounded sample of the same workload.
  e2e           tokens/s through the public API with host buffers: the H2D copy of the step's
                tokens and logits from pinned memory and the D2H read of the layer output are inside
                the timed region.
  gemm          (N = 1 only) decode GEMV packed-HBM GB/s and prefill grouped-GEMM TFLOP/s at the
                BASELINE config 0/1/2 shapes, each with its roofline fraction.

--impl reference times the reference's own CPU kernel for the same layer on a bounded sample per
step (a few experts with exactly the rows routed to them) and extrapolates by rows.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, INTER, N_EXPERTS, TOP_K, GROUP, FMT = 4096, 2048, 384, 6, 128, "tq1"
TOKENS = 16384
SEED = 20261125


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------------- synthetic data
def synth_expert_weights(n_local: int, expert0: int, device, fmt=None, hidden=HIDDEN, inter=INTER):
    """Seeded random-init experts generated on the device (deepseekternarized_b200/synth.py): trits i.i.d. P(0)=0.4,
    P(+-1)=0.3, scales lognormal(-4, 0.3) in fp16. Expert e's weights depend only on (SEED, e), so every sharding
    sees the same global model."""
    from deepseekternarized_b200.synth import synth_expert_weights as synth

    return synth(n_local, expert0, device, FMT if fmt is None else fmt, hidden, inter, SEED)


def synth_tokens(n_tokens: int, token0: int, n_experts=None, hidden=HIDDEN):
    """Host-side seeded tokens (bf16 ~N(0,1)) and router logits (f32 ~N(0,1)) in pinned memory."""
    n_experts = N_EXPERTS if n_experts is None else n_experts
    g = torch.Generator().manual_seed(SEED + 7 + token0)
    x = torch.randn(n_tokens, hidden, generator=g).bfloat16()
    logits = torch.randn(n_tokens, n_experts, generator=g)
    if torch.cuda.is_available():
        x, logits = x.pin_memory(), logits.pin_memory()
    return x, logits


# --------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []  # lines: (host time when read, text)
        self.t0 = self.t1 = self.t_load = None

    def mark_load(self):
        self.t_load = time.time()

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [ln for ts, ln in self.lines if self.t0 is None or (self.t0 <= ts <= (self.t1 or ts) + 0.05)]
        window = "timed region"
        if len(inside) < 3 and self.t_load is not None:
            # a timed region of a few sampling periods at most: add the samples of the identical steps run right before it
            inside = [ln for ts, ln in self.lines if self.t_load <= ts <= (self.t1 or ts) + 0.05]
            window = "timed region and the identical untimed steps directly before it"
        for ln in inside:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "window": window, "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------- CPU baseline
def cpu_layer_sample(n_sample_experts: int, rows_per_expert: int, threads: int):
    """Times the CPU ternary kernel on `n_sample_experts` experts with `rows_per_expert` routed rows each
    (gate+up 4096->4096 stacked, then down 2048->4096): the same three linears per expert the layer runs.
    Returns (seconds, rows, kind)."""
    from oracle import oracle as O

    ref = O.reference_module()
    torch.set_num_threads(threads)
    rng = np.random.default_rng(SEED)
    secs = 0.0
    lut = torch.from_numpy(O.tq1_lut())
    code = 1 if FMT == "tq1" else 2
    for _ in range(n_sample_experts):
        x = O.synth_acts(rng, (rows_per_expert, HIDDEN))
        h = O.synth_acts(rng, (rows_per_expert, INTER))
        for xin, (Nw, Kw) in ((x, (2 * INTER, HIDDEN)), (h, (HIDDEN, INTER))):
            p = rng.integers(0, 243, (Nw, -(-Kw // 5)), dtype=np.uint8) if FMT == "tq1" else rng.integers(0, 256, (Nw, Kw // 4), dtype=np.uint8)
            s = O.synth_scales(rng, (Nw, Kw // GROUP)).astype(np.float32)
            if ref is not None:
                out = torch.zeros(rows_per_expert, Nw)
                args = (out, torch.from_numpy(xin), torch.ones(rows_per_expert), torch.from_numpy(p), torch.from_numpy(s), Kw, GROUP, code, lut)
                t0 = time.perf_counter()
                ref.ternary_gemm(*args)
                secs += time.perf_counter() - t0
            else:
                t0 = time.perf_counter()
                O.gemm_f32(xin, p, s, Kw, GROUP, FMT)
                secs += time.perf_counter() - t0
    return secs, n_sample_experts * rows_per_expert, ("reference" if ref is not None else "port")


def cpu_baseline(rows_per_expert: int, budget_s: float = 15.0):
    threads = os.cpu_count() or 1
    s1, rows1, kind = cpu_layer_sample(1, rows_per_expert, threads)  # also sizes the sample
    n = int(max(1, min(8, budget_s / max(s1, 1e-3))))
    secs, rows, kind = cpu_layer_sample(n, rows_per_expert, threads)
    total_rows = TOKENS * TOP_K
    full = secs * total_rows / rows
    return {"value": TOKENS / full, "unit": "tokens/s", "cores": threads, "kind": kind,
            "sample": f"{n} of {N_EXPERTS} experts x {rows_per_expert} routed rows each (3 linears per expert), {secs:.2f} s, "
                      f"extrapolated by rows to {total_rows} rows"}


def run_reference_arm(args):
    """--impl reference: the reference's CPU kernel on this host's cores, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows_per_expert = TOKENS * TOP_K // N_EXPERTS
    s1, _, kind = cpu_layer_sample(1, rows_per_expert, threads)
    n = int(max(1, min(4, 20.0 / max(s1, 1e-3) / max(1, args.steps + args.warmup))))
    for _ in range(args.warmup):
        cpu_layer_sample(n, rows_per_expert, threads)
    t = []
    for _ in range(args.steps):
        secs, rows, kind = cpu_layer_sample(n, rows_per_expert, threads)
        t.append(secs * (TOKENS * TOP_K) / rows)
    ms = 1e3 * float(np.mean(t))
    v = TOKENS / (ms / 1e3)
    sample = f"{n} of {N_EXPERTS} experts x {rows_per_expert} rows per step, extrapolated by rows"
    print(json.dumps({
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def traffic_per_launch(n_gpus: int):
    """DRAM bytes per grouped-GEMM launch (mean of the gate+up and the down launch): dram__bytes_read.sum +
    dram__bytes_write.sum of one ncu capture on the reduced case (96 experts x 4096 tokens: 733 MB and 457 MB,
    profiles/prefill_kernel_tq1_moe_reduced_case.md), scaled by the experts and rows one launch processes (traffic is
    proportional to both). None for workloads the capture does not describe."""
    if FMT != "tq1" or TOKENS * 96 != 4096 * N_EXPERTS:
        return None
    scale = (N_EXPERTS / 96.0) / n_gpus
    return 0.5 * (733.4e6 + 457.1e6) * scale


def workload_config(n_gpus: int) -> dict:
    full = TOKENS == 16384 and N_EXPERTS == 384 and FMT == "tq1"
    return {"workload": "BASELINE config 4: expert-parallel MoE routed-expert layer" if full else
            "REDUCED case of BASELINE config 4 (fewer tokens/experts, same shapes): for profiler captures only", "tokens_per_step": TOKENS, "hidden": HIDDEN,
            "inter": INTER, "experts": N_EXPERTS, "top_k": TOP_K, "format": FMT, "group": GROUP, "scale_dtype": "fp16",
            "parallelism": f"ep{n_gpus}" + (" (dispatch and combine by this library's kernels over peer memory)" if n_gpus > 1 else ""), "l2": "weights (2.09 GB) and activations exceed the 126 MB L2; no flush needed"}


# --------------------------------------------------------------------------------------------- single-kernel numbers
def time_cuda(fn, iters: int, warmup: int = 3) -> float:
    """Mean milliseconds per call, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def gemm_microbench(device, peaks, which="all") -> dict:
    """Decode GEMV (BASELINE configs 0/1) and prefill grouped GEMM (config 2) at N = 1.

    Decode: one launch is a grouped GEMV over `copies` distinct weight sets of the same shape
    (each with its own M rows), so one launch streams > L2 of packed bytes from HBM.
    GB/s counts packed bytes + fp16 scales + bf16 activations in + fp32 outputs."""
    from deepseekternarized_b200.kernels import ternary_b200 as kb
    from deepseekternarized_b200.ternary.pack import pack, packed_cols

    out = {"decode": [], "prefill": []}
    g = torch.Generator(device=device).manual_seed(SEED + 99)

    def weights(E, N, K, fmt):
        p = torch.empty(E, N, packed_cols(fmt, K), dtype=torch.uint8, device=device)
        for e in range(E):
            u = torch.rand(N, K, generator=g, device=device)
            p[e] = pack(torch.where(u < 0.4, 0, torch.where(u < 0.7, 1, -1)).to(torch.int8), fmt)
        s = torch.exp(torch.randn(E, N, K // GROUP, generator=g, device=device) * 0.3 - 4.0).half()
        return kb.tile_weights(p, fmt, K), s  # tiled once, as a loaded model holds them

    decode_cases = (("tq2", 4096, 4096, (1, 16)), ("tq1", 2048, 4096, (1, 8)), ("tq1", 4096, 4096, (1, 4, 8, 32)),
                    ("tq1", 11008, 4096, (1, 8)))
    for fmt, N, K, Ms in (decode_cases if which in ("all", "decode") else ()):
        wbytes = N * packed_cols(fmt, K) + N * (K // GROUP) * 2  # canonical packed bytes + fp16 scales: the algorithmic bytes
        copies = max(2, int(np.ceil(400e6 / wbytes)))
        p, s = weights(copies, N, K, fmt)
        for M in Ms:
            x = torch.randn(copies * M, K, generator=g, device=device).bfloat16()
            offs = torch.arange(copies + 1, device=device, dtype=torch.int64) * M
            fn = lambda: kb.grouped_ternary_gemm_bf16(x, offs, [p], [s], K, GROUP, fmt, validate_offsets=False)
            ms = time_cuda(fn, 5)
            byts = copies * (wbytes + M * K * 2 + M * N * 4)
            gbs = byts / ms / 1e6
            out["decode"].append({"fmt": fmt, "N": N, "K": K, "M": M, "weight_sets_per_launch": copies, "ms": ms, "gbs": gbs,
                                  "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]})
        del p, s
    # config 2: 4096 tokens, 384 experts, top-6 -> 24576 rows; gate+up (N 4096, K 4096) and down (N 4096, K 2048)
    E, rows = N_EXPERTS, 4096 * TOP_K
    ids = torch.randn(4096, E, generator=g, device=device).topk(TOP_K, -1)[1].reshape(-1)
    order, offs = kb.sort_by_expert(ids, E)
    for (N, K) in (((2 * INTER, HIDDEN), (HIDDEN, INTER)) if which in ("all", "prefill") else ()):
        p, s = weights(E, N, K, FMT)
        x = torch.randn(rows, K, generator=g, device=device).bfloat16()
        fn = lambda: kb.grouped_ternary_gemm_bf16(x, offs, [p], [s], K, GROUP, FMT, out_dtype=torch.bfloat16, validate_offsets=False)
        ms = time_cuda(fn, 3, warmup=2)
        tf = 2.0 * rows * N * K / ms / 1e9
        out["prefill"].append({"fmt": FMT, "experts": E, "rows": rows, "N": N, "K": K, "ms": ms, "tflops": tf,
                               "frac_of_measured_bf16": tf / peaks["bf16_tflops"]})
        del p, s
    return out


# --------------------------------------------------------------------------------------------- main arm
def timed_ops(algo):
    """B200Ops plus CUDA events around every grouped GEMM launch and a count of launched kernels."""
    from deepseekternarized_b200.moe import B200Ops

    class _Timed(B200Ops):
        def __init__(self, algo_):
            super().__init__(algo_)
            self.events, self.launches, self.flops, self.timing = [], 0, 0.0, False

        def count(self, n):  # kernels launched by the layer itself (peer-memory dispatch / combine)
            self.launches += n

        def route(self, *a, **k):
            self.launches += 1
            return super().route(*a, **k)

        def sort(self, *a):
            self.launches += 3
            return super().sort(*a)

        def gather(self, *a, **k):
            self.launches += 1
            return super().gather(*a, **k)

        def swiglu(self, *a, **k):
            self.launches += 1
            return super().swiglu(*a, **k)

        def combine(self, *a):
            self.launches += 2
            return super().combine(*a)

        def gemm(self, x, offsets, packed, scales, K, group, fmt, out=None):
            self.launches += 1
            if not self.timing:
                return super().gemm(x, offsets, packed, scales, K, group, fmt, out=out)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            y = super().gemm(x, offsets, packed, scales, K, group, fmt, out=out)
            b.record()
            self.events.append((a, b))
            self.flops += 2.0 * x.size(0) * packed[0].size(1) * K
            return y

    return _Timed(algo)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--no-micro", action="store_true", help="skip the single-kernel decode/prefill numbers")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--micro-only", default=None, choices=["decode", "prefill", "all"],
                    help="run only the single-kernel numbers (decode GEMV sweep and/or prefill grouped GEMM) and print them: "
                    "for profiler captures of those kernels; not a bench line")
    ap.add_argument("--tokens", type=int, default=TOKENS, help="tokens per step over all ranks (default: BASELINE config 4)")
    ap.add_argument("--experts", type=int, default=N_EXPERTS, help="routed experts (default: BASELINE config 4); smaller "
                    "values give a reduced case for profiler captures and are named in the JSON line")
    ap.add_argument("--fmt", default=FMT, choices=["tq1", "tq2"], help="packing of the expert weights (default: BASELINE config 4, tq1)")
    args = ap.parse_args()
    globals()["TOKENS"], globals()["N_EXPERTS"], globals()["FMT"] = args.tokens, args.experts, args.fmt
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.micro_only:
        device = torch.device("cuda:0")
        torch.cuda.set_device(device)
        print(json.dumps({"micro_only": args.micro_only, "gemm": gemm_microbench(device, measured_peaks(), which=args.micro_only)}))
        return

    import torch.distributed as dist

    from deepseekternarized_b200.moe import B200Ops, ExpertParallelMoE, HostPipeline, MoELayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the CUDA library has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peaks = measured_peaks()

    n_local = N_EXPERTS // world
    t_local = TOKENS // world
    weights = synth_expert_weights(n_local, rank * n_local, device)
    ops = timed_ops(args.algo)
    layer = ExpertParallelMoE(weights, N_EXPERTS, TOP_K, ops=ops) if world > 1 else MoELayer(weights, TOP_K, ops=ops)
    x_host, logits_host = synth_tokens(t_local, rank * t_local)
    x_dev, logits_dev = x_host.to(device), logits_host.to(device)
    y_host = torch.empty(t_local, HIDDEN, dtype=torch.bfloat16).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_resident():
        return layer(x_dev, logits_dev)

    # the public host-buffer call: every step copies its inputs from pinned host memory and returns its result to host
    # memory; the copies of neighbouring steps overlap with compute on their own streams
    pipe = HostPipeline(layer, t_local, HIDDEN, N_EXPERTS, device)

    def step_e2e():
        pipe.submit(x_host, logits_host, y_host)

    def timed(fn, steps, finish=None):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()  # the closing event waits for the last result copy on its side stream
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step_resident()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # started ahead of the timed region (nvidia-smi takes a moment to deliver its first sample)
    sampler.mark_load()
    t_load = time.time()
    while True:  # the same steps, untimed, for at least 0.4 s: clocks settle and the sampler sees the GPU under this load
        for _ in range(20):
            step_resident()
        torch.cuda.synchronize()
        go = torch.tensor([1 if time.time() - t_load < 0.4 else 0], device=device)
        if world > 1:
            dist.all_reduce(go, op=dist.ReduceOp.MAX)  # every rank leaves the loop after the same number of steps
        if int(go.item()) == 0:
            break
    ops.launches, ops.timing = 0, True
    sampler.mark_begin()
    total_ms = timed(step_resident, args.steps)
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    launches = ops.launches
    ops.timing = False
    gemm_ms = [a.elapsed_time(b) for a, b in ops.events]
    gemm_flops = ops.flops
    for _ in range(2):
        step_e2e()
    e2e_ms = timed(step_e2e, args.steps, pipe.join)

    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = TOKENS / (ms_per_step / 1e3)
        achieved = gemm_flops / (sum(gemm_ms) / 1e3) / 1e12 if gemm_ms else None
        peak = peaks["bf16_tflops_sustained"]
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 operands (bf16 activations, exact fp16 scale*trit weights), f32 accumulation",
            "data": "synthetic", "config": workload_config(world), "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": TOKENS / (e2e_ms / args.steps / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(x_host.numel() * 2 + logits_host.numel() * 4) * world,
                    "d2h_bytes_per_step": int(y_host.numel() * 2) * world,
                    "call": "HostPipeline.submit per step (pinned host inputs and result; the copies of neighbouring steps "
                            "overlap with compute on two side streams; the closing event waits for the last result copy)"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": (achieved / peak) if achieved else None, "traffic": traffic_per_launch(world),
                         "kernel": "grouped expert GEMM (2 launches per step: gate+up, down)", "peak_source": peaks["source"] + " (sustained)",
                         "ms_per_launch": float(np.mean(gemm_ms)) if gemm_ms else None},
        }
        if world == 1 and not args.no_micro:
            line["gemm"] = gemm_microbench(device, peaks)
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(TOKENS * TOP_K // N_EXPERTS)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

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
                BASELINE config 0/1/2/3 shapes, each with its roofline fraction, its launch count and
                the clocks sampled during its own timed loops.
  parity_check  (N = 1 only) the output of the last timed step checked against the CPU oracle on a
                sample (see parity_check()).
  repeats       the timed region (exactly --steps steps) is run --repeats times; value, ms_per_step and
                e2e are the median region, with the fastest and slowest beside them.

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
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def close(self):
        if self.proc is not None:
            self.proc.terminate()  # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def window(self, t0: float, t1: float) -> dict:
        """Clock summary of the samples read between two host times (the sampler keeps running)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        return self._summary([ln for ts, ln in self.lines if t0 <= ts <= t1 + 0.05], "timed loops of this case")

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        inside = [ln for ts, ln in self.lines if self.t0 is None or (self.t0 <= ts <= (self.t1 or ts) + 0.05)]
        window = "timed region"
        if len(inside) < 3 and self.t_load is not None:
            # a timed region of a few sampling periods at most: add the samples of the identical steps run right before it
            inside = [ln for ts, ln in self.lines if self.t_load <= ts <= (self.t1 or ts) + 0.05]
            window = "timed region and the identical untimed steps directly before it"
        return self._summary(inside, window)

    def _summary(self, inside, window) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
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
            p = O.pack(O.synth_trits(rng, (Nw, Kw)), FMT)  # trits i.i.d. P(0) = 0.4, P(+-1) = 0.3, as the GPU arm's weights
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
    n = int(max(4, min(16, 240.0 / max(s1, 1e-3) / max(1, args.steps + args.warmup))))  # at least four experts per step
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
    dram__bytes_write.sum of one ncu capture on the reduced case (96 experts x 4096 tokens: 733 MB and 457 MB),
    scaled by the experts and rows one launch processes (traffic is proportional to both). A constant from that
    capture, not a measurement of this run; None for workloads the capture does not describe."""
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
def time_cuda(fn, iters: int, warmup: int = 3, repeats: int = 3, min_loop_ms: float = 60.0) -> dict:
    """Milliseconds per call from CUDA events on the current stream: `repeats` timed loops of at least `iters` calls
    and at least `min_loop_ms` each (long enough for the clock sampler to see the kernel under load); the median loop
    is the value, with the fastest and slowest beside it and the host-clock window of the loops."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        fn()
    b.record()
    torch.cuda.synchronize()
    iters = int(max(iters, min(2000, min_loop_ms / max(a.elapsed_time(b) / 5, 1e-3))))
    t0 = time.time()
    ms = []
    for _ in range(repeats):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b) / iters)
    return {"ms": float(np.median(ms)), "ms_min": float(min(ms)), "ms_max": float(max(ms)), "launches": iters * repeats,
            "window": (t0, time.time())}


def gemm_microbench(device, peaks, which="all", sampler=None, only=None) -> dict:
    """Single-kernel numbers at N = 1: decode GEMV (BASELINE configs 0, 1 and 3), prefill grouped GEMM (configs 2
    and 3, and the int8-activation mode on the config-2 shape) and the ternary lookup-table rows.

    Decode: one launch is a grouped GEMV over `copies` distinct weight sets of the same shape (each with its own M
    rows), so one launch streams > L2 of packed bytes from HBM. GB/s counts the CANONICAL packed bytes of the format
    named in the line + fp16 scales + bf16 activations in + fp32 outputs. TQ1 appears twice: read from its TQ1 tiles
    (1.6 bits per trit on the device) and read from a tiled TQ2 copy of the same trits (2 bits per trit on the device,
    "device_copy": "tq2"); both lines count TQ1's canonical bytes, so they compare as wall time."""
    from deepseekternarized_b200.kernels import ternary_b200 as kb
    from deepseekternarized_b200.ternary.ops import quant_act_int8
    from deepseekternarized_b200.ternary.pack import pack, packed_cols

    out = {"decode": [], "prefill": [], "table_lookup": []}
    g = torch.Generator(device=device).manual_seed(SEED + 99)

    def clocks(t):
        return sampler.window(*t.pop("window")) if sampler is not None else t.pop("window") and None

    def weights(E, N, K, fmt, k_terms=1, decode_copy=False):
        ps, ss = [], []
        for i in range(k_terms):
            p = torch.empty(E, N, packed_cols(fmt, K), dtype=torch.uint8, device=device)
            for e in range(E):
                u = torch.rand(N, K, generator=g, device=device)
                p[e] = pack(torch.where(u < 0.4, 0, torch.where(u < 0.7, 1, -1)).to(torch.int8), fmt)
            sc = torch.exp(torch.randn(E, N, K // GROUP, generator=g, device=device) * 0.3 - 4.0) * (0.25 if i else 1.0)
            ps.append(kb.tile_weights(p, fmt, K, decode_copy))  # tiled once, as a loaded model holds them
            ss.append(sc.half())
        return ps, ss

    # (format, N, K, Ms, stacked terms, read TQ1 through a tiled TQ2 copy of its trits)
    decode_cases = (("tq2", 4096, 4096, (1, 16), 1, False),
                    ("tq1", 2048, 4096, (1, 8), 1, False), ("tq1", 4096, 4096, (1, 4, 8, 32), 1, False), ("tq1", 11008, 4096, (1, 8), 1, False),
                    ("tq1", 2048, 4096, (1, 8), 1, True), ("tq1", 4096, 4096, (1, 4, 8, 32), 1, True), ("tq1", 11008, 4096, (1, 8), 1, True),
                    ("tq2", 2048, 4096, (1, 8, 64), 2, False), ("tq2", 4096, 2048, (1, 8, 64), 2, False))  # config 3: k = 2
    for fmt, N, K, Ms, k_terms, copy in (decode_cases if which in ("all", "decode") else ()):
        if only is not None and f"{fmt}:{N}:{K}:{k_terms}:{'copy' if copy else 'tiles'}" != only:
            continue  # a profiler capture of one case
        wbytes = k_terms * (N * packed_cols(fmt, K) + N * (K // GROUP) * 2)  # canonical packed bytes + fp16 scales: the algorithmic bytes
        copies = max(2, int(np.ceil(400e6 / wbytes)))
        p, s = weights(copies, N, K, fmt, k_terms, copy)
        for M in Ms:
            x = torch.randn(copies * M, K, generator=g, device=device).bfloat16()
            offs = torch.arange(copies + 1, device=device, dtype=torch.int64) * M
            fn = lambda: kb.grouped_ternary_gemm_bf16(x, offs, p, s, K, GROUP, fmt, validate_offsets=False)
            t = time_cuda(fn, 20)
            byts = copies * (wbytes + M * K * 2 + M * N * 4)
            gbs = byts / t["ms"] / 1e6
            line = {"fmt": fmt, "N": N, "K": K, "M": M, "terms": k_terms, "weight_sets_per_launch": copies, "gbs": gbs,
                    "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "clocks": clocks(t), **t}
            if copy:
                line["device_copy"] = "tq2"
            out["decode"].append(line)
        del p, s
    # Ternary lookup-table rows (the engram tables: 256-wide rows, group 128, TQ1, one or two stacked terms; a step of
    # 16 384 tokens looks up 24 rows per token). Table and output are larger than L2; GB/s counts packed row + scales + id
    # + the bf16 row written, per looked-up row.
    if which in ("all", "tables") and only is None:
        from deepseekternarized_b200.ternary.ops import LookupTable, PackedTerm, gather_dequant_rows

        V, K, n_ids = 4 * 1024 * 1024, 256, 24 * TOKENS
        ids = torch.randint(0, V, (n_ids,), generator=g, device=device)
        for fmt, k_terms in (("tq1", 2), ("tq1", 1), ("tq2", 1)):
            Kp = packed_cols(fmt, K)
            hi = 243 if fmt == "tq1" else 256
            terms = []
            for i in range(k_terms):
                pk = torch.randint(0, hi, (V, Kp), generator=g, device=device, dtype=torch.uint8)
                if fmt == "tq2":  # no 2-bit field holds the value 3
                    pk = pk & ~((pk >> 1) & pk & 0x55 | (((pk >> 1) & pk & 0x55) << 1))
                terms.append(PackedTerm(pk, torch.exp(torch.randn(V, K // GROUP, generator=g, device=device) * 0.3 - 4.0).half()))
            byts = n_ids * (k_terms * (Kp + (K // GROUP) * 2) + 8 + K * 2)
            table = LookupTable(terms, K, fmt, GROUP)
            for layout, fn in (("canonical arrays", lambda: gather_dequant_rows(terms, ids, K, fmt, GROUP, check=False)),
                               (f"one {table.record}-byte record per row", lambda: table.rows(ids, check=False))):
                t = time_cuda(fn, 20)
                gbs = byts / t["ms"] / 1e6
                out["table_lookup"].append({"fmt": fmt, "terms": k_terms, "layout": layout, "table_rows": V, "K": K, "rows_looked_up": n_ids,
                                            "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "clocks": clocks(t), **t})
            del terms, table
    # config 2: 4096 tokens, 384 experts, top-6 -> 24576 rows; gate+up (N 4096, K 4096) and down (N 4096, K 2048);
    # then the same shapes with two stacked TQ2 terms (config 3 prefill) and with int8 activations (the policy default)
    E, rows = N_EXPERTS, 4096 * TOP_K
    ids = torch.randn(4096, E, generator=g, device=device).topk(TOP_K, -1)[1].reshape(-1)
    order, offs = kb.sort_by_expert(ids, E)
    prefill_cases = (("tq1", 1, "bf16"), ("tq2", 2, "bf16"), ("tq1", 1, "int8"))
    for fmt, k_terms, act in (prefill_cases if which in ("all", "prefill") else ()):
        for (N, K) in ((2 * INTER, HIDDEN), (HIDDEN, INTER)):
            p, s = weights(E, N, K, fmt, k_terms)
            x = torch.randn(rows, K, generator=g, device=device).bfloat16()
            if act == "int8":  # the resident int8 path: quantise into the kernel's row format (timed), then the GEMM
                fn = lambda: kb.grouped_ternary_gemm_bf16(kb.NormRows(*quant_act_int8(x, as_f16=True)), offs, p, s, K, GROUP, fmt,
                                                          out_dtype=torch.float32, validate_offsets=False)
            else:
                fn = lambda: kb.grouped_ternary_gemm_bf16(x, offs, p, s, K, GROUP, fmt, out_dtype=torch.bfloat16, validate_offsets=False)
            t = time_cuda(fn, 17, warmup=2)
            tf = 2.0 * rows * N * K / t["ms"] / 1e9
            out["prefill"].append({"fmt": fmt, "terms": k_terms, "act": act, "experts": E, "rows": rows, "N": N, "K": K, "tflops": tf,
                                   "frac_of_measured_bf16": tf / peaks["bf16_tflops"], "clocks": clocks(t), **t})
            del p, s
    return out


# --------------------------------------------------------------------------------------------- parity of the benched output
def parity_check(layer, weights, x_dev, logits_dev, y_timed, n_experts_checked: int = 6, n_tokens_checked: int = 64) -> dict:
    """Checks the output of the last timed step (N = 1): the layer's steps are run once more on the same inputs with
    their intermediates kept; their result must equal the timed step's bit for bit. Then, against the CPU oracle (a
    checker only): routing ids of every token, the float32 outputs of both grouped GEMMs for a sample of experts
    against the fp64 dequantized product (the north-star tolerance: rel. Frobenius <= 2e-3, cosine >= 0.99999), and
    the combine of a sample of tokens recomputed from the GPU's own expert outputs (bit-exact)."""
    from deepseekternarized_b200.kernels import ternary_b200 as kb
    from deepseekternarized_b200.synth import expert_tensors
    from oracle import oracle as O

    ops, w, k = layer.ops, layer.w, layer.top_k
    T, E, hidden, inter, fmt = x_dev.size(0), w.n_experts, w.hidden, w.inter, w.fmt
    wts, ids = layer.route(logits_dev)
    order, offsets = ops.sort(ids, E)
    xs = layer.gather_for_experts(x_dev, order, k)
    gu = ops.gemm(xs, offsets, w.w13_packed, w.w13_scale, hidden, GROUP, fmt)
    gu32 = kb.grouped_ternary_gemm_bf16(xs, offsets, w.w13_packed, w.w13_scale, hidden, GROUP, fmt, out_dtype=torch.float32, validate_offsets=False)
    h = ops.swiglu(gu, wts.reshape(-1), order, inter, 0.0, for_weights=w.w2_packed)
    down = ops.gemm(h, offsets, w.w2_packed, w.w2_scale, inter, GROUP, fmt)
    down32 = kb.grouped_ternary_gemm_bf16(h, offsets, w.w2_packed, w.w2_scale, inter, GROUP, fmt, out_dtype=torch.float32, validate_offsets=False)
    y = ops.combine(down, order, ids, T, k)
    same = bool(torch.equal(y, y_timed))
    logits = logits_dev.cpu().numpy()
    w_ref, idx_ref = O.route_from_logits(logits, k)
    ids_ok = bool(np.array_equal(ids.cpu().numpy(), idx_ref))
    offs = offsets.cpu().numpy()
    order_h = order.cpu().numpy()
    counts = np.diff(offs)
    rng = np.random.default_rng(SEED)
    nonempty = np.nonzero(counts)[0]
    picks = {int(nonempty[np.argmin(counts[nonempty])]), int(np.argmax(counts)), int(nonempty[0]), int(nonempty[-1])}
    picks |= {int(v) for v in rng.choice(nonempty, max(0, n_experts_checked - 4), replace=False)}
    x = x_dev.float().cpu().numpy()
    h_rows = (h.data.float() * h.factor[:, None]) if isinstance(h, kb.NormRows) else h.float()
    rel, cos = 0.0, 1.0
    for e in sorted(picks):
        a, b = int(offs[e]), int(offs[e + 1])
        ts = expert_tensors(SEED, e, hidden, inter, fmt, 1, x_dev.device)
        w13 = [(t[0].cpu().numpy(), t[1].cpu().numpy()) for t in ts]
        w2 = [(t[2].cpu().numpy(), t[3].cpu().numpy()) for t in ts]
        for got, rows, terms, K in ((gu32[a:b].cpu().numpy(), x[order_h[a:b] // k], w13, hidden),
                                    (down32[a:b].cpu().numpy(), h_rows[a:b].cpu().numpy(), w2, inter)):
            y64 = O.gemm_f64(rows, terms, K, GROUP, fmt)
            rel, cos = max(rel, O.rel_fro(got, y64)), min(cos, O.cosine(got, y64))
    inv = np.empty(T * k, np.int64)
    inv[order_h] = np.arange(T * k)
    toks = rng.choice(T, min(n_tokens_checked, T), replace=False)
    pos = np.stack([inv[t * k + np.argsort(idx_ref[t], kind="stable")] for t in toks])
    d = down[torch.from_numpy(pos.reshape(-1)).to(x_dev.device)].float().cpu().numpy().reshape(len(toks), k, hidden)
    acc = np.zeros((len(toks), hidden), np.float32)
    for sl in range(k):
        acc += d[:, sl]
    comb = bool(np.array_equal(O.bf16_bits(y[torch.from_numpy(toks).to(x_dev.device)].float().cpu().numpy()), O.bf16_bits(O.bf16_round(acc))))
    return {"timed_output_equals_checked_steps": same, "routing_ids_exact": ids_ok, "rel_fro": rel, "cos": cos, "experts": len(picks),
            "gemm_tolerance_met": bool(rel <= 2e-3 and cos >= 0.99999), "combine_exact": comb, "tokens": int(len(toks)),
            "against": "CPU oracle: fp64 dequantized product of the sampled experts' rows; combine recomputed from the GPU's expert outputs"}


# --------------------------------------------------------------------------------------------- main arm
def timed_ops(algo):
    """B200Ops plus CUDA events around every grouped GEMM launch and a count of launched kernels."""
    from deepseekternarized_b200.moe import B200Ops

    class _Timed(B200Ops):
        def __init__(self, algo_):
            super().__init__(algo_)
            self.events, self.launches, self.flops, self.timing = [], 0, 0.0, False
            self.world = int(os.environ.get("WORLD_SIZE", "1"))

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
            # rows this launch multiplies: all of x on one GPU; under expert parallelism x is the receive buffer's whole
            # capacity and the rows that exist are the routed rows of this rank's experts: 1 / world of them on average
            rows = x.size(0) if self.world == 1 else TOKENS * TOP_K / self.world
            self.flops += 2.0 * rows * packed[0].size(1) * K
            return y

    return _Timed(algo)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ep-combine", default="auto", choices=["auto", "scatter", "pull"],
                    help="N > 1: how the experts' outputs return to their tokens' ranks (ExpertParallelMoE's combine)")
    ap.add_argument("--repeats", type=int, default=7, help="timed regions of --steps steps each; the median region is reported")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--no-micro", action="store_true", help="skip the single-kernel decode/prefill numbers")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-check", action="store_true", help="skip the parity check of the last timed step's output")
    ap.add_argument("--micro-only", default=None, choices=["decode", "prefill", "tables", "all"],
                    help="run only the single-kernel numbers (decode GEMV sweep and/or prefill grouped GEMM) and print them: "
                    "for profiler captures of those kernels; not a bench line")
    ap.add_argument("--micro-case", default=None, help="with --micro-only decode: run one decode case, named fmt:N:K:terms:tiles|copy "
                    "(e.g. tq2:4096:4096:1:tiles), for a profiler capture")
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
        sampler = ClockSampler(0)
        sampler.start()
        print(json.dumps({"micro_only": args.micro_only, "gemm": gemm_microbench(device, measured_peaks(), which=args.micro_only, sampler=sampler, only=args.micro_case)}))
        sampler.close()
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
    layer = ExpertParallelMoE(weights, N_EXPERTS, TOP_K, ops=ops, combine=args.ep_combine) if world > 1 else MoELayer(weights, TOP_K, ops=ops)
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
    region_ms = [timed(step_resident, args.steps) for _ in range(max(1, args.repeats))]  # each exactly --steps steps
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    launches = ops.launches // max(1, args.repeats)
    ops.timing = False
    total_ms = float(np.median(region_ms))
    gemm_ms = [a.elapsed_time(b) for a, b in ops.events]
    gemm_flops = ops.flops
    y_last = step_resident()
    phases = None
    if world > 1 and hasattr(layer, "phases_ms"):
        # a separate, untimed pass with a CUDA event after every phase of the expert-parallel step
        layer.profile_phases = True
        for _ in range(20):
            step_resident()
        torch.cuda.synchronize()
        layer.profile_phases = False
        phases = layer.phases_ms()
        pm = torch.tensor(list(phases.values()), device=device)
        dist.all_reduce(pm, op=dist.ReduceOp.MAX)  # the slowest rank's median per phase
        phases = {k: float(v) for k, v in zip(phases.keys(), pm.tolist())}
    for _ in range(2):
        step_e2e()
    e2e_region_ms = [timed(step_e2e, args.steps, pipe.join) for _ in range(max(1, args.repeats))]
    e2e_ms = float(np.median(e2e_region_ms))

    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = TOKENS / (ms_per_step / 1e3)
        achieved = gemm_flops / (sum(gemm_ms) / 1e3) / 1e12 if gemm_ms else None
        peak = peaks["bf16_tflops_sustained"]
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "repeats": max(1, args.repeats),
            "ms_per_step_min": min(region_ms) / args.steps, "ms_per_step_max": max(region_ms) / args.steps,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 operands (bf16 activations, exact fp16 scale*trit weights), f32 accumulation",
            "data": "synthetic", "config": workload_config(world), "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": TOKENS / (e2e_ms / args.steps / 1e3), "unit": "tokens/s",
                    "value_min": TOKENS / (max(e2e_region_ms) / args.steps / 1e3), "value_max": TOKENS / (min(e2e_region_ms) / args.steps / 1e3),
                    "h2d_bytes_per_step": int(x_host.numel() * 2 + logits_host.numel() * 4) * world,
                    "d2h_bytes_per_step": int(y_host.numel() * 2) * world,
                    "call": "HostPipeline.submit per step (pinned host inputs and result; the copies of neighbouring steps "
                            "overlap with compute on two side streams; the closing event waits for the last result copy)"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": (achieved / peak) if achieved else None, "traffic": traffic_per_launch(world),
                         "traffic_source": "ncu capture of the reduced case (96 experts x 4096 tokens), scaled by experts and rows; not measured in this run",
                         "ms_per_launch_min": float(np.min(gemm_ms)) if gemm_ms else None, "ms_per_launch_max": float(np.max(gemm_ms)) if gemm_ms else None,
                         "launches_timed": len(gemm_ms),
                         "kernel": "grouped expert GEMM (2 launches per step: gate+up, down)", "peak_source": peaks["source"] + " (sustained)",
                         "ms_per_launch": float(np.mean(gemm_ms)) if gemm_ms else None},
        }
        if phases is not None:
            line["phases_ms"] = {**phases, "sum": float(sum(phases.values())),
                                 "note": "median over 20 untimed steps with a CUDA event after each phase, max over ranks"}
        if world == 1 and not args.no_check:
            line["parity_check"] = parity_check(layer, weights, x_dev, logits_dev, y_last)
        if world == 1 and not args.no_micro:
            line["gemm"] = gemm_microbench(device, peaks, sampler=sampler)
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(TOKENS * TOP_K // N_EXPERTS)
        print(json.dumps(line))
    sampler.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

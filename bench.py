#!/usr/bin/env python
"""Benchmark of the fused-MoE hot path.

    python bench.py --gpus N --steps K --warmup W [--config C1] [--impl reference]

A "step" is one pass of the fused operator (moe_sorting -> gemm1+SiLU*up -> gemm2 -> combine)
over one batch of synthetic tokens.  At N=1 the workload is the Mixtral-8x7B-shape bf16
prefill configuration (tokens=4096, hidden=4096, intermediate=14336, experts=8, topk=2).
For N>1 the same global batch is split expert-parallel: tokens data-parallel, experts
sharded, NCCL all-to-all dispatch and return around the local operator ("strong" scaling).

One JSON line is printed by rank 0.  `value` is TFLOP/s with inputs resident in HBM, `e2e`
the same metric with host buffers (pinned H2D of activations and routing, D2H of the
output, every step), `roofline` the dominant kernel (gate+up GEMM) against the measured
dense bf16 peak, `cpu_baseline` the CPU oracle timed on a bounded token sample.

`--impl reference` times the CPU implementation of the same path (the repository's CPU
restatement: the reference project ships no source for this operator) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (T, H, I, E, K, quant)
    "C0": dict(T=128, H=512, I=1024, E=8, K=2, quant=0, label="cpu-ref-shape-bf16"),
    "C1": dict(T=4096, H=4096, I=14336, E=8, K=2, quant=0, label="mixtral-8x7b-prefill-bf16"),
    "C2": dict(T=8192, H=4096, I=14336, E=8, K=2, quant=1, label="mixtral-8x7b-prefill-fp8"),
    "C3": dict(T=16, H=4096, I=14336, E=8, K=2, quant=1, label="mixtral-8x7b-decode-fp8"),
    "C4": dict(T=8192, H=7168, I=2048, E=256, K=8, quant=2, routing="sigmoid",
               label="deepseek-v3-shape-fp8-block128"),
    # the same shape with power-of-two (UE8M0) scales applied inside the tensor core
    "C4m": dict(T=8192, H=7168, I=2048, E=256, K=8, quant=3, routing="sigmoid",
                label="deepseek-v3-shape-fp8-block128-ue8m0"),
}
QUANT_NAME = {0: "none", 1: "token_channel", 2: "block128", 3: "block128_ue8m0"}


def quantise_weight(wf, quant):
    """f32 [rows, cols] on the device -> (stored tensor, scales or None)."""
    import torch
    if quant == 0:
        return wf.to(torch.bfloat16), None
    if quant == 1:
        s = wf.abs().amax(dim=1) / 448.0
        s = torch.where(s > 0, s, torch.ones_like(s))
        return (wf * (1.0 / s)[:, None]).to(torch.float8_e4m3fn).view(torch.uint8), s
    rows, cols = wf.shape
    blocks = wf.view(rows // 128, 128, cols // 128, 128)
    s = blocks.abs().amax(dim=(1, 3)) / 448.0
    s = torch.where(s > 0, s, torch.ones_like(s))
    if quant == 3:      # power-of-two scales: the smallest power of two >= absmax/448
        s = torch.exp2(torch.ceil(torch.log2(s)))
    q = (blocks * (1.0 / s)[:, None, :, None]).to(torch.float8_e4m3fn).view(torch.uint8).view(rows, cols)
    return q, s.contiguous()


def route_on_device(logits, K, mode):
    import torch
    p = torch.softmax(logits, dim=-1) if mode == "softmax" else torch.sigmoid(logits)
    w, ids = torch.topk(p, K, dim=-1)
    w = (w / w.sum(dim=-1, keepdim=True)).float().contiguous()
    return ids.to(torch.int32).contiguous(), w

# DRAM bytes (dram__bytes_read.sum, dram__bytes_write.sum) of one gate+up GEMM launch on the
# workload of each configuration, each from the ncu capture summarised in the named file under
# profiles/ (the figures appear there as quoted).  A configuration whose kernel changed since its
# last capture has no entry and reports traffic = null.
GEMM1_DRAM_TRAFFIC = {
    "C1": dict(read=1957748480, write=241425664, source="profiles/grouped_gemm_bf16_mixtral_prefill.md",
               quotes=["1,957,748,480 B read + 241,425,664 B written"]),
    "C2": dict(read=1.300e9, write=456e6, source="profiles/grouped_gemm_pair_fp8_mixtral_prefill.md",
               quotes=["1.300 GB / 456 MB"]),
    "C3": dict(read=942.0e6, write=5.8e6, source="profiles/decode_fp8_stage_times.md", quotes=["942.0 MB + 5.8 MB"]),
    # captured on one eighth of the workload (32 of 256 experts, 1024 of 8192 tokens: the same rows
    # per expert); weights, activations and outputs all scale with that factor
    "C4m": dict(read=8 * 1.035734e9, write=8 * 19.909376e6, source="profiles/deepseek_block128_ue8m0_fp8.md",
                quotes=["1.035734", "19.909376"], scaled="x8 from the 32-expert / 1024-token capture"),
}
NOMINAL = dict(bf16_tflops=2250.0, fp8_tflops=4500.0, hbm_gbs=8000.0)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_burst=d["bf16_tflops"],
                    bf16_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


_FP8_PEAK = None


def measure_fp8_peak(dev):
    """Dense e4m3 tensor throughput of this GPU, measured once per run and only as a roofline
    denominator: torch._scaled_mm (cuBLASLt) on 8192^3, best of 10 launches (burst) and launches
    back to back for about four seconds (sustained) -- the way MEASURED_PEAKS.json holds the bf16
    figure.  Runs outside every timed region.  Returns None when the call is unavailable."""
    global _FP8_PEAK
    if _FP8_PEAK is not None:
        return _FP8_PEAK or None
    import torch
    try:
        n = 8192
        a = (torch.randn(n, n, device=dev) * 0.5).to(torch.float8_e4m3fn)
        b = (torch.randn(n, n, device=dev) * 0.5).to(torch.float8_e4m3fn).t()     # column-major operand
        one = torch.ones((), device=dev)

        def mm():
            return torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            mm()
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); mm(); e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        fl = 2.0 * n ** 3
        reps = max(10, int(4000.0 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            mm()
        e1.record(); torch.cuda.synchronize()
        _FP8_PEAK = dict(burst=fl / best / 1e9, sustained=fl * reps / e0.elapsed_time(e1) / 1e9,
                         how="torch._scaled_mm e4m3 8192^3, best of 10 and back to back for ~4 s")
        del a, b
    except Exception as exc:  # noqa: BLE001
        print(f"fp8 peak not measured: {exc!r}", file=sys.stderr)
        _FP8_PEAK = {}
    return _FP8_PEAK or None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        self.t = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0: float, t1: float) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [r for r in self.rows if t0 <= r[0] <= t1] or self.rows
        for _, line in rows:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


def flops_per_step(c) -> float:
    return 6.0 * c["T"] * c["K"] * c["H"] * c["I"]


# ------------------------------------------------------------------------------ CPU arm

def make_host_inputs(c, seed=0):
    """Synthetic inputs on the host: activations N(0,1), weights N(0,0.02), softmax top-K."""
    import torch
    from oracle import oracle as O
    T, H, I, E, K, quant = c["T"], c["H"], c["I"], c["E"], c["K"], c["quant"]
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=dev).cpu().numpy()
    ids, w = O.route(logits, K, c.get("routing", "softmax"))

    def weights(rows, cols):
        out_q, out_s = [], []
        for _ in range(E):
            q, sc = quantise_weight(torch.randn(rows, cols, generator=g, device=dev) * 0.02, quant)
            out_q.append((q.view(torch.int16) if quant == 0 else q).cpu())
            if sc is not None:
                out_s.append(sc.cpu())
        q = torch.stack(out_q).numpy()
        return (q.view(np.uint16) if quant == 0 else q), (torch.stack(out_s).numpy() if out_s else None)

    w1, s1 = weights(2 * I, H)
    w2, s2 = weights(H, I)
    return dict(x=x.view(torch.int16).cpu().numpy().view(np.uint16), w1=w1, w2=w2, w1_scale=s1, w2_scale=s2,
                topk_ids=ids, topk_w=w, quant=quant)


def host_cores() -> int:
    """Host threads the CPU arm uses: the cores this process may run on (torchrun exports
    OMP_NUM_THREADS=1, which would otherwise pin the OpenMP runtime to one thread)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_time_tokens(d, sel, threads=0):
    from oracle import oracle as O
    threads = threads or host_cores()
    t0 = time.perf_counter()
    O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], d["quant"], d["w1_scale"], d["w2_scale"],
                sel=sel, n_threads=threads)
    return time.perf_counter() - t0


def cpu_sample_size(d, c, budget_s: float, n_calls: int) -> int:
    """Tokens per timed call so that n_calls calls take about budget_s."""
    from oracle import oracle as O
    probe = np.arange(min(host_cores(), c["T"]), dtype=np.int32)
    t = max(cpu_time_tokens(d, probe), 1e-4)
    per_token = t / len(probe)
    n = int(budget_s / max(n_calls, 1) / per_token)
    n = max(len(probe), min(c["T"], n))
    return n


def run_reference(a, c):
    """CPU implementation of the path on the host cores, a bounded token sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    d = make_host_inputs(c)
    cores = host_cores()
    n = cpu_sample_size(d, c, budget_s=90.0, n_calls=a.steps + a.warmup)
    rng = np.random.default_rng(0)
    for _ in range(a.warmup):
        cpu_time_tokens(d, rng.choice(c["T"], n, replace=False).astype(np.int32))
    t = 0.0
    for _ in range(a.steps):
        t += cpu_time_tokens(d, rng.choice(c["T"], n, replace=False).astype(np.int32))
    fl = 6.0 * n * c["K"] * c["H"] * c["I"] * a.steps
    val = fl / t / 1e12
    sample = f"{n} of {c['T']} tokens per step (full weights, all {c['E']} experts), {a.steps} steps"
    cfg = workload_config(c, a.gpus)
    cfg["tokens"] = n                      # what one timed step processed
    cfg["full_batch_tokens"] = c["T"]
    line = {"impl": "reference", "metric": "fused_moe_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": t / a.steps * 1e3,
            "full_batch_ms_estimate": t / a.steps * 1e3 * (c["T"] / n),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype_name(c),
            "data": "synthetic", "config": cfg,
            "tokens_per_s": n * a.steps / t,
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement of the operator (the reference project ships no source for it); "
                    "ms_per_step is the measured time of one step over the token sample, "
                    "full_batch_ms_estimate scales it to the full batch"}
    print(json.dumps(line), flush=True)


def dtype_name(c):
    return "bf16" if c["quant"] == 0 else "fp8_e4m3"


def host_copy_of(d, c):
    """Device tensors of device_inputs() -> the numpy arrays the CPU oracle takes."""
    import torch
    w1 = d.get("w1_rowmajor", d["w1"])
    w2 = d.get("w2_rowmajor", d["w2"])
    hd = dict(x=d["x_full"].view(torch.int16).cpu().numpy().view(np.uint16),
              w1=(w1.view(torch.int16) if c["quant"] == 0 else w1).cpu().numpy(),
              w2=(w2.view(torch.int16) if c["quant"] == 0 else w2).cpu().numpy(),
              w1_scale=None if d["s1"] is None else d["s1"].cpu().numpy(),
              w2_scale=None if d["s2"] is None else d["s2"].cpu().numpy(),
              topk_ids=d["ids_full"].cpu().numpy(), topk_w=d["w_full"].cpu().numpy(), quant=c["quant"])
    if c["quant"] == 0:
        hd["w1"], hd["w2"] = hd["w1"].view(np.uint16), hd["w2"].view(np.uint16)
    return hd


def parity_sample(hd, c, got_rows, sel, partial_bf16=False):
    """Relative L2 error of the benchmarked output rows `got_rows` (bf16 bits, tokens `sel`)
    against the CPU oracle on the same inputs."""
    from oracle import oracle as O
    ref = O.fused_moe(hd["x"], hd["w1"], hd["w2"], hd["topk_ids"], hd["topk_w"], c["quant"], hd["w1_scale"],
                      hd["w2_scale"], sel=sel, partial_bf16=partial_bf16)
    gf, rf = O.bf16_to_f32(got_rows), O.bf16_to_f32(ref)
    return float(np.linalg.norm(gf - rf) / max(np.linalg.norm(rf), 1e-30))


def workload_config(c, gpus):
    return {"workload": c["label"], "tokens": c["T"], "hidden": c["H"], "intermediate": c["I"],
            "experts": c["E"], "topk": c["K"], "quant": QUANT_NAME[c["quant"]],
            "parallelism": "single" if gpus == 1 else f"ep{gpus}",
            "l2_policy": "weights (GBs) stream from HBM every step: inputs larger than L2, no flush"}


# ------------------------------------------------------------------------------ GPU arm

def device_inputs(c, dev, rank=0, world=1, seed=0):
    """Synthetic inputs generated on the device.  Weights are drawn per expert from a
    generator seeded by (seed, expert), so every rank of an expert-parallel run holds exactly
    the experts a single-GPU run would."""
    import torch
    T, H, I, E, K, quant = c["T"], c["H"], c["I"], c["E"], c["K"], c["quant"]
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=dev)
    ids, w = route_on_device(logits, K, c.get("routing", "softmax"))
    e_local = E // world
    w1s, w2s, s1s, s2s = [], [], [], []
    for e in range(rank * e_local, (rank + 1) * e_local):
        ge = torch.Generator(device=dev)
        ge.manual_seed(seed * 1000003 + 17 + e)
        for rows, cols, wl, sl in ((2 * I, H, w1s, s1s), (H, I, w2s, s2s)):
            q, sc = quantise_weight(torch.randn(rows, cols, generator=ge, device=dev) * 0.02, quant)
            wl.append(q)
            if sc is not None:
                sl.append(sc)
    w1, w2 = torch.stack(w1s), torch.stack(w2s)
    s1 = torch.stack(s1s).contiguous() if s1s else None
    s2 = torch.stack(s2s).contiguous() if s2s else None
    t_local = T // world
    sl = slice(rank * t_local, (rank + 1) * t_local)
    return dict(x=x[sl].contiguous(), ids=ids[sl].contiguous(), w=w[sl].contiguous(), w1=w1, w2=w2, s1=s1, s2=s2,
                x_full=x, ids_full=ids, w_full=w)


class Env:
    """Process-wide state of one benchmark run: rank, device, process group."""

    def __init__(self, a):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != a.gpus and self.world == 1 and a.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            if os.environ.get("NCCL_DEBUG", "").upper() not in ("INFO", "TRACE"):
                os.environ["NCCL_DEBUG"] = "WARN"
            os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # stdout carries only the JSON line
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        t = self.torch.tensor([v], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def timed_steps(env, fn, n):
    """Times exactly n calls of fn on the current stream: barrier + synchronize on both sides,
    CUDA events on the launching stream, maximum over ranks.  Also records an event after every
    step so the median and the minimum step are known.  Returns (total_ms, per_step_ms list,
    wall t0, wall t1)."""
    torch = env.torch
    env.barrier()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
    t0 = time.time()
    evs[0].record()
    for i in range(n):
        fn()
        evs[i + 1].record()
    env.barrier()
    t1 = time.time()
    total = env.max_over_ranks(evs[0].elapsed_time(evs[n]))
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(n)]
    return total, per, t0, t1


def roofline_entry(c, cfg_name, info, per, clocks, ms_total, ms_step, peaks, fp8_peak, resized):
    """Roofline of the dominant kernel (the gate+up GEMM) and of the whole step, from the stage
    times measured with events between the kernels.  Fractions are given against the measured
    peak of this pool and against the nominal figure, each labelled."""
    g1_ms = per["gemm1"]
    step_ms = ms_step                 # the timed loop's mean step (not the sum of the event-separated stages)
    fp8 = c["quant"] != 0
    kernel = info["gemm1_kernel_name"] + " (gate+up, SiLU*up epilogue)"
    tr = None if resized else GEMM1_DRAM_TRAFFIC.get(cfg_name)
    wbytes = c["E"] * 2 * c["I"] * c["H"] * (2 if c["quant"] == 0 else 1)
    if c["T"] <= 64:
        # decode: weight streaming bounds the step; report the gate+up GEMM against HBM
        achieved = wbytes / (g1_ms * 1e-3) / 1e9
        all_w = c["E"] * 3 * c["I"] * c["H"] * (2 if c["quant"] == 0 else 1)
        step_achieved = all_w / (step_ms * 1e-3) / 1e9
        r = {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
             "frac": achieved / peaks["hbm_gbs"], "peak_kind": peaks["source"] + " copy bandwidth",
             "frac_of_nominal": achieved / NOMINAL["hbm_gbs"],
             "step": {"achieved": step_achieved, "frac": step_achieved / peaks["hbm_gbs"],
                      "frac_of_nominal": step_achieved / NOMINAL["hbm_gbs"],
                      "what": "all weight bytes / mean step time of the timed loop"}}
    else:
        achieved = 4.0 * c["T"] * c["K"] * c["H"] * c["I"] / (g1_ms * 1e-3) / 1e12
        step_achieved = flops_per_step(c) / (step_ms * 1e-3) / 1e12
        # Denominator: the sustained figure when this loop ran in the regime it was measured in
        # (back-to-back launches under the power cap: sw_power_cap active and the median SM clock
        # well below the maximum, or a loop longer than a second), otherwise the burst figure.
        capped = bool(clocks and clocks.get("sm_mhz") and "sw_power_cap" in clocks.get("reasons", [])
                      and clocks["sm_mhz"] < 0.8 * clocks["sm_max_mhz"])
        sustained_regime = ms_total > 1000.0 or capped
        if fp8 and fp8_peak:
            burst, sust = fp8_peak["burst"], fp8_peak["sustained"]
            kind = "measured in this run: " + fp8_peak["how"]
        elif fp8:
            burst, sust = 2.0 * peaks["bf16_burst"], 2.0 * peaks["bf16_sustained"]
            kind = f"{peaks['source']} cuBLAS bf16 x2 (the fp8 peak could not be measured in this run)"
        else:
            burst, sust = peaks["bf16_burst"], peaks["bf16_sustained"]
            kind = f"{peaks['source']} cuBLAS bf16"
        peak = sust if sustained_regime else burst
        nominal = NOMINAL["fp8_tflops"] if fp8 else NOMINAL["bf16_tflops"]
        r = {"bound": "tensor", "kernel": kernel, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
             "frac": achieved / peak, "peak_kind": kind + (", sustained" if sustained_regime else ", burst"),
             "frac_of_burst": achieved / burst, "frac_of_sustained": achieved / sust,
             "frac_of_nominal": achieved / nominal,
             "step": {"achieved": step_achieved, "frac_of_burst": step_achieved / burst,
                      "frac_of_sustained": step_achieved / sust, "frac_of_nominal": step_achieved / nominal,
                      "what": "6*T*K*H*I / mean step time of the timed loop"}}
        if c["E"] >= 64:
            # fine-grained shape at the ridge: also the weight stream against HBM
            r["hbm"] = {"achieved": wbytes / (g1_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": wbytes / (g1_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                        "frac_of_nominal": wbytes / (g1_ms * 1e-3) / 1e9 / NOMINAL["hbm_gbs"]}
    r["ms_per_launch"] = g1_ms
    r["traffic"] = None if tr is None else tr["read"] + tr["write"]
    if tr is not None:
        r["traffic_source"] = f"{tr['source']}: {' / '.join(tr['quotes'])}" + (f" ({tr['scaled']})" if "scaled" in tr else "")
    r["gemm2_kernel"] = info["gemm2_kernel_name"]
    return r


def measure_single(env, a, c, cfg_name, headline, sampler):
    """One configuration on one GPU: device-resident timed loop, per-kernel stage times, roofline,
    parity spot check against the CPU oracle and the CPU baseline; for the headline also the
    end-to-end loop with host buffers."""
    import therock_b200 as M
    from therock_b200 import api
    torch, dev = env.torch, env.dev
    layout = a.weight_layout
    traits = M.FusedMoeTraits(prec_w="bf16" if c["quant"] == 0 else "fp8", quant=QUANT_NAME[c["quant"]],
                              weight_layout=layout, partial_dtype=a.partial_dtype, gemm_mode=a.gemm_mode)
    d = device_inputs(c, dev)
    if layout == "tiled128":          # offline pre-shuffle of the weights (not part of the timed step)
        from therock_b200 import weights as Wt
        d["w1_rowmajor"], d["w2_rowmajor"] = d["w1"], d["w2"]
        d["w1"], d["w2"] = Wt.tile_weights(d["w1"]), Wt.tile_weights(d["w2"])
    T, H = d["x"].shape
    args = M.FusedMoeArgs(a=d["x"], g=d["w1"], d=d["w2"], topk_ids=d["ids"], topk_weight=d["w"],
                          g_scale=d["s1"], d_scale=d["s2"])
    args.o = torch.empty_like(d["x"])
    args.workspace = torch.empty(M.fused_moe_workspace_size(traits, args), dtype=torch.uint8, device=dev)
    info = M.describe_run(traits, args)          # the kernels fmoe_run picks for these dimensions

    def step():
        return M.fused_moe(traits, args)

    steps = a.steps if headline else max(20, min(a.steps, 100))
    for _ in range(max(a.warmup, 3)):
        step()
    # Launch-bound steps (decode-sized batches) are replayed from a CUDA graph: the operator
    # neither synchronises nor allocates, so one capture of the step replaces its launches.
    use_graph = a.graph == "on" or (a.graph == "auto" and c["T"] <= 64)
    timed_step = step
    if use_graph:
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        cuda_graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            step()
            side.synchronize()
            with torch.cuda.graph(cuda_graph, stream=side):
                step()
        torch.cuda.synchronize()
        timed_step = cuda_graph.replay
        for _ in range(3):
            timed_step()
    ms_total, per_step, t0, t1 = timed_steps(env, timed_step, steps)
    clocks = sampler.summary(t0, t1) if sampler else None
    ms_step = ms_total / steps
    fl = flops_per_step(c)
    res = {"value": fl / ms_step / 1e9, "unit": "TFLOP/s", "ms_per_step": ms_step,
           "ms_per_step_median": float(np.median(per_step)), "ms_per_step_min": float(np.min(per_step)),
           "steps": steps, "tokens_per_s": c["T"] / (ms_step * 1e-3), "dtype": dtype_name(c),
           "config": workload_config(c, 1), "clocks": clocks, "gpu_launches": info["launches"] * steps,
           "kernels": {"gemm1": info["gemm1_kernel_name"], "gemm2": info["gemm2_kernel_name"],
                       "launches_per_step": info["launches"]}}
    res["config"]["launch"] = "cuda_graph_replay" if use_graph else "stream"
    res["config"]["weight_layout"] = layout
    res["config"]["partial_dtype"] = a.partial_dtype
    if a.kernel_only:
        return res, None

    # per-kernel durations over the same number of steps (events between the kernels)
    prof = api.StageProfile(steps)
    env.barrier()
    for _ in range(steps):
        prof.run(traits, args)
    stage = prof.read()
    prof.close()
    assert api.check_status(args.workspace) == 0
    runs = max(stage["runs"], 1)
    per = {k: stage[k] / runs for k in api.STAGES}
    res["stage_ms"] = per
    peaks = measured_peaks()
    fp8_peak = measure_fp8_peak(dev) if c["quant"] != 0 and c["T"] > 64 else None
    resized = a.tokens > 0 or a.experts > 0       # captured traffic belongs to the full-size workload
    res["roofline"] = roofline_entry(c, cfg_name, info, per, clocks, ms_total, ms_step, peaks, fp8_peak, resized)

    e2e = None
    if headline:
        # end to end: host buffers in, host buffer out, every step; the copies of neighbouring
        # steps overlap the compute (therock_b200.api.HostPipeline)
        x_h = d["x"].cpu().pin_memory()
        ids_h = d["ids"].cpu().pin_memory()
        w_h = d["w"].cpu().pin_memory()
        out_h = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
        outs = [torch.empty_like(d["x"]) for _ in range(2)]

        def pipe_step(x, ids, w, slot):
            args.a, args.topk_ids, args.topk_weight, args.o = x, ids, w, outs[slot]
            return M.fused_moe(traits, args, stream=torch.cuda.current_stream())
        # one CUDA-graph launch per step: operator on this batch, copy-in of the next batch and
        # copy-out of the previous result as concurrent branches (therock_b200.api.GraphPipeline)
        pipe = api.GraphPipeline(pipe_step, x_h, ids_h, w_h, out_h, dev)
        n_e2e = max(3, min(a.steps, 100))
        for _ in range(3):
            pipe.submit()
        pipe.flush()
        env.barrier()
        e0 = pipe.mark()
        for _ in range(n_e2e):
            pipe.submit()
        e1 = pipe.mark()
        pipe.flush()
        env.barrier()
        ms_e2e = e0.elapsed_time(e1)
        args.a, args.topk_ids, args.topk_weight, args.o = d["x"], d["ids"], d["w"], outs[0]
        e2e = {"value": fl / (ms_e2e / n_e2e) / 1e9, "unit": "TFLOP/s",
               "h2d_bytes_per_step": x_h.numel() * 2 + ids_h.numel() * 4 + w_h.numel() * 4,
               "d2h_bytes_per_step": out_h.numel() * 2, "ms_per_step": ms_e2e / n_e2e, "steps": n_e2e}

    # CPU baseline (the oracle on a bounded token sample of the same workload) and a parity spot
    # check of the benchmarked run against the same oracle
    from oracle import oracle as O
    O.build()
    hd = host_copy_of(d, c)
    n = cpu_sample_size(hd, c, budget_s=15.0 if headline else 6.0, n_calls=1)
    sel = np.random.default_rng(0).choice(c["T"], n, replace=False).astype(np.int32)
    t = cpu_time_tokens(hd, sel)
    res["cpu_baseline"] = {"value": 6.0 * n * c["K"] * c["H"] * c["I"] / t / 1e12, "unit": "TFLOP/s",
                           "cores": host_cores(), "kind": "port",
                           "sample": f"{n} of {c['T']} tokens, full weights, one pass ({t:.1f} s)"}
    # the parity tokens do not depend on the size of the timed CPU sample: the same eight every run
    n_par = min(8, c["T"])
    par_sel = np.sort(np.random.default_rng(1).choice(c["T"], n_par, replace=False)).astype(np.int32)
    got = step().view(torch.int16).cpu().numpy().view(np.uint16)[par_sel]
    res["parity_rel_l2"] = parity_sample(hd, c, got, par_sel, partial_bf16=(a.partial_dtype == "bf16"))
    res["parity_tokens"] = n_par
    del d, args, hd
    torch.cuda.empty_cache()
    return res, e2e


def measure_ep(env, a, c, sampler):
    """The configuration split expert-parallel over env.world GPUs of one node: tokens
    data-parallel, experts sharded, dispatch and return around the local operator."""
    import therock_b200 as M
    from therock_b200 import api, ep
    torch, dist, dev, world, rank = env.torch, env.dist, env.dev, env.world, env.rank
    if c["E"] % world or c["T"] % world:
        raise SystemExit("experts and tokens must divide over the ranks")
    traits = M.FusedMoeTraits(prec_w="bf16" if c["quant"] == 0 else "fp8", quant=QUANT_NAME[c["quant"]],
                              weight_layout=a.weight_layout)
    d = device_inputs(c, dev, rank, world)
    T_local, H = d["x"].shape
    # Transport: peer-memory kernels (no host sync) unless FMOE_EP_MODE=nccl or the peer buffers
    # cannot be set up, in which case NCCL all-to-all collectives are used.
    ep_transport = "nccl_all_to_all"
    moe = None
    if os.environ.get("FMOE_EP_MODE", "peer") != "nccl":
        try:
            moe = ep.PeerExpertParallelMoE(c["E"], world, rank, traits, d["w1"], d["w2"], d["s1"], d["s2"],
                                           tokens_per_rank=T_local, topk=c["K"], hidden=H, fused=a.ep_fused == "on",
                                           fp8_wire=a.ep_fp8_wire == "on",
                                           dedup=None if a.ep_dedup == "auto" else a.ep_dedup == "on")
            ep_transport = "peer_memory"
        except Exception as exc:  # noqa: BLE001
            if rank == 0:
                print(f"peer-memory expert parallelism unavailable ({exc!r}); using NCCL", file=sys.stderr)
    ok = torch.tensor([1 if ep_transport == "peer_memory" else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0:
        ep_transport = "nccl_all_to_all"
        local = ep.make_local_moe(traits, d["w1"], d["w2"], d["s1"], d["s2"])
        moe = ep.ExpertParallelMoE(c["E"], world, rank, local)
        launches_per_step = 8 + 2     # operator kernels + pack and combine kernels
    else:
        launches_per_step = moe.launches_per_step

    def step():
        return moe.forward(d["x"], d["ids"], d["w"])

    for _ in range(max(a.warmup, 3)):
        step()
    ms_total, per_step, t0, t1 = timed_steps(env, step, a.steps)
    clocks = sampler.summary(t0, t1) if sampler else None
    ms_step = ms_total / a.steps
    fl = flops_per_step(c)
    res = {"value": fl / ms_step / 1e9, "unit": "TFLOP/s", "ms_per_step": ms_step,
           "ms_per_step_median": float(np.median(per_step)), "ms_per_step_min": float(np.min(per_step)),
           "steps": a.steps, "tokens_per_s": c["T"] / (ms_step * 1e-3), "dtype": dtype_name(c),
           "config": workload_config(c, world), "clocks": clocks, "gpu_launches": launches_per_step * a.steps}
    res["config"]["launch"] = "stream"
    res["config"]["weight_layout"] = a.weight_layout
    res["config"]["ep_transport"] = ep_transport
    res["config"]["ep_step"] = "fused kernels" if getattr(moe, "fused", False) else "single-purpose kernels"
    res["config"]["ep_wire"] = "e4m3 rows + scales" if getattr(moe, "fp8_wire", False) else "bf16 rows"
    res["config"]["ep_rows"] = "one per (token, owner rank)" if getattr(moe, "dedup", False) else "one per (token, expert)"
    if a.kernel_only:
        return res, None

    # phases of the step (events around plan / dispatch / local operator / return / combine of a
    # few extra steps, this rank only)
    env.barrier()
    moe.trace = []
    n_tr = 10
    for _ in range(n_tr):
        step()
    torch.cuda.synchronize()
    tr, moe.trace = moe.trace, None
    ep_stage = {}
    for (n0, e0_), (n1, e1_) in zip(tr[:-1], tr[1:]):
        if n1 != "start":
            ep_stage[n1] = ep_stage.get(n1, 0.0) + e0_.elapsed_time(e1_) / n_tr
    res["ep_stage_ms"] = ep_stage

    # end to end: host buffers in, host buffer out, every step
    x_h = d["x"].cpu().pin_memory()
    ids_h = d["ids"].cpu().pin_memory()
    w_h = d["w"].cpu().pin_memory()
    out_h = torch.empty(T_local, H, dtype=torch.bfloat16).pin_memory()
    if ep_transport == "peer_memory" and a.e2e_pipeline == "graph":
        # the whole expert-parallel step has no host synchronisation inside, so it is captured,
        # with the copies of the neighbouring batches, in one graph per pipeline slot
        ep_out = [torch.empty_like(d["x"]) for _ in range(2)]

        def pipe_step(x, ids, w, slot):
            return moe.forward(x, ids, w, out=ep_out[slot])
        pipe = api.GraphPipeline(pipe_step, x_h, ids_h, w_h, out_h, dev)
        submit, finish = pipe.submit, pipe.flush
    elif ep_transport == "peer_memory":
        # three streams driven from the host; the step itself is one captured graph per slot
        ep_out = [torch.empty_like(d["x"]) for _ in range(2)]
        ep_graphs = [None, None]

        def pipe_step(x, ids, w, slot):
            if ep_graphs[slot] is None:
                moe.forward(x, ids, w, out=ep_out[slot])          # warm-up outside capture
                torch.cuda.current_stream().synchronize()
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=torch.cuda.current_stream()):
                    moe.forward(x, ids, w, out=ep_out[slot])
                ep_graphs[slot] = g_
            ep_graphs[slot].replay()
            return ep_out[slot]
        pipe = api.HostPipeline(pipe_step, T_local, H, c["K"], dev, depth=2)
        submit, finish = (lambda: pipe.submit(x_h, ids_h, w_h, out_h)), pipe.drain
    else:
        def pipe_step(x, ids, w, slot):
            return moe.forward(x, ids, w)
        pipe = api.HostPipeline(pipe_step, T_local, H, c["K"], dev, depth=2)
        submit, finish = (lambda: pipe.submit(x_h, ids_h, w_h, out_h)), pipe.drain
    n_e2e = max(3, min(a.steps, 100))
    for _ in range(3):
        submit()
    finish()
    env.barrier()
    e0 = pipe.mark()
    for _ in range(n_e2e):
        submit()
    e1 = pipe.mark()
    finish()
    env.barrier()
    ms_e2e = env.max_over_ranks(e0.elapsed_time(e1))
    e2e = {"value": fl / (ms_e2e / n_e2e) / 1e9, "unit": "TFLOP/s",
           "h2d_bytes_per_step": (x_h.numel() * 2 + ids_h.numel() * 4 + w_h.numel() * 4) * world,
           "d2h_bytes_per_step": out_h.numel() * 2 * world, "ms_per_step": ms_e2e / n_e2e, "steps": n_e2e}

    # Every rank's device status words (a bounded wait that ran out leaves a code there) and a
    # parity check of rank 0's own token slice against the CPU oracle.  Partial rows cross NVLink
    # as bf16, so the oracle runs in its bf16-partial mode.
    status = moe.check_status() if hasattr(moe, "check_status") else 0
    st = torch.tensor([status], device=dev, dtype=torch.int64)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    res["ep_status"] = int(st.item())
    out_now = step()
    torch.cuda.synchronize()
    env.barrier()
    if rank == 0:
        from oracle import oracle as O
        O.build()
        got_all = out_now.view(torch.int16).cpu().numpy().view(np.uint16)
        del moe
        full = device_inputs(c, dev, 0, 1)           # every expert's weights, as one GPU would hold them
        hd = host_copy_of(full, c)
        del full
        torch.cuda.empty_cache()
        sel = np.random.default_rng(0).choice(T_local, min(8, T_local), replace=False).astype(np.int32)
        res["parity_rel_l2"] = parity_sample(hd, c, got_all[sel], sel, partial_bf16=True)
        res["parity_tokens"] = int(len(sel))
        res["parity_what"] = "rank 0's token slice against the CPU oracle (bf16 partial rows)"
    env.barrier()
    return res, e2e


def run_gpu(a, c):
    import therock_b200 as M
    env = Env(a)
    M.lib()  # fails loudly when the CUDA library has not been built
    if a.scaling == "weak" and env.world > 1:
        c = dict(c)
        c["T"] *= env.world               # tokens per GPU fixed as N grows
        c["label"] += f"-weak{env.world}"
    sampler = ClockSampler(env.local_rank) if env.rank == 0 else None
    if env.world == 1:
        res, e2e = measure_single(env, a, c, a.config, True, sampler)
    else:
        res, e2e = measure_ep(env, a, c, sampler)
    line = {"metric": "fused_moe_tflops", "value": res.pop("value"), "unit": res.pop("unit"), "n_gpus": a.gpus,
            "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": res.pop("ms_per_step"),
            "higher_is_better": True, "scaling": a.scaling if env.world > 1 else "strong", "vs_baseline": None,
            "dtype": res.pop("dtype"), "data": "synthetic", "config": res.pop("config")}
    res.pop("steps", None)
    if e2e is not None:
        line["e2e"] = e2e
    line.update(res)
    # The other single-GPU configurations the targets are quoted on, measured in the same run
    # (fewer steps each) and attached to the one line.
    if env.world == 1 and a.per_config == "on" and a.config == "C1" and not a.kernel_only \
            and a.tokens == 0 and a.experts == 0:
        line["per_config"] = {}
        for name in ("C2", "C3", "C4", "C4m"):
            try:
                r, _ = measure_single(env, a, dict(CONFIGS[name]), name, False, sampler)
                line["per_config"][name] = r
            except Exception as exc:  # noqa: BLE001
                line["per_config"][name] = {"error": repr(exc)[:300]}
        if _FP8_PEAK:
            line["fp8_peak_tflops"] = _FP8_PEAK
    if sampler:
        sampler.stop()
    if env.rank == 0:
        print(json.dumps(line), flush=True)
    env.close()



def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="C1", choices=sorted(CONFIGS))
    ap.add_argument("--tokens", type=int, default=0,
                    help="override the token count (small cases for profiler captures)")
    ap.add_argument("--experts", type=int, default=0,
                    help="override the expert count (shrinks the weights for profiler captures)")
    ap.add_argument("--weight-layout", choices=["row_major", "tiled128"], default="row_major",
                    help="tiled128: weights pre-shuffled so every 128x128-byte operand tile is contiguous")
    ap.add_argument("--graph", choices=["auto", "on", "off"], default="auto",
                    help="replay the step from a CUDA graph in the timed loop (auto: decode-sized batches)")
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong",
                    help="N > 1: strong = the configuration's global batch is split over the GPUs; "
                         "weak = every GPU keeps the configuration's token count")
    ap.add_argument("--partial-dtype", choices=["f32", "bf16"], default="f32",
                    help="how the K weighted expert outputs are held before the ordered sum")
    ap.add_argument("--per-config", choices=["on", "off"], default="on",
                    help="single GPU, default workload: also measure C2, C3, C4 and attach them as per_config")
    ap.add_argument("--ep-fp8-wire", choices=["on", "off"], default="on",
                    help="N>1, fp8 configurations, fused step: token rows cross NVLink as e4m3 + scales (on) or bf16 (off)")
    ap.add_argument("--ep-dedup", choices=["auto", "on", "off"], default="auto",
                    help="N>1, fused step: one row per (token, owner rank) instead of per (token, expert); auto = from K >= 4")
    ap.add_argument("--ep-fused", choices=["on", "off"], default="on",
                    help="N > 1, peer memory: the fused step (send / recv_ready / wait_combine) or the single-purpose kernels")
    ap.add_argument("--gemm-mode", type=int, choices=[0, 1, 2], default=0,
                    help="0 = the library's per-GEMM choice, 1 = single-CTA kernel, 2 = CTA-pair kernel (profiling)")
    ap.add_argument("--e2e-pipeline", choices=["graph", "streams"], default="graph",
                    help="N > 1 end-to-end loop: one CUDA graph per step that also holds the copies, or three "
                         "streams driven from the host around a graph of the step")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the device-resident timed loop: no stage profile, e2e or CPU baseline")
    a = ap.parse_args()
    c = dict(CONFIGS[a.config])
    if a.tokens > 0:
        c["T"] = a.tokens
        c["label"] += f"-tokens{a.tokens}"
    if a.experts > 0:
        c["E"] = a.experts
        c["label"] += f"-experts{a.experts}"
    if a.impl == "reference":
        run_reference(a, c)
    else:
        run_gpu(a, c)


if __name__ == "__main__":
    main()

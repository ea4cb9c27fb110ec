"""Benchmark of the moe_fused_linear hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload gate_up|down]

One step = one pass of the hot path over one synthetic batch of the Qwen3-30B-A3B gate_up
shape: grouped-GEMM forward, input gradient (dX) and weight gradient (dW) for 65536
expanded rows (8192 tokens x top-8), hidden 2048 -> 1536, 128 experts, bf16 with fp32
accumulation.  `value` is the algorithmic TFLOP/s (2*M*N*K per GEMM, real rows only) of the
whole job with inputs resident in HBM; `e2e` is the same figure through the public Python
API with inputs in pinned host memory (router epilogue, sort, gather and the three GEMMs,
host->device and device->host copies inside the timed region).

`e2e` copies the step's results (y, dX and dW) back into pinned host
memory inside the timed region as well.

With N > 1 the 128 experts are sharded over the ranks (expert parallel); every rank routes
its own 8192 tokens and rows travel to the rank that owns their expert and results travel
back (weak scaling: per-GPU rows are fixed).  Default transport: rows are stored into the
owner's memory over NVLink by a copy kernel, and the forward / dX epilogues store their
results straight into the source rank's memory (`--ep-transport peer`); `--ep-transport
nccl` moves both directions by NCCL all-to-all instead.  By default a token of x crosses once
per destination rank and is expanded into its expert rows on the owner (`--ep-dispatch dedup`;
`rows` sends one row per token and expert).  After the timed loop one step's results are
checked against the single-GPU kernels (`ep_check` in the line).

At N = 1 the line also carries `extra_workloads`: the same measurement on the down_proj
shape with Zipf(1.2) routing (skewed, ragged and empty groups).

`--suite kernels` times the surrounding kernels (SiLU-mul, router, sort, gather / expand, combine,
NF4 decode and NF4-fused forward, fused-LoRA MLP, fused gate/up, block forward, the library
grouped GEMM as a yardstick), one JSON line each; `--suite block` the MoE block forward on N GPUs.
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

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT), str(ROOT / "transformers-qwen3-moe-fused_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np
import torch

WORKLOADS = {
    # name: (tokens, hidden(K), out(N), experts, top_k, routing)
    "gate_up": dict(tokens=8192, K=2048, N=1536, E=128, k=8, routing="softmax-top8 of N(0,1) logits"),
    "down": dict(tokens=8192, K=768, N=2048, E=128, k=8, routing="zipf(1.2) expert ids, 3 experts emptied"),
}
# DRAM bytes (ncu dram__bytes_read.sum + dram__bytes_write.sum) of one launch of each GEMM on a reduced
# case, with that case's algorithmic bytes, as recorded beside the ncu summaries.  Traffic grows in
# proportion to rows and experts, so the ratio carries over to the full workload.
NCU_TRAFFIC_FILE = ROOT / "profiles" / "grouped_gemm_dram_traffic.json"


def ncu_traffic_ratio(kernel: str):
    """(DRAM bytes / algorithmic bytes, description of the capture) or (None, reason)."""
    try:
        rec = json.loads(NCU_TRAFFIC_FILE.read_text())
        k = rec["kernels"][kernel]
        return float(k["dram_bytes"]) / float(k["algorithmic_bytes"]), rec["case"]
    except (OSError, KeyError, ValueError) as exc:
        return None, f"no ncu traffic record: {exc}"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def make_routing(cfg, seed: int):
    """Expert id per expanded row (tokens*k,), int64, on the CPU."""
    g = torch.Generator().manual_seed(seed)
    T, E, k = cfg["tokens"], cfg["E"], cfg["k"]
    if cfg["routing"].startswith("softmax"):
        logits = torch.randn(T, E, generator=g)
        return logits, None
    pmf = (torch.arange(E, dtype=torch.float64) + 1) ** -1.2
    ids = torch.multinomial(pmf / pmf.sum(), T * k, replacement=True, generator=g)
    for dead in (5, 64, 127):
        ids[ids == dead] = 0
    perm = torch.randperm(E, generator=g)
    return None, perm[ids]


class ClockSampler:
    """Samples SM clock, power and throttle reasons while a timed region runs: NVML every 10 ms from a
    thread of this process (read-only queries; a default run's timed region lasts 20-odd ms), or
    `nvidia-smi -lms 100` where NVML cannot be loaded."""

    PERIOD_S = 0.010

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []       # nvidia-smi rows
        self.samples = []    # NVML samples: (sm MHz, power W, reasons bit mask)
        self.proc = None
        self.nvml = None
        self.stop_flag = threading.Event()

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                return int(ids[self.index])
        return self.index

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                self.samples.append((float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)),
                                     n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0,
                                     int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))))
            except Exception:
                break
            time.sleep(self.PERIOD_S)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.nvml is not None:
            n = self.nvml
            self.stop_flag.set()
            self.thread.join(timeout=2)
            names = (("hw_slowdown", n.nvmlClocksThrottleReasonHwSlowdown),
                     ("hw_thermal_slowdown", n.nvmlClocksThrottleReasonHwThermalSlowdown),
                     ("sw_thermal_slowdown", n.nvmlClocksThrottleReasonSwThermalSlowdown),
                     ("sw_power_cap", n.nvmlClocksThrottleReasonSwPowerCap))
            reasons = sorted({name for _, _, mask in self.samples for name, bit in names if mask & bit})
            sm = [c for c, _, _ in self.samples]
            return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                    "sm_max_mhz": self.max_mhz, "power_w_max": max((p for _, p, _ in self.samples), default=None),
                    "reasons": reasons, "samples": len(sm), "source": f"nvml, {int(self.PERIOD_S * 1000)} ms period"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 3), ("hw_thermal_slowdown", 4), ("sw_thermal_slowdown", 5), ("sw_power_cap", 6)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvidia-smi, 100 ms period"}


def cpu_reference_arm(cfg, steps: int, warmup: int, sample_rows: int):
    """The reference's CPU implementation of the path (one torch mat-vec / outer product per
    row, qwen3_moe_fused/functional.py:7-61 of the reference) on all host threads, on a
    bounded sample of the workload's rows."""
    from oracle import cpu_baseline as C

    torch.set_num_threads(os.cpu_count() or 1)
    K, N, E = cfg["K"], cfg["N"], cfg["E"]
    g = torch.Generator().manual_seed(0)
    w = torch.randn(E, N, K, generator=g) * 0.02
    x = torch.randn(sample_rows, K, generator=g)
    dy = torch.randn(sample_rows, N, generator=g)
    experts = torch.sort(torch.randint(0, E, (sample_rows,), generator=g)).values
    flops = 3 * 2.0 * sample_rows * N * K

    def step():
        C.rowloop_fwd(x, w, experts)
        C.rowloop_bwd_input(dy, w, experts)
        C.rowloop_bwd_weight(dy, x, w, experts)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return flops / dt / 1e12, dt, torch.get_num_threads()


def _optional(fn, *args):
    """fn(*args), or None if it raises: for figures that must not cost the run its result line."""
    try:
        return fn(*args)
    except Exception as exc:  # noqa: BLE001
        print(f"[bench] {fn.__name__} failed: {exc}", file=sys.stderr)
        return None


def cpu_vectorised_arm(cfg, sample_rows: int):
    """The fairer CPU figure beside the reference's row loops: the same three results on the same kind of sample
    with one GEMM per expert over the sorted rows (stable sort + `x_e @ W_e.T`), all host threads.  TFLOP/s."""
    from oracle import cpu_baseline as C

    torch.set_num_threads(os.cpu_count() or 1)
    K, N, E = cfg["K"], cfg["N"], cfg["E"]
    g = torch.Generator().manual_seed(0)
    w = torch.randn(E, N, K, generator=g) * 0.02
    x = torch.randn(sample_rows, K, generator=g)
    dy = torch.randn(sample_rows, N, generator=g)
    experts = torch.sort(torch.randint(0, E, (sample_rows,), generator=g)).values
    m_sizes = torch.bincount(experts, minlength=E)

    def step():
        C.vectorised_fwd(x, w, m_sizes)
        C.vectorised_bwd_input(dy, w, m_sizes)
        C.vectorised_bwd_weight(dy, x, w, m_sizes)

    step()
    dt = C.time_call(step, repeats=2)
    return 3 * 2.0 * sample_rows * N * K / dt / 1e12


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = args.cpu_rows
    steps = max(1, min(args.steps, 2))
    warm = 1 if args.warmup > 0 else 0
    tf, dt, cores = cpu_reference_arm(cfg, steps, warm, rows)
    sample = f"{rows} of {cfg['tokens'] * cfg['k']} sorted rows, fp32, fwd+dX+dW row loops, {steps} timed step(s)"
    line = {
        "impl": "reference", "metric": "moe_fused_linear fwd+dX+dW algorithmic TFLOP/s", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args, cfg),
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def config_dict(args, cfg):
    return {"workload": f"Qwen3-30B-A3B {args.workload} grouped GEMM fwd+dX+dW: {cfg['tokens']} tokens x top-{cfg['k']} = "
                        f"{cfg['tokens'] * cfg['k']} rows/GPU, in={cfg['K']}, out={cfg['N']}, experts={cfg['E']}",
            "routing": cfg["routing"], "l2": "inputs larger than L2 (weights alone exceed 400 MB); no flush needed",
            "parallelism": "single GPU" if args.gpus == 1 else (
                f"expert parallel ep{args.gpus}, rows pushed over peer memory ({'x once per token and destination rank' if args.ep_dispatch == 'dedup' and args.ep_chunks == 1 else 'one row per token and expert'}), GEMM epilogues store to the source rank"
                if args.ep_transport == "peer" else f"expert parallel ep{args.gpus} (NCCL all-to-all dispatch/combine)")}


_TIME_OVERRIDE = {}  # {"iters": n, "warmup": m} for profiling runs (few launches per kernel)


def time_cuda(fn, iters: int = 20, warmup: int = 3, flush=None, inner: int = 1) -> float:
    """Median device time of fn() in ms (CUDA events around every call; an optional buffer larger
    than L2 is rewritten between calls so that small inputs are not served from cache).  Some
    device work is always queued ahead of the first event (the flush, else a short spin), so the
    host's launch latency of fn() is not counted as kernel time.  `inner` > 1 times that many
    back-to-back calls per sample (for kernels whose working set is several times L2), which
    amortises the event overhead of a few microseconds."""
    iters = _TIME_OVERRIDE.get("iters", iters)
    warmup = _TIME_OVERRIDE.get("warmup", warmup)
    inner = _TIME_OVERRIDE.get("inner", inner)
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if flush is not None:
            flush.add_(1)
        else:
            torch.cuda._sleep(200_000)  # ~0.1 ms of device time for the host to get ahead
        a.record()
        for _ in range(inner):
            fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b) / inner)
    return float(np.median(times))


def run_kernel_suite(args):
    """Roofline figures for the HBM-bound kernels of the path and for the NF4 / LoRA / block
    compositions.  One JSON line per measurement."""
    import __graft_entry__ as entry

    entry.build()
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.grouped_gemm.forward_4bit import grouped_gemm_forward_4bit
    from qwen3_moe_fused.kernels.fast_lora import fast_lora
    from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx
    from qwen3_moe_fused.kernels.routing import _combine, _expand_rows, _gather_rows, softmax_topk
    from qwen3_moe_fused.kernels.silu_mul import silu_mul_backward_inplace, silu_mul_forward
    from qwen3_moe_fused.moe_block import moe_block_forward
    from qwen3_moe_fused.quantize.nf4 import dequantize_4bit, quantize_nf4

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, kind = measured_peaks()
    hbm = peaks["hbm_gbs"]
    bf = torch.bfloat16
    flush = torch.zeros(64 * 1024 * 1024, device=dev, dtype=torch.float32)  # 256 MB
    torch.manual_seed(0)
    if args.kernel_iters:
        _TIME_OVERRIDE.update(iters=args.kernel_iters, warmup=1, inner=1)

    def emit(name, ms, nbytes=None, flops=None, **extra):
        line = {"suite": "kernels", "kernel": name, "ms": ms}
        if nbytes is not None:
            line.update(algorithmic_bytes=nbytes, gbs=nbytes / ms / 1e6, frac_of_hbm=nbytes / ms / 1e6 / hbm, hbm_peak_gbs=hbm, peak_kind=kind)
        if flops is not None:
            line.update(flops=flops, tflops=flops / ms / 1e9)
        line.update(extra)
        flag = _lib.read_error_flag()
        if flag:
            line["kernel_wait_error"] = {"code": flag >> 16, "cta": flag & 0xffff}
        print(json.dumps(line), flush=True)

    # ---- SiLU-mul at the down-projection input size ----
    n = 65536 * 768
    e, g, dh = (torch.randn(n, device=dev, dtype=bf) for _ in range(3))
    emit("silu_mul_fwd bf16 65536x768", time_cuda(lambda: silu_mul_forward(e, g), inner=5), 3 * 2 * n)
    emit("silu_mul_bwd_inplace bf16 65536x768", time_cuda(lambda: silu_mul_backward_inplace(dh, e, g), inner=5), 6 * 2 * n)
    del e, g, dh

    # ---- router ----
    for T in (8192, 16384, 1 << 20):
        logits = torch.randn(T, 128, device=dev)
        fl = flush if T < (1 << 20) else None
        emit(f"router softmax-top8 fp32 logits T={T}", time_cuda(lambda: softmax_topk(logits, 8, True, bf), flush=fl),
             4 * T * 128 + T * 8 * (8 + 2))
        del logits

    # ---- sort by expert ----
    for M in (65536, 131072, 1 << 24):
        s = torch.randint(0, 128, (M,), device=dev)
        fl = flush if M < (1 << 24) else None
        emit(f"sort_by_expert int64 ids M={M} E=128", time_cuda(lambda: get_expert_counts_and_idx(s, 128), flush=fl), M * (8 + 8))
        del s

    # ---- expand+gather and combine at the block size (16384 tokens, top-8, hidden 2048) ----
    T, k, H = 16384, 8, 2048
    hidden = torch.randn(T, H, device=dev, dtype=bf)
    sel = torch.randint(0, 128, (T * k,), device=dev)
    _, sort_idx, inv_sort_idx = get_expert_counts_and_idx(sel, 128)
    w = torch.rand(T, k, device=dev, dtype=bf)
    emit("gather_rows bf16 16384 tokens x8 x2048", time_cuda(lambda: _gather_rows(hidden, sort_idx, k), flush=flush), 2 * (T * H + T * k * H) + 4 * T * k)
    emit("expand_rows (same rows, token-major) bf16 16384 tokens x8 x2048", time_cuda(lambda: _expand_rows(hidden, inv_sort_idx, k), flush=flush),
         2 * (T * H + T * k * H) + 4 * T * k)
    y = torch.randn(T * k, H, device=dev, dtype=bf)
    emit("combine bf16 16384 tokens x8 x2048", time_cuda(lambda: _combine(y, inv_sort_idx, w), inner=5), 2 * (T * k * H + T * H) + 6 * T * k)
    del hidden, y

    # ---- NF4: decode alone, fused forward vs decode + GEMM (128 experts, 1536 x 2048, blocksize 64, three batch sizes) ----
    E, N, K = 128, 1536, 2048
    wfull = (torch.randn(E, N, K, device=dev) * 0.02).to(bf)
    packed, state = quantize_nf4(wfull, 64)
    del wfull
    nel = E * N * K
    emit("nf4_dequant 128x1536x2048 -> bf16", time_cuda(lambda: dequantize_4bit(packed, state, bf), inner=5), nel // 2 + nel // 64 * 4 + nel * 2)
    if args.hbm_only:
        assert _lib.read_error_flag() == 0
        return
    for tokens in (512, 4096, 32768):
        M = tokens * 8
        x = torch.randn(M, K, device=dev, dtype=bf)
        m_sizes = torch.full((E,), M // E, device=dev, dtype=torch.int32)
        flops = 2.0 * M * N * K
        fused = time_cuda(lambda: grouped_gemm_forward_4bit(x, packed, state, m_sizes, fused=True), iters=10)
        unfused = time_cuda(lambda: grouped_gemm_forward(x, dequantize_4bit(packed, state, bf), m_sizes), iters=10)
        auto = time_cuda(lambda: grouped_gemm_forward_4bit(x, packed, state, m_sizes), iters=10)
        wbytes = nel // 2 + nel // 64 * 4
        emit(f"nf4 fused forward M={M}", fused, wbytes + 2 * M * (K + N), flops, unfused_ms=unfused, speedup_vs_unfused=unfused / fused,
             public_api_ms=auto, public_api_note="grouped_gemm_forward_4bit picks decode-inside or decode-once by rows per expert")
        del x
    # ---- fused-LoRA expert MLP, rank 16, NF4 base, forward + backward ----
    I, Hh, R = 768, 2048, 16
    mk = lambda *shape, sc: (torch.randn(*shape, device=dev) * sc).to(bf)
    G, U, Wd = mk(E, I, Hh, sc=0.02), mk(E, I, Hh, sc=0.02), mk(E, Hh, I, sc=0.02)
    (Gq, Gs), (Uq, Us), (Wq, Ws) = (quantize_nf4(t, 64) for t in (G, U, Wd))
    del G, U, Wd
    lor = [mk(E, R, Hh, sc=0.02), mk(E, I, R, sc=0.01), mk(E, R, Hh, sc=0.02), mk(E, I, R, sc=0.01), mk(E, R, I, sc=0.02), mk(E, Hh, R, sc=0.01)]
    for t in lor:
        t.requires_grad_()
    for tokens in (512, 4096):
        M = tokens * 8
        x = torch.randn(M, Hh, device=dev, dtype=bf, requires_grad=True)
        m_sizes = torch.full((E,), M // E, device=dev, dtype=torch.int32)
        dy = torch.randn(M, Hh, device=dev, dtype=bf)

        def step():
            out = fast_lora(x, Gq, Gs, lor[0], lor[1], 1.0, Uq, Us, lor[2], lor[3], 1.0, Wq, Ws, lor[4], lor[5], 1.0, m_sizes)
            out.backward(dy)

        emit(f"fast_lora NF4 base r=16 fwd+bwd M={M}", time_cuda(step, iters=5, warmup=2), flops=3 * 3 * 2.0 * M * I * Hh)
        del x, dy
    del packed, state, Gq, Uq, Wq, lor

    # ---- library comparison: torch's own grouped GEMM (a CUTLASS library kernel) on the gate_up forward ----
    M, N, K = 65536, 1536, 2048
    x = torch.randn(M, K, device=dev, dtype=bf)
    wg = mk(E, N, K, sc=0.02)
    m_sizes = torch.full((E,), M // E, device=dev, dtype=torch.int32)
    ours = time_cuda(lambda: grouped_gemm_forward(x, wg, m_sizes), iters=20)
    try:
        offs = torch.cumsum(m_sizes, 0).to(torch.int32)
        wt = wg.transpose(1, 2)
        lib_ms = time_cuda(lambda: torch._grouped_mm(x, wt, offs=offs), iters=20)
        emit("gate_up forward vs torch._grouped_mm (library)", ours, flops=2.0 * M * N * K, library_ms=lib_ms,
             library_tflops=2.0 * M * N * K / lib_ms / 1e9, speedup_vs_library=lib_ms / ours)
    except Exception as exc:  # the library op is optional: report why it is missing
        emit("gate_up forward vs torch._grouped_mm (library)", ours, flops=2.0 * M * N * K, library="unavailable: " + str(exc)[:120])
    del x, wg

    # ---- gate + up + SiLU-mul in one kernel against the three kernels it stands for (block size) ----
    from qwen3_moe_fused.kernels.fused_mlp import gate_up_silu_forward

    M, I_, K = 131072, 768, 2048
    x = torch.randn(M, K, device=dev, dtype=bf)
    wg, wu = mk(E, I_, K, sc=0.02), mk(E, I_, K, sc=0.02)
    m_sizes = torch.full((E,), M // E, device=dev, dtype=torch.int32)
    fused_ms = time_cuda(lambda: gate_up_silu_forward(x, wg, wu, m_sizes), iters=10)
    three_ms = time_cuda(lambda: silu_mul_forward(grouped_gemm_forward(x, wg, m_sizes), grouped_gemm_forward(x, wu, m_sizes)), iters=10)
    emit("gate_up_silu fused forward, 131072 rows, 2048 -> 768 x 2", fused_ms, flops=2 * 2.0 * M * I_ * K, three_kernels_ms=three_ms,
         speedup_vs_three_kernels=three_ms / fused_ms)
    del x, wg, wu

    # ---- one full MoE block forward at the block workload (16384 tokens) ----
    T = 16384
    hidden = torch.randn(1, T, 2048, device=dev, dtype=bf)
    gate = mk(128, 2048, sc=0.02)
    gp, up, dp = mk(128, 768, 2048, sc=0.02), mk(128, 768, 2048, sc=0.02), mk(128, 2048, 768, sc=0.02)
    with torch.no_grad():
        ms = time_cuda(lambda: moe_block_forward(hidden, gate, gp, up, dp, 8, True), iters=10)
    emit("moe block forward, 16384 tokens, 128 experts top-8", ms, flops=2.0 * T * 2048 * 128 + 3 * 2.0 * T * 8 * 768 * 2048,
         tokens_per_s=T / ms * 1e3, tokens_per_s_48_layers=T / ms * 1e3 / 48)
    assert _lib.read_error_flag() == 0


def run_block_suite(args):
    """Forward of one sparse MoE block over 16384 tokens in total (strong scaling: 16384 / N tokens and
    128 / N experts per rank), tokens/s over all ranks.  N = 1: `moe_block_forward`; N > 1: `PeerMoeBlock`."""
    import __graft_entry__ as entry

    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    if rank == 0:
        entry.build()
    if world > 1:
        dist.barrier()
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.moe_block import moe_block_forward

    H, I, E, k = 2048, 768, 128, 8
    weak = args.block_tokens_per_gpu is not None
    T_total = args.block_tokens_per_gpu * world if weak else 16384
    T, e_local = T_total // world, E // world
    bf = torch.bfloat16
    g0 = torch.Generator().manual_seed(5)
    gate_w = (torch.randn(E, H, generator=g0) * 0.02).to(bf).to(dev)
    g1 = torch.Generator().manual_seed(50 + rank)
    mk = lambda *shape: (torch.randn(*shape, generator=g1) * 0.02).to(bf).to(dev)
    gp, up, dp = mk(e_local, I, H), mk(e_local, I, H), mk(e_local, H, I)
    hidden = torch.randn(T, H, generator=g1).to(bf).to(dev)
    if world == 1:
        def fn():
            with torch.no_grad():
                moe_block_forward(hidden.view(1, T, H), gate_w, gp, up, dp, k, True)
    else:
        from qwen3_moe_fused.parallel_ep import PeerMoeBlock

        block = PeerMoeBlock(world, rank, dev, H, T * k, bf, capacity_factor=2.0, max_tokens=T if args.ep_dispatch == "dedup" else None)
        block.forward(hidden, gate_w, gp, up, dp, k, True, check_capacity=True)

        def fn():
            block.forward(hidden, gate_w, gp, up, dp, k, True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)
    err = _lib.read_error_flag()
    if rank == 0:
        flops = 2.0 * T_total * H * E + 3 * 2.0 * T_total * k * I * H
        print(json.dumps({"suite": "block", "what": f"MoE block forward, {T_total} tokens in total, 128 experts, top-8, bf16",
                          "n_gpus": world, "scaling": "weak" if weak else "strong", "steps": args.steps, "ms": ms,
                          "tokens_per_s": T_total / ms * 1e3, "tokens_per_s_48_layers": T_total / ms * 1e3 / 48,
                          "tflops": flops / ms / 1e9, "kernel_wait_errors": err,
                          "transport": "single GPU" if world == 1 else "peer memory (tokens pushed once per destination rank + row indices, "
                                       "down-projection epilogue stores to the token's rank)"}),
              flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure_single_gpu_workload(name: str, steps: int, warmup: int, dev):
    """fwd + dX + dW of one workload on one GPU, inputs resident: per-kernel CUDA-event times inside a
    back-to-back loop and launched alone.  Used for the `extra_workloads` entry of the line."""
    from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.grouped_gemm.forward_transposed import grouped_gemm_forward_transposed
    from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx
    from qwen3_moe_fused.kernels.routing import softmax_topk

    cfg = dict(WORKLOADS[name])
    T, K, N, E, k = cfg["tokens"], cfg["K"], cfg["N"], cfg["E"], cfg["k"]
    M = T * k
    bf = torch.bfloat16
    logits_h, ids_h = make_routing(cfg, seed=0)
    if logits_h is not None:
        ids_d = softmax_topk(logits_h.to(dev), k, True, bf)[1].view(-1)
    else:
        ids_d = ids_h.to(dev)
    m_sizes, _, _ = get_expert_counts_and_idx(ids_d, E)
    gen = torch.Generator(device=dev).manual_seed(4321)
    x = torch.randn(M, K, generator=gen, device=dev).to(bf)
    dy = torch.randn(M, N, generator=gen, device=dev).to(bf)
    w = (torch.randn(E, N, K, generator=gen, device=dev) * 0.02).to(bf)
    fns = {"fwd": lambda: grouped_gemm_forward(x, w, m_sizes), "dx": lambda: grouped_gemm_forward_transposed(dy, w, m_sizes),
           "dw": lambda: grouped_gemm_backward_dw(x, dy, m_sizes, bf)}
    for _ in range(max(warmup, 3)):
        for fn in fns.values():
            fn()
    torch.cuda.synchronize()
    marks = []
    for _ in range(steps):
        row = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        row[0].record()
        for i, fn in enumerate(fns.values()):
            fn()
            row[i + 1].record()
        marks.append(row)
    torch.cuda.synchronize()
    step_ms = marks[0][0].elapsed_time(marks[-1][3]) / steps
    flops_one = 2.0 * M * N * K
    peaks, _ = measured_peaks()
    out = {"workload": config_dict(argparse.Namespace(workload=name, gpus=1, ep_transport="peer"), cfg)["workload"],
           "routing": cfg["routing"], "rows_per_expert": {"max": int(m_sizes.max()), "empty_experts": int((m_sizes == 0).sum())},
           "steps": steps, "ms_per_step": step_ms, "value": 3 * flops_one / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "kernels": {}}
    for i, kname in enumerate(fns):
        ms = float(np.mean([r[i].elapsed_time(r[i + 1]) for r in marks]))
        alone = time_cuda(fns[kname], iters=20)
        out["kernels"][kname] = {"ms": ms, "tflops": flops_one / (ms * 1e-3) / 1e12, "isolated_ms": alone,
                                 "isolated_tflops": flops_one / (alone * 1e-3) / 1e12,
                                 "isolated_frac_of_burst_peak": flops_one / (alone * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="gate_up", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-rows", type=int, default=4096, help="rows of the bounded CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra_workloads entry (down_proj shape, Zipf routing)")
    ap.add_argument("--suite", default="hotpath", choices=["hotpath", "kernels", "block"],
                    help="hotpath: the contract line (default); kernels: roofline lines of the surrounding kernels; "
                         "block: MoE block forward, 16384 tokens over N GPUs")
    ap.add_argument("--hbm-only", action="store_true", help="kernel suite: only the HBM-bound kernels (profiling runs)")
    ap.add_argument("--kernel-iters", type=int, default=None, help="kernel suite: timed launches per kernel (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--tokens", type=int, default=None, help="override tokens per GPU (reduced profiling case)")
    ap.add_argument("--experts", type=int, default=None, help="override the expert count (reduced profiling case)")
    ap.add_argument("--only", default=None, choices=["fwd", "dx", "dw"], help="run one of the three GEMMs per step")
    ap.add_argument("--ep-transport", default="peer", choices=["peer", "nccl"],
                    help="N > 1: rows move by peer-memory stores fused with the GEMM epilogue (default) or by NCCL all-to-all")
    ap.add_argument("--block-tokens-per-gpu", type=int, default=None,
                    help="block suite: tokens per GPU (weak scaling) instead of 16384 tokens in total")
    ap.add_argument("--push-ctas", type=int, default=0,
                    help="N > 1, peer transport: CTAs of the row push that overlaps a GEMM (0: four per SM)")
    ap.add_argument("--ep-overlap", default="on", choices=["on", "off"],
                    help="N > 1, peer transport: run the second row push beside the first GEMM (on) or before it (off)")
    ap.add_argument("--ep-dispatch", default="dedup", choices=["dedup", "rows"],
                    help="N > 1, peer transport: x travels once per (token, destination rank) and is expanded by the owner "
                         "(dedup, default) or once per (token, expert) (rows)")
    ap.add_argument("--ep-chunks", type=int, default=1,
                    help="N > 1, peer transport: chunks of local experts whose exchange and GEMMs are pipelined")
    ap.add_argument("--gemm-path", default="auto", choices=["auto", "tc", "tc_single", "simt"],
                    help="kernel family for the grouped GEMMs (default: CTA-pair tcgen05 where eligible)")
    ap.add_argument("--watchdog-s", type=int, default=600,
                    help="dump every thread's stack and exit if the run has not finished after this many seconds (0: off)")
    args = ap.parse_args()
    if args.watchdog_s > 0:
        import faulthandler

        faulthandler.dump_traceback_later(args.watchdog_s, exit=True)
    cfg = dict(WORKLOADS[args.workload])
    if args.tokens:
        cfg["tokens"] = args.tokens
    if args.experts:
        cfg["E"] = args.experts
    if args.impl == "reference":
        run_reference(args, cfg)
        return
    if args.suite == "kernels":
        run_kernel_suite(args)
        return
    if args.suite == "block":
        run_block_suite(args)
        return

    import __graft_entry__ as entry

    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # peer buffers are addressed directly, never through multicast
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    if rank == 0:
        entry.build()
    if world > 1:
        dist.barrier()

    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.grouped_gemm.forward_transposed import grouped_gemm_forward_transposed
    from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx
    from qwen3_moe_fused.kernels.routing import _expand_rows, softmax_topk

    _lib.load()
    _lib.set_gemm_path({"auto": _lib.PATH_AUTO, "tc": _lib.PATH_TC, "tc_single": _lib.PATH_TC_SINGLE, "simt": _lib.PATH_SIMT}[args.gemm_path])
    T, K, N, E, k = cfg["tokens"], cfg["K"], cfg["N"], cfg["E"], cfg["k"]
    M = T * k
    E_local = E // world
    gen = torch.Generator().manual_seed(1234 + rank)
    bf = torch.bfloat16

    # ---- synthetic inputs (host, pinned) ----
    logits_h, ids_h = make_routing(cfg, seed=rank)
    hidden_h = torch.randn(T, K, generator=gen).to(bf).pin_memory()
    dy_h = torch.randn(M, N, generator=gen).to(bf).pin_memory()
    if logits_h is not None:
        logits_h = logits_h.pin_memory()
    else:
        ids_h = ids_h.pin_memory()
    w = (torch.randn(E_local, N, K, generator=torch.Generator().manual_seed(99 + rank)) * 0.02).to(bf).to(dev)

    if world > 1:
        from qwen3_moe_fused.parallel_ep import ExpertParallelPlan

    def route(logits_d, ids_d):
        """(T * k,) expert id of every expanded row, token-major."""
        if logits_d is not None:
            return softmax_topk(logits_d, k, True, bf)[1].view(-1)
        return ids_d

    def route_and_sort(logits_d, ids_d):
        return get_expert_counts_and_idx(route(logits_d, ids_d), E)

    # ---- resident inputs for the kernel-only measurement ----
    logits_d = logits_h.to(dev) if logits_h is not None else None
    ids_d = ids_h.to(dev) if ids_h is not None else None
    hidden_d = hidden_h.to(dev)
    dy_d = dy_h.to(dev)
    m_sizes, sort_idx, inv_sort_idx = route_and_sort(logits_d, ids_d)
    x_d = _expand_rows(hidden_d, inv_sort_idx, k)  # rows in expert order, every token row read once
    plan = None
    peer = None
    if world > 1 and args.ep_transport == "nccl":
        plan = ExpertParallelPlan.build(m_sizes, world, rank, dev)
    elif world > 1:
        from qwen3_moe_fused.parallel_ep import PeerChannel, PeerPlan, peer_fence, peer_grouped_gemm, peer_push

        # The local experts are split into chunks with a plan and a buffer region each, so that the
        # exchange of one chunk overlaps the GEMMs of another.  Receive buffers hold up to twice the
        # even share of rows; results return into buffers of M rows.
        n_chunks = max(1, min(args.ep_chunks, E_local))
        bounds = [E_local * i // n_chunks for i in range(n_chunks + 1)]
        counts_all = PeerPlan.gather_counts(m_sizes, world)
        cap = 2 * M
        region = cap // n_chunks // 8 * 8
        ch_x, ch_dy = PeerChannel(cap, K, bf, dev), PeerChannel(cap, N, bf, dev)
        peer = {"plans": [PeerPlan.from_counts(counts_all, world, rank, (bounds[i], bounds[i + 1])) for i in range(n_chunks)],
                "x": [ch_x.rows(i * region, region) for i in range(n_chunks)],
                "dy": [ch_dy.rows(i * region, region) for i in range(n_chunks)],
                "w": [w[bounds[i]:bounds[i + 1]] for i in range(n_chunks)],
                "y": PeerChannel(M, N, bf, dev), "dx": PeerChannel(M, K, bf, dev),
                "x_all": ch_x, "dy_all": ch_dy, "token": torch.zeros(1, device=dev), "n": n_chunks}
        assert all(int(pl.recv_rows) <= region for pl in peer["plans"]), "receive buffer too small for this routing"
        dedup = args.ep_dispatch == "dedup" and n_chunks == 1
        if dedup:
            # x travels as token rows, once per destination rank, plus a 4-byte index per expanded row;
            # the owner expands its rows locally into the buffer the GEMMs read
            from qwen3_moe_fused.parallel_ep import (expand_received, gather_counts_and_tokens, peer_push_index, peer_push_tokens,
                                                     slot_bases, token_positions)

            pos, n_tok = token_positions(route(logits_d, ids_d).view(T, k), E, world)
            _, tokens_all = gather_counts_and_tokens(m_sizes, n_tok, world)
            peer.update(pos=pos, base=slot_bases(tokens_all, rank), tok=PeerChannel(world * T, K, bf, dev),
                        idx=PeerChannel(cap, 1, torch.int32, dev), sort_idx=sort_idx,
                        tokens_out=int(tokens_all[rank].sum() - tokens_all[rank, rank]))
        peer["dedup"] = dedup
        peer_fence(peer["token"])
    torch.cuda.synchronize()

    comm_stream = torch.cuda.Stream(device=dev) if world > 1 else None
    ev = lambda: torch.cuda.Event(enable_timing=True)
    kernel_ms = {"fwd": [], "dx": [], "dw": []}
    # three GEMMs, each preceded by the kernel that builds its per-expert tensor maps; per step at
    # N > 1 also two row pushes (peer) or four row permutations (nccl)
    nck = max(1, min(args.ep_chunks, E_local))
    launches_per_step = 6 if world == 1 else (8 * nck + (2 if peer["dedup"] else 0) if args.ep_transport == "peer" else 10)

    def step_resident(record: bool):
        if world == 1:
            marks = [ev() for _ in range(4)]
            y = dx = dw = None
            marks[0].record()
            if args.only in (None, "fwd"):
                y = grouped_gemm_forward(x_d, w, m_sizes)
            marks[1].record()
            if args.only in (None, "dx"):
                dx = grouped_gemm_forward_transposed(dy_d, w, m_sizes)
            marks[2].record()
            if args.only in (None, "dw"):
                dw = grouped_gemm_backward_dw(x_d, dy_d, m_sizes, bf)
            marks[3].record()
            return marks if record else None, (y, dx, dw)
        if peer is not None:
            # expert parallel over peer memory: rows are pushed to their experts' ranks by copy kernels,
            # the forward and dX epilogues store their results straight into the source ranks' memory; a
            # one-element all-reduce orders each phase across the ranks.
            #   comm:    push dY | fence | x: tokens + indices | fence | expand
            #   compute:                 | dX                          | forward | dW | fence
            # dY goes first and is exposed; x (token rows once per destination rank: a third to a quarter of
            # the bytes of one row per (token, expert)) travels beside the dX GEMM.  Measured alternatives at
            # 2 GPUs: x first and the push of dY beside the forward GEMM is slower (1.65 against 1.51 ms: both
            # send over NVLink and the GEMM's remote stores queue behind the push, whatever the push's CTA
            # count); per chunk of local experts (--ep-chunks > 1) is slower too (fences and launches).
            marks = [ev() for _ in range(4)]
            main = torch.cuda.current_stream()
            nc = peer["n"]
            e_x = [torch.cuda.Event() for _ in range(nc)]
            e_dy = [torch.cuda.Event() for _ in range(nc)]
            push_stream = comm_stream if args.ep_overlap == "on" else main
            comm_stream.wait_stream(main)

            def run_forward():
                for i in range(nc):
                    main.wait_event(e_x[i])
                    peer_grouped_gemm(peer["plans"][i], peer["x"][i], peer["w"][i], peer["y"])

            def run_dx():
                for i in range(nc):
                    main.wait_event(e_dy[i])
                    peer_grouped_gemm(peer["plans"][i], peer["dy"][i], peer["w"][i], peer["dx"], transposed=True)

            def push(rows, chans, events, ctas):
                for i in range(nc):
                    peer_push(peer["plans"][i], rows, chans[i], ctas)
                    peer_fence(peer["token"])
                    events[i].record()

            with torch.cuda.stream(push_stream):
                push(dy_d, peer["dy"], e_dy, 0)
                if peer["dedup"]:
                    peer_push_tokens(hidden_d, peer["pos"], peer["base"], peer["tok"], rank, max_ctas=args.push_ctas)
                    peer_push_index(peer["plans"][0], peer["pos"], peer["base"], peer["sort_idx"], k, peer["idx"])
                    peer_fence(peer["token"])
                    expand_received(peer["tok"].local, peer["idx"].local.view(-1), peer["plans"][0].recv_rows, peer["x"][0].local)
                    e_x[0].record()
                else:
                    push(x_d, peer["x"], e_x, args.push_ctas)     # beside the dX GEMM
            main.wait_event(e_dy[0])
            marks[0].record()   # marks 0-1: dX, 1-2: forward (including its wait for x), 2-3: dW
            run_dx()
            marks[1].record()
            run_forward()
            marks[2].record()
            dw = [grouped_gemm_backward_dw(peer["x"][i].local, peer["dy"][i].local, peer["plans"][i].local_m_sizes, bf)
                  for i in range(nc)]
            marks[3].record()
            peer_fence(peer["token"])  # results of every rank have arrived; buffers may be reused
            return marks if record else None, (peer["y"].local, peer["dx"].local, dw[0])
        # expert parallel: rows to their experts, compute, results back.  The all-to-alls and
        # their permutation passes run on a second stream so that they overlap the GEMMs:
        #   comm:    dispatch x | dispatch dy |            combine y |           combine dx
        #   compute:            | forward     | dX         | dW
        marks = [ev() for _ in range(4)]
        main = torch.cuda.current_stream()
        e_x, e_dy, e_y, e_dx, e_done = (torch.cuda.Event() for _ in range(5))
        comm_stream.wait_stream(main)
        with torch.cuda.stream(comm_stream):
            xl = plan.dispatch(x_d)
            e_x.record()
            dyl = plan.dispatch(dy_d)
            e_dy.record()
        main.wait_event(e_x)
        marks[0].record()
        y = plan.grouped(grouped_gemm_forward, xl, w)
        marks[1].record()
        e_y.record()
        with torch.cuda.stream(comm_stream):
            comm_stream.wait_event(e_y)
            y_back = plan.combine(y)
        main.wait_event(e_dy)
        dx = plan.grouped(grouped_gemm_forward_transposed, dyl, w)
        marks[2].record()
        e_dx.record()
        with torch.cuda.stream(comm_stream):
            comm_stream.wait_event(e_dx)
            dx_back = plan.combine(dx)
            e_done.record()
        dw = plan.grouped_dw(grouped_gemm_backward_dw, xl, dyl, bf, E_local)
        marks[3].record()
        main.wait_event(e_done)
        return marks if record else None, (y_back, dx_back, dw)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    n_warm = args.warmup if (args.no_e2e and args.only) else max(args.warmup, 3)
    for _ in range(n_warm):
        step_resident(False)
    # the sampler starts before the barrier: its set-up takes milliseconds on rank 0 alone, which the other
    # ranks would otherwise spend inside their timed region waiting for rank 0's first fence
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    t_start, t_end = ev(), ev()
    all_marks = []
    t_start.record()
    host_t0 = time.perf_counter()
    for _ in range(args.steps):
        marks, _ = step_resident(True)
        all_marks.append(marks)
    host_issue_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps  # host time to enqueue a step
    t_end.record()
    barrier()
    resident_ms = t_start.elapsed_time(t_end) / args.steps
    # device time between the last GEMM of a step and the first GEMM of the next (exchange, fences, idle)
    gaps = [all_marks[i][3].elapsed_time(all_marks[i + 1][0]) for i in range(len(all_marks) - 1)]
    clocks = sampler.stop() if rank == 0 else None  # samples of the resident loop only
    first, second = ("dx", "fwd") if peer is not None else ("fwd", "dx")  # the peer schedule runs dX first
    for marks in all_marks:
        kernel_ms[first].append(marks[0].elapsed_time(marks[1]))
        kernel_ms[second].append(marks[1].elapsed_time(marks[2]))
        kernel_ms["dw"].append(marks[2].elapsed_time(marks[3]))

    # ---- end to end through the public API, inputs in pinned host memory ----
    h2d = hidden_h.numel() * 2 + dy_h.numel() * 2 + (logits_h.numel() * 4 if logits_h is not None else ids_h.numel() * 8)
    # results of a step: y (M, N), dX (M, K), dW (E_local, N, K), all bf16, plus m_sizes
    d2h = 2 * (M * N + M * K + E_local * N * K) + E * 4

    # Inputs are double-buffered on the device: the upload of step i+1 (copy stream) runs beside the
    # compute of step i.  Every step's inputs still cross PCIe inside the timed region.
    copy_stream = torch.cuda.Stream(device=dev)
    back_stream = torch.cuda.Stream(device=dev)  # results -> pinned host memory, beside the next step's compute
    slots = [{"hd": torch.empty_like(hidden_d), "dyd": torch.empty_like(dy_d),
              "lg": torch.empty_like(logits_d) if logits_d is not None else None,
              "idd": torch.empty_like(ids_d) if ids_d is not None else None,
              "ready": torch.cuda.Event(), "free": torch.cuda.Event()} for _ in range(2)]
    back = [] if args.no_e2e else [
        {"y": torch.empty((M, N), dtype=bf).pin_memory(), "dx": torch.empty((M, K), dtype=bf).pin_memory(),
         "dw": torch.empty((E_local, N, K), dtype=bf).pin_memory(), "ms": torch.empty(E, dtype=torch.int32).pin_memory(),
         "done": torch.cuda.Event()} for _ in range(2)]

    def upload(slot):
        sl = slots[slot]
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(sl["free"])  # the step that last read this slot has finished
            sl["hd"].copy_(hidden_h, non_blocking=True)
            sl["dyd"].copy_(dy_h, non_blocking=True)
            if sl["lg"] is not None:
                sl["lg"].copy_(logits_h, non_blocking=True)
            else:
                sl["idd"].copy_(ids_h, non_blocking=True)
            sl["ready"].record()

    def step_e2e(i, last):
        sl = slots[i % 2]
        torch.cuda.current_stream().wait_event(sl["ready"])
        if not last:
            upload((i + 1) % 2)
        hd, dyd, lg, idd = sl["hd"], sl["dyd"], sl["lg"], sl["idd"]
        ms, si, inv = route_and_sort(lg, idd)
        # expert-major rows of x; the deduplicated dispatch sends tokens and expands them on the owner instead
        xs = None if (peer is not None and peer["dedup"]) else _expand_rows(hd, inv, k)
        if world == 1:
            y = grouped_gemm_forward(xs, w, ms)
            dx = grouped_gemm_forward_transposed(dyd, w, ms)
            dw = grouped_gemm_backward_dw(xs, dyd, ms, bf)
        elif peer is not None:
            cx, cdy = peer["x_all"], peer["dy_all"]
            if peer["dedup"]:
                pos_i, n_tok_i = token_positions(route(lg, idd).view(T, k), E, world)
                counts_i, tokens_i = gather_counts_and_tokens(ms, n_tok_i, world)
                pl = PeerPlan.from_counts(counts_i, world, rank)
                base_i = slot_bases(tokens_i, rank)
                peer_push_tokens(hd, pos_i, base_i, peer["tok"], rank)
                peer_push_index(pl, pos_i, base_i, si, k, peer["idx"])
            else:
                pl = PeerPlan.build(ms, world, rank)
                peer_push(pl, xs, cx)
            peer_push(pl, dyd, cdy)
            peer_fence(peer["token"])
            if peer["dedup"]:
                expand_received(peer["tok"].local, peer["idx"].local.view(-1), pl.recv_rows, cx.local)
            peer_grouped_gemm(pl, cx, w, peer["y"])
            peer_grouped_gemm(pl, cdy, w, peer["dx"], transposed=True)
            dw = grouped_gemm_backward_dw(cx.local, cdy.local, pl.local_m_sizes, bf)
            peer_fence(peer["token"])
            y, dx = peer["y"].local, peer["dx"].local
        else:
            pl = ExpertParallelPlan.build(ms, world, rank, dev)
            xl, dyl = pl.dispatch(xs), pl.dispatch(dyd)
            y = pl.combine(pl.grouped(grouped_gemm_forward, xl, w))
            dx = pl.combine(pl.grouped(grouped_gemm_forward_transposed, dyl, w))
            dw = pl.grouped_dw(grouped_gemm_backward_dw, xl, dyl, bf, E_local)
        sl["free"].record()
        # device -> host copy of the step's results (y, dX, dW, m_sizes) into pinned memory, on a stream of
        # its own so that it runs beside the next step; the host buffers alternate like the input slots
        bk = back[i % 2]
        bk["done"].synchronize()  # the copy that last wrote these host buffers has finished
        computed = torch.cuda.Event()
        computed.record()
        with torch.cuda.stream(back_stream):
            back_stream.wait_event(computed)
            for name, t in (("y", y), ("dx", dx), ("dw", dw), ("ms", ms)):
                bk[name][:t.shape[0]].copy_(t, non_blocking=True)
            bk["done"].record()
        bk["keep"] = (y, dx, dw, ms)  # the device tensors stay allocated until their copy has finished
        if world > 1 and peer is not None:
            # y / dX live in buffers that the next step's remote stores overwrite: the copy has to finish first
            torch.cuda.current_stream().wait_event(bk["done"])

    e2e_ms = float("nan")
    e2e_sampler = None
    if not args.no_e2e:
        upload(0)
        for i in range(3):
            step_e2e(i, i == 2)
        if rank == 0:
            e2e_sampler = ClockSampler(local_rank)
            e2e_sampler.start()
        barrier()
        e0, e1 = ev(), ev()
        e0.record()
        upload(0)  # the first step's upload is inside the timed region too
        for i in range(args.steps):
            step_e2e(i, i == args.steps - 1)
        torch.cuda.current_stream().wait_stream(back_stream)  # the last step's results have reached the host
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / args.steps
        for bk in back:
            bk.pop("keep", None)
    e2e_clocks = e2e_sampler.stop() if e2e_sampler is not None else None

    # ---- each GEMM alone (N = 1): isolated launches with idle time between them, i.e. at burst
    # clocks, to set beside the burst cuBLAS figure; the timed loop above runs under the power cap ----
    burst_ms = {}
    if world == 1 and not args.only:
        burst_ms["fwd"] = time_cuda(lambda: grouped_gemm_forward(x_d, w, m_sizes), iters=20)
        burst_ms["dx"] = time_cuda(lambda: grouped_gemm_forward_transposed(dy_d, w, m_sizes), iters=20)
        burst_ms["dw"] = time_cuda(lambda: grouped_gemm_backward_dw(x_d, dy_d, m_sizes, bf), iters=20)

    # ---- the row exchange alone (N > 1): one dispatch of x, timed on the device ----
    xchg_ms, remote_bytes = float("nan"), 0
    if world > 1:
        own = int(m_sizes.view(world, E_local)[rank].sum())
        remote_bytes = (M - own) * K * 2
        if peer is not None:
            if peer["dedup"]:
                remote_bytes = peer["tokens_out"] * K * 2 + (M - own) * 4

            def exchange():
                if peer["dedup"]:
                    peer_push_tokens(hidden_d, peer["pos"], peer["base"], peer["tok"], rank)
                    peer_push_index(peer["plans"][0], peer["pos"], peer["base"], peer["sort_idx"], k, peer["idx"])
                else:
                    for i in range(peer["n"]):
                        peer_push(peer["plans"][i], x_d, peer["x"][i])
                peer_fence(peer["token"])
        else:
            def exchange():
                plan.dispatch(x_d)
        for _ in range(3):
            exchange()
        barrier()
        x0, x1 = ev(), ev()
        x0.record()
        for _ in range(10):
            exchange()
        x1.record()
        barrier()
        xchg_ms = x0.elapsed_time(x1) / 10

    # ---- N > 1: one step's results against the single-GPU kernels (not timed) ----
    ep_check = None
    if world > 1 and not args.only and args.ep_chunks == 1:
        _, (y_ep, dx_ep, dw_ep) = step_resident(False)
        barrier()
        # every rank's rows and gradients, and every rank's share of the weights, on every rank
        xs_all = [torch.empty_like(x_d) for _ in range(world)]
        dys_all = [torch.empty_like(dy_d) for _ in range(world)]
        dist.all_gather(xs_all, x_d)
        dist.all_gather(dys_all, dy_d)
        counts_all = torch.empty(world * E, dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(counts_all, m_sizes.to(torch.int32).contiguous())
        counts_all = counts_all.view(world, E)
        if rank == 0:
            rel = lambda a, b: float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-30))
            w_full = torch.cat([(torch.randn(E_local, N, K, generator=torch.Generator().manual_seed(99 + r)) * 0.02).to(bf).to(dev)
                                for r in range(world)])
            errs = {"y": rel(y_ep[:M], grouped_gemm_forward(x_d, w_full, m_sizes)),
                    "dx": rel(dx_ep[:M], grouped_gemm_forward_transposed(dy_d, w_full, m_sizes))}
            # dW of this rank's experts: their rows from every rank, expert by expert
            begins = (counts_all.long().cumsum(dim=1) - counts_all.long()).cpu()
            cnt = counts_all.cpu()
            take = lambda rows_all: torch.cat([rows_all[r][int(begins[r, e]):int(begins[r, e]) + int(cnt[r, e])]
                                               for e in range(E_local) for r in range(world)])
            m_local = cnt[:, :E_local].sum(dim=0).to(torch.int32).to(dev)
            errs["dw"] = rel(dw_ep, grouped_gemm_backward_dw(take(xs_all), take(dys_all), m_local, bf))
            ep_check = {"what": "rank 0's y and dX rows and its experts' dW after one expert-parallel step, against the "
                                "single-GPU kernels on the same rows; max |a - b| / max |b|", "tolerance": 1e-2, **errs,
                        "ok": all(v <= 1e-2 for v in errs.values())}
            del w_full
        del xs_all, dys_all
        barrier()

    # max over ranks
    times = torch.tensor([resident_ms, e2e_ms, float(np.mean(kernel_ms["fwd"])), float(np.mean(kernel_ms["dx"])),
                          float(np.mean(kernel_ms["dw"])), xchg_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    resident_ms, e2e_ms, fwd_ms, dx_ms, dw_ms, xchg_ms = times.tolist()
    err_flag = _lib.read_error_flag()

    if rank == 0:
        peaks, peaks_kind = measured_peaks()
        flops_one = 2.0 * M * N * K  # per GEMM per GPU
        total_flops = 3 * flops_one * world
        per_kernel = {"fwd": fwd_ms, "dx": dx_ms, "dw": dw_ms}
        if args.only:
            per_kernel = {args.only: per_kernel[args.only]}
        total_flops = len(per_kernel) * flops_one * world
        dominant = max(per_kernel, key=per_kernel.get)
        achieved = flops_one / (per_kernel[dominant] * 1e-3) / 1e12
        alg_bytes = 2.0 * (M * K + E_local * N * K + M * N)
        # Which measured cuBLAS figure the timed loop is comparable with: the sustained one only when the
        # loop ran long enough for the power cap to act (>= 1 s) and the sampled SM clock sat below its
        # maximum; a short loop at full clock is the burst regime.
        timed_s = resident_ms * 1e-3 * args.steps
        sm, sm_max = (clocks or {}).get("sm_mhz"), (clocks or {}).get("sm_max_mhz")
        sustained = timed_s >= 1.0 and sm is not None and sm_max is not None and sm < 0.97 * sm_max
        peak_name = "bf16_tflops_sustained" if sustained else "bf16_tflops"
        peak = peaks[peak_name]
        ratio, traffic_case = ncu_traffic_ratio(dominant) if args.gemm_path == "auto" and world == 1 else (None, "not captured for this configuration")
        line = {
            "metric": "moe_fused_linear fwd+dX+dW algorithmic TFLOP/s", "value": total_flops / (resident_ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": n_warm, "ms_per_step": resident_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(args, cfg),
            "kernels": {name: {"ms": ms, "tflops": flops_one / (ms * 1e-3) / 1e12,
                               "frac_of_sustained_peak": flops_one / (ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
                               "frac_of_burst_peak": flops_one / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
                               "frac_of_nominal_2250": flops_one / (ms * 1e-3) / 1e12 / 2250.0,
                               "algorithmic_gbs": alg_bytes / (ms * 1e-3) / 1e9}
                        for name, ms in per_kernel.items()},
            "roofline": {"bound": "tensor", "kernel": f"tc grouped gemm {dominant}", "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak, "peak_kind": f"{peak_name}, {peaks_kind}",
                         "frac_of_burst_peak": achieved / peaks["bf16_tflops"],
                         "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"],
                         "regime": {"timed_region_s": timed_s, "sm_mhz_median": sm, "sm_max_mhz": sm_max,
                                    "denominator": "sustained" if sustained else "burst",
                                    # tensor work per SM clock: comparable across runs whose clocks differ
                                    "flop_per_sm_clock": (flops_one / (per_kernel[dominant] * 1e-3) / (sm * 1e6)) if sm else None},
                         "traffic": ratio * alg_bytes if ratio is not None else None,
                         "traffic_note": f"ncu DRAM bytes / algorithmic bytes of the capture, scaled by units ({traffic_case})",
                         "algorithmic_bytes": alg_bytes},
            "e2e": {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "inputs double-buffered: the upload of step i+1 runs beside the compute of step i; y, dX, dW and "
                            "m_sizes of every step are copied back into pinned host memory inside the timed region",
                    "tokens_per_s": T * world / (e2e_ms * 1e-3), "clocks": e2e_clocks},
            "gpu_launches": args.steps * (2 if args.only else launches_per_step),
            "tokens_per_s": T * world / (resident_ms * 1e-3),
            "clocks": clocks, "kernel_wait_errors": err_flag,
        }
        for name in per_kernel:  # spread over the timed steps (this rank), as the reference's do_bench quantiles
            q = np.percentile(kernel_ms[name], [20, 50, 80])
            line["kernels"][name].update(ms_p20=float(q[0]), ms_p50=float(q[1]), ms_p80=float(q[2]))
        for name, ms in burst_ms.items():
            line["kernels"][name].update(isolated_ms=ms, isolated_tflops=flops_one / (ms * 1e-3) / 1e12,
                                         isolated_frac_of_burst_peak=flops_one / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"])
        line["step_issue"] = {"host_ms_per_step": host_issue_ms,
                              "between_steps_ms": ({"p50": float(np.median(gaps)), "max": float(np.max(gaps))} if gaps else None),
                              "note": "host time to enqueue one step; device time from a step's last GEMM to the next step's first"}
        if ep_check is not None:
            line["ep_check"] = ep_check
        if world > 1:
            line["exchange"] = {"what": "dispatch of x alone (rows to their experts' ranks), rank 0's remote bytes",
                                "transport": args.ep_transport, "dispatch": (args.ep_dispatch if peer is not None and peer["dedup"] else "rows"),
                                "ms": xchg_ms, "remote_bytes": remote_bytes,
                                "gbs_out": remote_bytes / (xchg_ms * 1e-3) / 1e9, "nvlink_peak_gbs_per_direction": 900.0}
        if world == 1 and not args.no_extra and not args.only and args.workload == "gate_up" and not args.tokens and not args.experts:
            line["extra_workloads"] = [measure_single_gpu_workload("down", min(args.steps, 50), args.warmup, dev)]
            line["kernel_wait_errors"] = err_flag | _lib.read_error_flag()
        if world == 1 and not args.no_cpu_baseline:
            tf, dt, cores = cpu_reference_arm(cfg, 1, 0, args.cpu_rows)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"{args.cpu_rows} of {M} sorted rows, fp32, fwd+dX+dW row loops, 1 pass, {dt:.1f} s",
                                    "vectorised_tflops": _optional(cpu_vectorised_arm, cfg, args.cpu_rows),
                                    "vectorised_note": "same sample, one fp32 GEMM per expert instead of one mat-vec per row "
                                                       "(not the reference's algorithm; the fairer CPU figure)"}
        print(json.dumps(line), flush=True)
        if ep_check is not None and not ep_check["ok"]:
            raise SystemExit(f"expert-parallel results differ from the single-GPU kernels: {ep_check}")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

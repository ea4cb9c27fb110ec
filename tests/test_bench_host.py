"""Host-side logic of bench.py that needs no GPU: workload table, synthetic routing, the ncu traffic
record, and the JSON line of the CPU reference arm (run as a child process, as a launcher would)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

import bench

ROOT = Path(__file__).resolve().parent.parent


def test_workloads_have_the_baseline_shapes():
    """gate_up: 8192 tokens x top-8, 2048 -> 1536, 128 experts; down: 65536 rows, 768 -> 2048."""
    g, d = bench.WORKLOADS["gate_up"], bench.WORKLOADS["down"]
    assert (g["tokens"], g["k"], g["K"], g["N"], g["E"]) == (8192, 8, 2048, 1536, 128)
    assert (d["tokens"] * d["k"], d["K"], d["N"], d["E"]) == (65536, 768, 2048, 128)
    text = " ".join(json.loads((ROOT / "BASELINE.json").read_text())["configs"])
    for needle in ("8192 tokens", "(128,1536,2048)", "(128,2048,768)", "Zipf(s=1.2)", "top-8"):
        assert needle in text


def test_softmax_routing_is_seeded_and_ragged():
    cfg = bench.WORKLOADS["gate_up"]
    logits, ids = bench.make_routing(cfg, seed=0)
    again, _ = bench.make_routing(cfg, seed=0)
    other, _ = bench.make_routing(cfg, seed=1)
    assert ids is None and logits.shape == (cfg["tokens"], cfg["E"]) and logits.dtype == torch.float32
    assert torch.equal(logits, again) and not torch.equal(logits, other)
    sel = torch.topk(torch.softmax(logits, dim=1), cfg["k"], dim=1).indices
    counts = np.bincount(sel.reshape(-1).numpy(), minlength=cfg["E"])
    assert counts.sum() == cfg["tokens"] * cfg["k"] and counts.min() > 0
    # ragged around 512 rows per expert: some experts just above two full 256-token tiles
    assert counts.std() > 5 and ((counts > 512) & (counts <= 576)).sum() >= 4


def test_zipf_routing_has_empty_and_heavy_experts():
    cfg = bench.WORKLOADS["down"]
    logits, ids = bench.make_routing(cfg, seed=0)
    assert logits is None and ids.shape == (cfg["tokens"] * cfg["k"],) and ids.dtype == torch.int64
    counts = np.bincount(ids.numpy(), minlength=cfg["E"])
    assert (counts == 0).sum() >= 3, "three experts are emptied"
    assert counts.max() > counts.sum() // 4, "the heaviest expert holds more than a quarter of the rows"
    assert int(ids.min()) >= 0 and int(ids.max()) < cfg["E"]
    # seeded: the same call gives the same ids
    assert torch.equal(ids, bench.make_routing(cfg, seed=0)[1])


def test_ncu_traffic_record():
    for kernel in ("fwd", "dx", "dw"):
        ratio, case = bench.ncu_traffic_ratio(kernel)
        assert ratio is not None and 0.5 < ratio < 1.5, (kernel, ratio, case)
        assert "ncu" in case and "16384 rows" in case
    ratio, why = bench.ncu_traffic_ratio("no such kernel")
    assert ratio is None and "no ncu traffic record" in why
    rec = json.loads(bench.NCU_TRAFFIC_FILE.read_text())
    assert rec["command"].startswith("python bench.py")


def test_peaks_have_a_fallback():
    peaks, kind = bench.measured_peaks()
    assert kind in ("measured", "fallback")
    for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
        assert float(peaks[key]) > 0
    assert bench.FALLBACK_PEAKS["bf16_tflops"] == 1590.0 and bench.FALLBACK_PEAKS["hbm_gbs"] == 6650.0


def test_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs the CPU port on a bounded sample and prints one JSON line with
    the reference arm's keys; under a launcher only rank 0 prints."""
    env = dict(os.environ)
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0", "--cpu-rows", "64"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] and "64 of 65536" in line["cpu_baseline"]["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "gate_up" in line["config"]["workload"] and "model" not in line["config"]

    env["RANK"] = "1"
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert res.returncode == 0 and not [ln for ln in res.stdout.splitlines() if ln.startswith("{")]


def test_vectorised_cpu_figure_computes_the_same_results_as_the_row_loops():
    from oracle import cpu_baseline as C

    g = torch.Generator().manual_seed(1)
    E, N, K, M = 5, 7, 9, 40
    w = torch.randn(E, N, K, generator=g)
    x, dy = torch.randn(M, K, generator=g), torch.randn(M, N, generator=g)
    experts = torch.sort(torch.randint(0, E - 1, (M,), generator=g)).values   # the last expert stays empty
    m_sizes = torch.bincount(experts, minlength=E)
    assert torch.allclose(C.vectorised_fwd(x, w, m_sizes), C.rowloop_fwd(x, w, experts), atol=1e-5)
    assert torch.allclose(C.vectorised_bwd_input(dy, w, m_sizes), C.rowloop_bwd_input(dy, w, experts), atol=1e-5)
    assert torch.allclose(C.vectorised_bwd_weight(dy, x, w, m_sizes), C.rowloop_bwd_weight(dy, x, w, experts), atol=1e-5)
    small = dict(tokens=64, K=32, N=16, E=4, k=2, routing="softmax")
    assert bench.cpu_vectorised_arm(small, 64) > 0

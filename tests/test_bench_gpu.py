"""The two benchmark scripts run end to end on a GPU with shortened legs, and their output carries the keys the
bench contract names (this guards the scripts themselves; the numbers are not judged here)."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_bench_line_has_every_contract_key():
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bench.py"), "--workload", "c1", "--steps", "5", "--warmup", "3", "--e2e-steps", "1",
         "--c5-steps", "2", "--c4-reps", "2", "--cpu-seconds", "0.5"],
        capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    (line,) = [json.loads(x) for x in proc.stdout.splitlines() if x.startswith("{")]
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "roofline", "cpu_baseline", "e2e", "clocks", "gpu_launches",
                "strong_c5", "c4_fused_gemm"):
        assert key in line, key
    assert line["n_gpus"] == 1 and line["steps"] == 5 and line["gpu_launches"] == 10  # one forward, one backward a step
    assert set(line["roofline"]) >= {"bound", "achieved", "peak", "unit", "frac", "traffic"}
    assert set(line["cpu_baseline"]) >= {"value", "unit", "cores", "kind", "sample"}
    e2e = line["e2e"]
    assert e2e["h2d_bytes_per_step"] == e2e["d2h_bytes_per_step"] == 3 * 256 * 1024 * 4
    assert e2e["copy_ceiling"]["ms_per_step"] > 0 and e2e["gpu_launches"] > 0
    strong = line["strong_c5"]
    assert strong["next_rank_block_reproduced_bit_exactly"] is True and strong["tokens_total"] == 65536
    assert line["c4_fused_gemm"]["ms"] > 0 and line["c4_fused_gemm"]["cublas_x2_plus_swiglu_ms"] > 0


def test_bench_all_runs_every_kind_of_provider():
    proc = subprocess.run(
        [sys.executable, str(ROOT / "benchmarks" / "bench_all.py"), "--configs", "c1", "--providers", "b200", "b200-safe",
         "b200-packed", "b200-graph", "ref-triton-fast", "ref-triton-packed", "ref-triton-geglu-erf", "torch-eager",
         "geglu-tanh", "liger", "--rep", "3",
         "--warmup", "1", "--save", "/tmp/swiglu_bench_all_test.json"],
        capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    rows = json.loads(Path("/tmp/swiglu_bench_all_test.json").read_text())["rows"]
    own = [r for r in rows if r["provider"].startswith("b200") and "unavailable" not in r]
    assert {r["mode"] for r in own} == {"forward", "backward", "full"} and len(own) == 12
    for r in own:
        assert r["gbs_per_gpu"] > 0 and r["peak_mib"] > 0 and "call_allocates_mib" in r
    # comparators either ran or say why not; they never take the script down
    for provider in ("ref-triton-fast", "ref-triton-packed", "ref-triton-geglu-erf", "liger"):
        mine = [r for r in rows if r["provider"] == provider]
        assert mine and (all("unavailable" in r for r in mine) or len(mine) == 3)

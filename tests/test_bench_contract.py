"""Host-side pieces of bench.py that need no GPU: the CPU arm (--impl reference) as the driver launches it, alone
and as ranks of a two-process job, and the helpers behind the roofline and strong-scaling fields."""
import json
import os
import subprocess
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def run_reference(extra_env, *args):
    env = dict(os.environ, **extra_env)
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1",
                           "--workload", "c1", *args], capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr
    return [json.loads(line) for line in proc.stdout.splitlines() if line.startswith("{")]


def test_reference_arm_prints_one_line_with_the_contract_fields():
    (line,) = run_reference({"OMP_NUM_THREADS": "1"})  # what torch.distributed.run exports to its workers
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["gpu_launches"] == 0 and line["steps"] == 2
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    base = line["cpu_baseline"]
    assert base["kind"] in ("reference", "port") and base["value"] == line["value"]
    # the arm undoes the single-thread setting it inherits: every core this process may use
    assert base["cores"] == len(os.sched_getaffinity(0))
    # ms_per_step is the measured time of one step over the sample, not an extrapolation
    sample_rows = min(256, (60 << 20) // (1024 * 4))
    assert abs(line["value"] - sample_rows / (line["ms_per_step"] * 1e-3)) <= 1e-6 * line["value"]
    assert line["config"]["global_tokens"] == 256 and "c1" in line["config"]["workload"]


def test_reference_arm_under_two_ranks_runs_on_rank_zero_only():
    common = {"WORLD_SIZE": "2", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29599", "OMP_NUM_THREADS": "1"}
    (line,) = run_reference(dict(common, RANK="0", LOCAL_RANK="0"), "--gpus", "2")
    assert line["n_gpus"] == 2 and line["config"]["global_tokens"] == 512  # the configuration of the 2-GPU job
    assert line["config"]["parallelism"].startswith("rows x2")
    assert run_reference(dict(common, RANK="1", LOCAL_RANK="1"), "--gpus", "2") == []


def test_reference_arm_does_not_map_the_cuda_library():
    code = ("import sys; sys.argv = ['bench.py', '--impl', 'reference', '--steps', '1', '--warmup', '1', '--workload', 'c1']\n"
            "import runpy; runpy.run_path(%r, run_name='__main__')\n"
            "print('MAPPED' if 'libswiglu_b200' in open('/proc/self/maps').read() else 'NOT MAPPED')\n" % str(ROOT / "bench.py"))
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr
    assert proc.stdout.strip().endswith("NOT MAPPED")


def test_roofline_traffic_scales_with_the_workload():
    from kernel_pocs_b200 import workloads as W

    ws = W.workloads()
    c2 = bench.scaled_bwd_traffic(ws["c2"], ws["c2"].tokens)
    assert c2 == 4 * (704_655_872 + 413_662_464)                      # four times the 8192-row capture
    assert bench.scaled_bwd_traffic(ws["c2"], 8192) == 704_655_872 + 413_662_464
    assert 0.94 < c2 / ws["c2"].bytes_bwd() < 0.96                    # writes still in L2 at kernel end are missing
    fp32 = bench.scaled_bwd_traffic(ws["c3-fp32"], ws["c3-fp32"].tokens)
    assert abs(fp32 / ws["c3-fp32"].bytes_bwd() - c2 / ws["c2"].bytes_bwd()) < 1e-9


def test_weighted_hash_is_exact_and_order_sensitive():
    a = torch.arange(-300, 300, dtype=torch.float32).bfloat16()
    b = a.flip(0)
    assert bench.weighted_hash(a) == bench.weighted_hash(a.clone())
    assert bench.weighted_hash(a) != bench.weighted_hash(b)
    assert isinstance(bench.weighted_hash(a.float()), int)

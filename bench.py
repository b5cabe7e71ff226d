"""Headline benchmark of the SwiGLU path: forward + backward on the Llama-3-8B MLP shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl native|reference]

One "step" is one pass of the hot path over one batch: ``h = swiglu(gate, up)`` followed by the
backward ``(dgate, dup)`` from ``dh`` (in place over gate/up, the operator's default), called
through the public autograd API.  At N GPUs every rank holds its own block of token rows of
the workload (weak scaling: rows are independent, there is no data-path collective; NCCL only
carries the barrier and the max-over-ranks of the timings).

Prints ONE JSON line on rank 0.  ``value`` is device-timed tokens/s with inputs resident in HBM;
``e2e`` is the same step driven from pinned HOST buffers with the host-to-device and
device-to-host copies inside the timed region; ``roofline`` rates the dominant kernel (the
backward) against the measured HBM copy bandwidth of this GPU pool; ``cpu_baseline`` times the
reference's CPU path (its ATen composite + autograd, restated in oracle/) on a bounded sample
of the same workload on the host cores.

``--impl reference`` times that CPU path alone, same metric and configuration.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch

DTYPE_NAME = {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16"}
METRIC = "swiglu_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this GPU pool, used when MEASURED_PEAKS.json is absent
# dram__bytes_read.sum + dram__bytes_write.sum of one backward launch on the c2 workload: the ncu
# capture of the first 8192 of its 32768 token rows (profiles/swiglu_fwd_bwd_c2_8192rows_ncu_full.md:
# 704.66 MB read + 413.66 MB written) scaled by 4; the traffic of this pure stream grows in proportion
# to the rows.  Reads equal the algorithmic reads exactly; writes are short by what L2 still holds
# when the kernel ends.
BWD_DRAM_TRAFFIC_BYTES_C2 = 4 * (704_655_872 + 413_662_464)


def parse_args():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c3-fp32", "c5"])
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--preserve-inputs", action="store_true", help="out-of-place backward instead of the default in-place")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="time limit of the cpu_baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def measured_hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ---------------------------------------------------------------------------------------------
# clocks during the timed region
# ---------------------------------------------------------------------------------------------

class ClockSampler:
    """Samples the SM clock and the clock-event reasons of one GPU while a region runs.
    Reads only (NVML queries, or nvidia-smi when the NVML binding is missing)."""

    NAMES = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.004):
        self.samples = []  # (sm_mhz, reasons bitmask)
        self.sm_max = None
        self._stop = threading.Event()
        self.backend = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self.backend = "nvml"
            self.thread = threading.Thread(target=self._poll_nvml, args=(period_s,), daemon=True)
            self.thread.start()
        except Exception:
            try:
                self.proc = subprocess.Popen(
                    ["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.active",
                     "--format=csv,noheader,nounits", "-i", str(index), "-lms", "50"],
                    stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                self.backend = "nvidia-smi"
                self.thread = threading.Thread(target=self._read_smi, daemon=True)
                self.thread.start()
            except Exception:
                self.backend = None

    @staticmethod
    def _physical_index(index: int) -> int:
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            if index < len(ids) and ids[index].isdigit():
                return int(ids[index])
        return index

    def _poll_nvml(self, period_s):
        nv = self._nv
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            try:
                self.samples.append((float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)),
                                     int(reasons_fn(self._h))))
            except Exception:
                pass
            time.sleep(period_s)

    def _read_smi(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            try:
                self.sm_max = float(parts[1])
                self.samples.append((float(parts[0]), int(parts[2], 16)))
            except Exception:
                continue

    def mark(self) -> int:
        return len(self.samples)

    def stop(self):
        self._stop.set()
        if self.backend == "nvidia-smi":
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, lo: int = 0, hi: int | None = None):
        rows = self.samples[lo:hi]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["no samples"], "samples": 0,
                    "source": self.backend}
        mask = 0
        for _, m in rows:
            mask |= m
        return {"sm_mhz": statistics.median(r[0] for r in rows), "sm_min_mhz": min(r[0] for r in rows),
                "sm_max_mhz": self.sm_max, "reasons": [n for bit, n in self.NAMES.items() if mask & bit],
                "samples": len(rows), "source": self.backend}


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU path (ATen composite + autograd), restated in oracle/
# ---------------------------------------------------------------------------------------------

def cpu_sample_rows(w) -> int:
    # ~60 MB per tensor: a couple of hundred milliseconds per step on a handful of cores
    rows = max(1, (60 << 20) // (w.width * torch.empty((), dtype=w.dtype).element_size()))
    return min(w.tokens, rows)


def time_cpu_path(w, limit_s: float, min_steps: int = 3, fixed_steps: int | None = None, warmup: int = 1):
    """tokens/s of fwd+bwd on the host for a row sample of workload ``w``."""
    from kernel_pocs_b200 import workloads as W
    from oracle import oracle as O

    rows = cpu_sample_rows(w)
    gate, up, dh = W.generate_rows(w, 0, rows, "cpu")
    for _ in range(warmup):
        O.aten_fwd_bwd(gate, up, dh)
    times = []
    t_begin = time.perf_counter()
    while True:
        t0 = time.perf_counter()
        O.aten_fwd_bwd(gate, up, dh)
        times.append(time.perf_counter() - t0)
        if fixed_steps is not None:
            if len(times) >= fixed_steps:
                break
        elif len(times) >= min_steps and time.perf_counter() - t_begin > limit_s:
            break
    sec = sum(times) / len(times)
    return {
        "value": rows / sec,
        "unit": UNIT,
        "cores": torch.get_num_threads(),
        "host_cpus": os.cpu_count(),
        "kind": "port",
        "sample": f"first {rows} of {w.tokens} token rows of {w.name} ({w.width} wide, {DTYPE_NAME[w.dtype]}), "
                  f"{len(times)} steps of fwd+bwd by the ATen composite + autograd, mean {sec * 1e3:.1f} ms/step",
        "ms_per_step_sample": sec * 1e3,
        "steps": len(times),
    }


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    res = time_cpu_path(w, 0.0, fixed_steps=args.steps, warmup=max(args.warmup, 1))
    rows = cpu_sample_rows(w)
    line = {
        "impl": "reference",
        "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": res["ms_per_step_sample"] * (w.tokens / rows),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE_NAME[w.dtype], "data": "synthetic",
        "config": config_of(w, args, 1),
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU path of the reference (its PyTorch composite + autograd) on this host; ms_per_step is the "
                "sample time scaled to the full workload",
    }
    print(json.dumps(line), flush=True)


def config_of(w, args, world):
    return {
        "workload": f"{w.name}: {w.note}; gate/up/dh {DTYPE_NAME[w.dtype]} [{w.tokens}, {w.width}] per GPU, "
                    f"N(0,{w.std:g}^2), seed {w.seed}",
        "tokens_per_gpu": w.tokens, "width": w.width, "global_tokens": w.tokens * world,
        "backward": "out-of-place" if args.preserve_inputs else "in-place",
        "parallelism": f"rows x{world}, no collective",
        "l2": "inputs >> L2 (2.8 GB forward, 4.7 GB backward per step vs 126 MB); between timed steps, untimed: gate/up "
              "restored from pristine copies, then one read-only pass over dh evicts the copies' dirty lines"
              if w.name != "c1" else "fits L2 (parity case, launch-bound)",
    }


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def main():
    args = parse_args()
    from kernel_pocs_b200 import workloads as W

    w = W.workloads()[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, w)
        return

    from kernel_pocs_b200 import build as product_build

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SwiGLU path has no CPU fallback")

    if rank == 0:
        product_build.build()
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        dist.barrier()

    from kernel_pocs_b200 import _lib
    from kernels.swiglu import swiglu

    # weak scaling: rank r owns rows [r*T, (r+1)*T) of a [world*T, width] matrix
    lo = rank * w.tokens
    gate0, up0, dh = W.generate_rows(w, lo, lo + w.tokens, device)
    gate = gate0.clone().requires_grad_(True)
    up = up0.clone().requires_grad_(True)
    preserve = bool(args.preserve_inputs)

    def restore():
        # untimed, between steps: put the pristine gate/up back (the in-place backward overwrote
        # them), then stream dh once (read-only, 0.94 GB > L2) so that the dirty lines the copies
        # left in L2 are written back before the timed kernels start
        with torch.no_grad():
            gate.copy_(gate0)
            up.copy_(up0)
            dh.sum()

    def step(events=None):
        if events:
            events[0].record()
        h = swiglu(gate, up, 1.0, 1.0, preserve)
        if events:
            events[1].record()
        dgate, dup = torch.autograd.grad(h, (gate, up), dh)
        if events:
            events[2].record()
        return h, dgate, dup

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        restore()
        step()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    time.sleep(0.3 if sampler else 0.0)

    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    mark0 = sampler.mark() if sampler else 0
    launches0 = _lib.launch_count()
    wall0 = time.perf_counter()
    for k in range(args.steps):
        restore()  # untimed: between the previous step's last event and this step's first
        step(evs[k])
    barrier()
    wall = time.perf_counter() - wall0
    launches = _lib.launch_count() - launches0
    mark1 = sampler.mark() if sampler else 0

    fwd_ms = [e[0].elapsed_time(e[1]) for e in evs]
    bwd_ms = [e[1].elapsed_time(e[2]) for e in evs]
    step_ms = [e[0].elapsed_time(e[2]) for e in evs]
    total_ms = sum(step_ms)
    t = torch.tensor([total_ms, sum(fwd_ms), sum(bwd_ms)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, fwd_total, bwd_total = t.tolist()
    ms_per_step = total_ms / args.steps
    tokens_total = w.tokens * world
    value = tokens_total / (ms_per_step * 1e-3)

    # ---- end to end from pinned host buffers -------------------------------------------------
    e2e = None
    if not args.no_e2e:
        from kernel_pocs_b200.host_path import swiglu_fwd_bwd_host, workspace_bytes

        es = gate0.element_size()
        hg, hu, hd = (torch.empty(x.shape, dtype=x.dtype, pin_memory=True) for x in (gate0, up0, dh))
        hg.copy_(gate0), hu.copy_(up0), hd.copy_(dh)
        outs = tuple(torch.empty(gate0.shape, dtype=gate0.dtype, pin_memory=True) for _ in range(3))
        ws = torch.empty(workspace_bytes(w.tokens, w.width, w.dtype), dtype=torch.uint8, device=device)

        def e2e_step():
            # one call of the host-buffer entry point: chunks of rows are copied in, run through
            # the forward and the in-place backward, and copied out, three chunks in flight
            swiglu_fwd_bwd_host(hg, hu, hd, 1.0, 1.0, out=outs, workspace=ws)

        for _ in range(2):
            e2e_step()
        barrier()
        e2e_launches0 = _lib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_launches = _lib.launch_count() - e2e_launches0
        te = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = te.item() / args.e2e_steps
        # the bytes that came back are the device path's results
        restore()
        h_dev, dgate_dev, dup_dev = step()
        for got, want in zip(outs, (h_dev, dgate_dev, dup_dev)):
            if not torch.equal(got[:64], want[:64].cpu()) or not torch.equal(got[-64:], want[-64:].cpu()):
                raise SystemExit("e2e: the bytes copied back to the host differ from the device result")
        e2e = {"value": tokens_total / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 3 * gate0.numel() * es * world, "d2h_bytes_per_step": 3 * gate0.numel() * es * world,
               "steps": args.e2e_steps, "gpu_launches": e2e_launches,
               "path": "swiglu_b200_host_fwd_bwd: pinned host gate/up/dh -> device workspace in row chunks, forward + "
                       "in-place backward per chunk, h/dgate/dup -> pinned host; copies of neighbouring chunks overlap "
                       "the kernels"}
        del ws

    if sampler:
        sampler.stop()

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        bwd_avg_s = bwd_total / args.steps * 1e-3
        fwd_avg_s = fwd_total / args.steps * 1e-3
        bwd_gbs = w.bytes_bwd() / bwd_avg_s / 1e9
        fwd_gbs = w.bytes_fwd() / fwd_avg_s / 1e9
        both_gbs = (w.bytes_fwd() + w.bytes_bwd()) / (ms_per_step * 1e-3) / 1e9
        dt = DTYPE_NAME[w.dtype]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": config_of(w, args, world),
            "hbm_gbs_per_gpu": {"fwd": fwd_gbs, "bwd": bwd_gbs, "fwd_bwd": both_gbs,
                                "fwd_ms": fwd_avg_s * 1e3, "bwd_ms": bwd_avg_s * 1e3,
                                "frac_of_measured_copy": both_gbs / peak, "frac_of_nominal_8000": both_gbs / 8000.0},
            "roofline": {"bound": "hbm", "kernel": f"swiglu_bwd_kernel<{dt}, 16 B vectors, "
                                                   f"{'out-of-place' if preserve else 'in-place'}>",
                         "achieved": bwd_gbs, "peak": peak, "unit": "GB/s", "frac": bwd_gbs / peak,
                         "peak_source": f"{peak_kind} copy bandwidth (burst)",
                         "traffic": BWD_DRAM_TRAFFIC_BYTES_C2 if w.name == "c2" else None,
                         "algorithmic_bytes": w.bytes_bwd()},
            "clocks": sampler.summary(mark0, mark1) if sampler else None,
            "e2e": e2e,
            "gpu_launches": launches,
            "wall_s_timed_loop_incl_restores": wall,
        }
        if not args.no_cpu_baseline and world == 1:
            res = time_cpu_path(w, args.cpu_seconds)
            line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

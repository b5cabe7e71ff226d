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
# dram__bytes_read.sum + dram__bytes_write.sum of ONE in-place bf16 backward launch over 8192 token
# rows of width 14336 (an ncu capture of the first quarter of the c2 workload: 704.66 MB read,
# 413.66 MB written).  The kernel is a pure stream, so its traffic grows in proportion to the
# elements it processes: `roofline.traffic` is this figure scaled by elements and element size.
# Reads equal the algorithmic reads exactly; writes are short by what L2 still holds when the
# kernel ends.
BWD_DRAM_TRAFFIC_CAPTURE = {"bytes": 704_655_872 + 413_662_464, "elements": 8192 * 14336, "itemsize": 2}


def scaled_bwd_traffic(w, tokens: int) -> int:
    c = BWD_DRAM_TRAFFIC_CAPTURE
    itemsize = torch.empty((), dtype=w.dtype).element_size()
    return round(c["bytes"] * (tokens * w.width / c["elements"]) * (itemsize / c["itemsize"]))


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
    ap.add_argument("--no-strong-c5", action="store_true", help="skip the strong-scaling sub-record")
    ap.add_argument("--c5-steps", type=int, default=20)
    ap.add_argument("--no-c4", action="store_true", help="skip the fused-GEMM sub-record")
    ap.add_argument("--c4-reps", type=int, default=20)
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


def host_threads() -> int:
    """Host cores this process may use.  torch.distributed.run exports OMP_NUM_THREADS=1 to its
    workers; the CPU arm undoes that for itself, since it is the only work on the host."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_step_fn():
    """(kind, step) for the CPU arm.  ``step(gate, up, dh)`` runs one forward + backward on host
    tensors: through the reference's own ``swiglu()`` when the unmodified copy of its module is
    present under baseline/_ref ("reference"), else through the restatement of that same CPU
    path in oracle/ ("port").  Both evaluate the ATen composite and its autograd backward."""
    try:
        from benchmarks import fetch_reference

        ref = fetch_reference.load()

        def step(gate, up, dh):
            g = gate.detach().clone().requires_grad_(True)
            u = up.detach().clone().requires_grad_(True)
            h = ref.swiglu(g, u)  # host tensors: kernels/swiglu/swiglu.py:396-397 -> torch_swiglu_reference
            dgate, dup = torch.autograd.grad(h, (g, u), dh)
            return h.detach(), dgate, dup

        return "reference", step
    except Exception:
        from oracle import oracle as O

        return "port", O.aten_fwd_bwd


def time_cpu_path(w, limit_s: float, min_steps: int = 3, fixed_steps: int | None = None, warmup: int = 1):
    """tokens/s of fwd+bwd on the host for a row sample of workload ``w``."""
    from kernel_pocs_b200 import workloads as W

    torch.set_num_threads(host_threads())
    kind, step = cpu_step_fn()
    rows = cpu_sample_rows(w)
    gate, up, dh = W.generate_rows(w, 0, rows, "cpu")
    for _ in range(warmup):
        step(gate, up, dh)
    times = []
    t_begin = time.perf_counter()
    while True:
        t0 = time.perf_counter()
        step(gate, up, dh)
        times.append(time.perf_counter() - t0)
        if fixed_steps is not None:
            if len(times) >= fixed_steps:
                break
        elif len(times) >= min_steps and time.perf_counter() - t_begin > limit_s:
            break
    sec = sum(times) / len(times)
    how = ("the reference's own swiglu() on host tensors + autograd" if kind == "reference"
           else "the ATen composite + autograd as the reference's swiglu() evaluates them for host tensors")
    return {
        "value": rows / sec,
        "unit": UNIT,
        "cores": torch.get_num_threads(),
        "host_cpus": os.cpu_count(),
        "kind": kind,
        "sample": f"first {rows} of {w.tokens} token rows of {w.name} ({w.width} wide, {DTYPE_NAME[w.dtype]}), "
                  f"{len(times)} steps of fwd+bwd by {how}, mean {sec * 1e3:.1f} ms/step",
        "sample_rows": rows,
        "ms_per_step_sample": sec * 1e3,
        "steps": len(times),
    }


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = max(1, int(os.environ.get("WORLD_SIZE", "1")), args.gpus)
    res = time_cpu_path(w, 0.0, fixed_steps=args.steps, warmup=max(args.warmup, 1))
    rows = res["sample_rows"]
    line = {
        "impl": "reference",
        "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": res["ms_per_step_sample"],
        "ms_per_step_full_workload_extrapolated": res["ms_per_step_sample"] * (w.tokens * world / rows),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE_NAME[w.dtype], "data": "synthetic",
        "config": config_of(w, args, world),
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU path of the reference (its PyTorch composite + autograd) on this host, all host threads, "
                f"rank 0 only; one step = fwd+bwd over a {rows}-row sample of the workload and ms_per_step is the "
                "measured time of that step; tokens/s = sample rows / that time",
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
# host placement and the copy ceiling of the end-to-end leg
# ---------------------------------------------------------------------------------------------

def gpu_pci_address(index: int) -> str | None:
    """PCI address "dddd:bb:dd.f" of the visible device ``index`` (NVML first, torch's device
    properties otherwise)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(ClockSampler._physical_index(index))
        bus_id = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus_id = bus_id.decode() if isinstance(bus_id, bytes) else bus_id
        return bus_id.lower()[-12:]  # NVML pads the domain to eight digits
    except Exception:
        pass
    try:
        p_ = torch.cuda.get_device_properties(index)
        return f"{p_.pci_domain_id:04x}:{p_.pci_bus_id:02x}:{p_.pci_device_id:02x}.0"
    except Exception:
        return None


def bind_host_near_gpu(index: int) -> dict:
    """Pins this process to the CPUs of the NUMA node its GPU hangs off, BEFORE any pinned buffer
    is allocated, so that the staging memory of the end-to-end leg is local to the GPU's PCIe
    root.  Host side only (scheduler affinity of this process); nothing on the GPU changes.
    Returns what it found for the JSON line."""
    info = {"pci": gpu_pci_address(index), "numa_node": None, "cpus_bound": None}
    if info["pci"] is None:
        return info
    try:
        node = int((Path("/sys/bus/pci/devices") / info["pci"] / "numa_node").read_text().strip())
    except Exception:
        return info
    info["numa_node"] = node
    if node < 0:  # the platform reports no affinity (one node, or a virtual machine)
        return info
    try:
        cpus = set()
        for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["cpus_bound"] = len(allowed)
    except Exception:
        pass
    return info


def copy_ceiling_ms(pinned_in, pinned_out, device, chunk_bytes: int, steps: int, barrier):
    """What the host link allows for one end-to-end step with no kernel at all: the step's input
    bytes host-to-device on one stream and its output bytes device-to-host on another, at the same
    time, one plain asynchronous copy per chunk, every rank at once.  Returns ms per step."""
    staging_in = torch.empty(chunk_bytes, dtype=torch.uint8, device=device)
    staging_out = torch.empty(chunk_bytes, dtype=torch.uint8, device=device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    flat_in = [t.view(-1).view(torch.uint8) for t in pinned_in]
    flat_out = [t.view(-1).view(torch.uint8) for t in pinned_out]

    def one_step():
        with torch.cuda.stream(s_in):
            for t in flat_in:
                for off in range(0, t.numel(), chunk_bytes):
                    n = min(chunk_bytes, t.numel() - off)
                    staging_in[:n].copy_(t[off:off + n], non_blocking=True)
        with torch.cuda.stream(s_out):
            for t in flat_out:
                for off in range(0, t.numel(), chunk_bytes):
                    n = min(chunk_bytes, t.numel() - off)
                    t[off:off + n].copy_(staging_out[:n], non_blocking=True)

    one_step()
    barrier()
    cur = torch.cuda.current_stream(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(cur)
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    for _ in range(steps):
        one_step()
    cur.wait_stream(s_in)
    cur.wait_stream(s_out)
    e1.record(cur)
    barrier()
    return e0.elapsed_time(e1) / steps


# ---------------------------------------------------------------------------------------------
# strong scaling of the Llama-3-70B activation shape (rows split over the ranks, no collective)
# ---------------------------------------------------------------------------------------------

def weighted_hash(t: torch.Tensor) -> int:
    """Order-sensitive integer hash of a tensor's bit patterns (exact: integer arithmetic)."""
    bits = t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32).reshape(-1).to(torch.int64)
    weights = torch.arange(bits.numel(), device=t.device, dtype=torch.int64) % 65521 + 1
    return int((bits * weights).sum().item())


def run_strong_c5(W, swiglu_forward, swiglu_backward, launch_count, device, rank, world, dist, barrier, steps):
    """[65536, 28672] bf16, seed 4, split by contiguous token rows over the ranks.  Aggregate
    tokens/s = all tokens / max over ranks of the median step time; per-GPU GB/s from each rank's
    own time; a checksum of every output bit over all ranks (identical at every rank count exactly
    when the results are); and a cross-check that the first rows of the next rank's block,
    generated and computed here, hash like that rank's own."""
    w = W.workloads()["c5"]
    lo, hi = W.row_shard(w.tokens, world, rank)
    gate0, up0, dh = W.generate_rows(w, lo, hi, device)
    gate, up = gate0.clone(), up0.clone()

    def restore():
        gate.copy_(gate0)
        up.copy_(up0)
        dh.sum()

    def step():
        h, g2, u2 = swiglu_forward(gate, up)
        dgate, dup = swiglu_backward(dh, g2, u2)  # in place over gate/up, the operator's default
        return h, dgate, dup

    for _ in range(3):
        restore()
        h, dgate, dup = step()  # kept, as in the timed loop: the allocator then already owns the second h buffer
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    barrier()
    launches0 = launch_count()
    for a, b in evs:
        restore()
        a.record()
        h, dgate, dup = step()
        b.record()
    barrier()
    launches = launch_count() - launches0
    per_step = sorted(a.elapsed_time(b) for a, b in evs)
    # the median, so that a one-off host stall inside a step (a cudaMalloc of the caching allocator, say) does not
    # decide the figure; the mean is reported beside it
    mine_ms = per_step[len(per_step) // 2] if len(per_step) % 2 else 0.5 * (per_step[len(per_step) // 2 - 1] + per_step[len(per_step) // 2])
    mine_mean_ms = sum(per_step) / steps
    probe = min(64, hi - lo)
    own_hash = [weighted_hash(t[:probe]) for t in (h, dgate, dup)]
    checksum = [int(t.view(torch.int16).sum(dtype=torch.int64).item()) for t in (h, dgate, dup)]
    del h, dgate, dup, gate, up, gate0, up0, dh
    torch.cuda.empty_cache()

    # the first rows of the NEXT rank's block, generated and computed on this device
    nlo, nhi = W.row_shard(w.tokens, world, (rank + 1) % world)
    nprobe = min(64, nhi - nlo)
    ng, nu, nd = W.generate_rows(w, nlo, nlo + nprobe, device)
    nh, ng2, nu2 = swiglu_forward(ng, nu)
    ndg, ndu = swiglu_backward(nd, ng2, nu2)
    neighbour_hash = [weighted_hash(t) for t in (nh, ndg, ndu)]

    # hashes do not fit a double exactly: gather them as int64 beside the timings
    ints = torch.tensor([*own_hash, *neighbour_hash, *checksum], dtype=torch.int64, device=device)
    if world > 1:
        all_ms = [torch.zeros(2, dtype=torch.float64, device=device) for _ in range(world)]
        dist.all_gather(all_ms, torch.tensor([mine_ms, mine_mean_ms], dtype=torch.float64, device=device))
        all_ints = [torch.zeros_like(ints) for _ in range(world)]
        dist.all_gather(all_ints, ints)
        all_mean_ms = [float(t[1].item()) for t in all_ms]
        all_ms = [float(t[0].item()) for t in all_ms]
        all_ints = [t.tolist() for t in all_ints]
    else:
        all_ms, all_mean_ms, all_ints = [mine_ms], [mine_mean_ms], [ints.tolist()]
    if rank != 0:
        return None
    shards = [W.row_shard(w.tokens, world, r) for r in range(world)]
    bytes_per_row = 8 * w.width * 2
    cross_ok = all(all_ints[r][3:6] == all_ints[(r + 1) % world][0:3] for r in range(world))
    total = [sum(all_ints[r][6 + i] for r in range(world)) for i in range(3)]
    worst = max(all_ms)
    return {
        "workload": f"c5: {w.note}; gate/up/dh bf16 [{w.tokens}, {w.width}] in total, N(0,1), seed {w.seed}, "
                    f"contiguous token rows split over {world} GPU(s), no collective",
        "scaling": "strong", "n_gpus": world, "steps": steps, "tokens_total": w.tokens,
        "ms_per_step": worst, "value": w.tokens / (worst * 1e-3), "unit": UNIT,
        "ms_per_step_by_rank": all_ms, "ms_per_step_mean_by_rank": all_mean_ms,
        "timing": "per step one CUDA-event pair; per rank the median step, over ranks the maximum",
        "hbm_gbs_per_gpu": [(b - a) * bytes_per_row / (ms * 1e-3) / 1e9 for (a, b), ms in zip(shards, all_ms)],
        "gpu_launches_rank0": launches,
        "output_checksum_h_dgate_dup": total,
        "next_rank_block_reproduced_bit_exactly": cross_ok,
    }


# ---------------------------------------------------------------------------------------------
# fused gate/up projection + SwiGLU (benchmark configuration c4), beside the unfused sequence
# ---------------------------------------------------------------------------------------------

def measured_tensor_peaks():
    try:
        d = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


def run_c4_fused_gemm(device, reps: int):
    """X bf16 [16384, 4096] ~ N(0,1), W_gate and W_up bf16 [14336, 4096] ~ N(0, 0.02^2), seed 3.  The fused tcgen05
    kernel (one launch: both projections and the activation) and the unfused sequence it replaces (two cuBLAS
    GEMMs, then this library's SwiGLU kernel) are timed ALTERNATELY in one loop, each call between its own pair of
    CUDA events, so both see the same clocks under the power cap.  FLOPs: 4*M*N*K."""
    from kernel_pocs_b200.fused_mlp import check_status, gate_up_swiglu_forward
    from kernels.swiglu import swiglu_forward

    m, n, k = 16384, 14336, 4096
    g = torch.Generator(device=device).manual_seed(3)
    x = torch.randn(m, k, generator=g, device=device).bfloat16()
    wg = (0.02 * torch.randn(n, k, generator=g, device=device)).bfloat16()
    wu = (0.02 * torch.randn(n, k, generator=g, device=device)).bfloat16()

    def fused():
        return gate_up_swiglu_forward(x, wg, wu)

    def unfused():
        return swiglu_forward(x @ wg.t(), x @ wu.t())[0]

    for _ in range(3):
        fused(), unfused()
    check_status(device)
    times = {"fused": [], "unfused": []}
    for _ in range(reps):
        for name, fn in (("fused", fused), ("unfused", unfused)):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = fn()
            b.record()
            times[name].append((a, b))
            del out
    torch.cuda.synchronize(device)
    check_status(device)
    ms = {name: sum(a.elapsed_time(b) for a, b in evs) / len(evs) for name, evs in times.items()}
    burst, sustained, kind = measured_tensor_peaks()
    flops = 4.0 * m * n * k
    tf = flops / (ms["fused"] * 1e-3) / 1e12
    return {
        "workload": f"c4: X bf16 [{m}, {k}], W_gate/W_up bf16 [{n}, {k}], seed 3; h = silu(X Wg^T) * (X Wu^T)",
        "kernel": "swiglu_gemm_fwd (tcgen05 CTA pairs, SwiGLU epilogue)", "reps": reps,
        "ms": ms["fused"], "tflops": tf, "frac_of_bf16_burst": tf / burst, "frac_of_bf16_sustained": tf / sustained,
        "peaks": {"bf16_tflops": burst, "bf16_tflops_sustained": sustained, "source": kind},
        "cublas_x2_plus_swiglu_ms": ms["unfused"], "speedup_over_unfused": ms["unfused"] / ms["fused"],
        "timing": "alternating calls in one loop, one CUDA-event pair per call, mean",
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
    affinity0 = os.sched_getaffinity(0)
    placement = bind_host_near_gpu(local_rank)
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
    # no collector pause between the two launches of a step: the device would idle inside the step's events
    import gc

    gc.collect()
    gc.disable()
    barrier()
    mark0 = sampler.mark() if sampler else 0
    launches0 = _lib.launch_count()
    wall0 = time.perf_counter()
    for k in range(args.steps):
        restore()  # untimed: between the previous step's last event and this step's first
        step(evs[k])
    barrier()
    wall = time.perf_counter() - wall0
    gc.enable()
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
        # the ceiling: the same bytes over the same link with no kernel in between, every rank at once
        ceil_ms = copy_ceiling_ms((hg, hu, hd), outs, device, 32 << 20, args.e2e_steps, barrier)
        tc = torch.tensor([ceil_ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(tc, op=dist.ReduceOp.MAX)
        ceil_ms = tc.item()
        step_bytes = 3 * gate0.numel() * es
        e2e = {"value": tokens_total / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": step_bytes * world, "d2h_bytes_per_step": step_bytes * world,
               "steps": args.e2e_steps, "gpu_launches": e2e_launches,
               "copy_ceiling": {"value": tokens_total / (ceil_ms * 1e-3), "unit": UNIT, "ms_per_step": ceil_ms,
                                "gbs_per_direction_per_gpu": step_bytes / (ceil_ms * 1e-3) / 1e9,
                                "what": "the step's input bytes host-to-device and its output bytes device-to-host at "
                                        "the same time on two streams, plain 32 MiB asynchronous copies from/to the "
                                        "same pinned buffers, no kernel, all ranks at once (max over ranks)"},
               "frac_of_copy_ceiling": ceil_ms / e2e_ms,
               "gbs_per_direction_per_gpu": step_bytes / (e2e_ms * 1e-3) / 1e9,
               "host_placement": placement,
               "path": "swiglu_b200_host_fwd_bwd: pinned host gate/up/dh -> device workspace in row chunks, forward + "
                       "in-place backward per chunk, h/dgate/dup -> pinned host; copies of neighbouring chunks overlap "
                       "the kernels"}
        del ws, hg, hu, hd, outs
    os.sched_setaffinity(0, affinity0)

    if sampler:
        sampler.stop()

    # ---- strong scaling of c5 over the same ranks ------------------------------------------------
    strong = None
    if not args.no_strong_c5:
        from kernels.swiglu import swiglu_backward, swiglu_forward

        h_dev = dgate_dev = dup_dev = None
        del gate, up, gate0, up0, dh
        torch.cuda.empty_cache()
        strong = run_strong_c5(W, swiglu_forward, swiglu_backward, _lib.launch_count, device, rank, world,
                               dist if world > 1 else None, barrier, args.c5_steps)

    # ---- the fused projection (a tensor-core kernel: its own roofline), on rank 0 -----------------
    c4 = None
    if not args.no_c4:
        torch.cuda.empty_cache()
        if rank == 0:
            c4 = run_c4_fused_gemm(device, args.c4_reps)
        barrier()

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
                         "traffic": scaled_bwd_traffic(w, w.tokens),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch over 8192 "
                                           "rows x 14336 bf16, scaled by elements x element size",
                         "algorithmic_bytes": w.bytes_bwd()},
            "clocks": sampler.summary(mark0, mark1) if sampler else None,
            "e2e": e2e,
            "strong_c5": strong,
            "c4_fused_gemm": c4,
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

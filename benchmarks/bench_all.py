"""SwiGLU section of the kernel benchmark: GB/s, tokens/s and roofline fraction per configuration.

    python benchmarks/bench_all.py [--configs c1 c2 c3 ...] [--modes forward backward full]
                                   [--providers b200 b200-safe torch-eager] [--rep 50] [--warmup 20]
                                   [--save results.json]
    python -m torch.distributed.run --nproc-per-node G benchmarks/bench_all.py --configs c5 --strong

Takes the place of the reference's per-kernel sweep (kernels/swiglu/benchmarks/benchmark_swiglu.py:
providers x modes x shapes, CUDA-event timing with the two fastest and two slowest repetitions
dropped, :97-120) and of the empty benchmarks/bench_all.py the reference ships.  What it adds: every
row carries the algorithmic byte count (forward 3*N*s, backward 5*N*s, full 8*N*s bytes), the
achieved GB/s, its fraction of the measured HBM copy bandwidth of this pool and of the nominal
8 TB/s, and tokens/s.  Like the reference's sweep (:123-131) every row also carries the peak device
memory of one call (torch.cuda.max_memory_allocated after an untimed setup), and what the call
allocated on top of its inputs: the in-place backward is the reason the operator's default mode
needs less.

Providers
    b200         this library, in-place backward (the operator's default)
    b200-safe    this library, preserve_inputs=True
    b200-graph   the launches of b200-safe captured once in CUDA graphs and replayed (launch-bound small shapes)
    b200-packed  this library, packed gate|up layout
    b200-perseq  this library, one call per sequence of the variable-length batch (c3 configurations only)
    torch-eager  the PyTorch composite (torch_swiglu_reference + autograd) on the same GPU
    ref-triton-fast, ref-triton-safe, ref-triton-packed, ref-triton-geglu-tanh, ref-triton-geglu-erf
                 the reference's own Triton kernels (its swiglu_forward / swiglu_backward and the packed
                 twins, in-place and preserve_inputs), from the unmodified copy that
                 benchmarks/fetch_reference.py places under baseline/_ref; reported as unavailable when
                 the copy is absent or its JIT fails.  Same launch wrappers, same timing, same GPU.
    liger        Liger's LigerSiLUMulFunction (context only, as in the reference's sweep)
    geglu-tanh, geglu-erf   the sibling GeGLU operator of this library (in-place backward), same byte model

Configurations are the synthetic workloads of kernel_pocs_b200/workloads.py plus ragged variants
of the variable-length one: width 11009, and the same with the first token row sliced off so that
gate, up and dh all start 2 bytes past a 16-byte boundary (the freshly allocated forward output
does not, so the forward of that variant runs with mutually misaligned tensors).

With --strong under torchrun, each rank takes a contiguous block of the token rows (no collective
on the data path) and rank 0 reports aggregate tokens/s = tokens / max over ranks of the time.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import torch

from kernel_pocs_b200 import workloads as W

NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def hbm_peak():
    try:
        return float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def time_cuda(fn, setup, warmup: int, rep: int):
    """Per-repetition CUDA-event timing; ``setup`` runs untimed before each repetition.
    Returns (trimmed mean, median, min) in milliseconds."""
    for _ in range(warmup):
        setup()
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(rep):
        setup()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    trimmed = times[2:-2] if len(times) > 8 else times
    return sum(trimmed) / len(trimmed), times[len(times) // 2], times[0]


def time_back_to_back(fn, calls: int = 10, reps: int = 3):
    """Milliseconds per call with `calls` calls between ONE pair of events (best of `reps`): what a launch costs
    when the host is ahead of the device, as it is inside a training step.  Timed call by call, a kernel of a
    fifth of a millisecond also pays for the host's way through its Python wrapper while the device idles."""
    fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(calls):
            fn()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) / calls)
    return best


def peak_memory(fn, setup):
    """(peak bytes allocated during one call, bytes the call allocated beyond what was live before it)."""
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    setup()
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    fn()
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated()
    return peak, peak - before


def make_case(name: str, device, rank: int, world: int, strong: bool, max_rows: int = 0):
    """Returns (workload, gate, up, dh) for this rank."""
    base = name.split("+")[0]
    w = W.workloads()[base]
    variant = name.split("+")[1] if "+" in name else ""
    if variant in ("w11009", "w11009-off1"):
        w = W.Workload(name, w.tokens, 11009, w.dtype, w.seed, w.std, w.note + ", odd width 11009")
    if max_rows and w.tokens > max_rows:
        w = W.Workload(w.name, max_rows, w.width, w.dtype, w.seed, w.std, w.note + f", first {max_rows} token rows")
    lo, hi = W.row_shard(w.tokens, world, rank) if strong else (0, w.tokens)
    gate, up, dh = W.generate_rows(w, lo, hi, device)
    if variant == "w11009-off1":
        gate, up, dh = gate[1:], up[1:], dh[1:]  # contiguous, but 11009*s bytes past the allocation start
    return w, gate, up, dh


def clone_like(t: torch.Tensor) -> torch.Tensor:
    """A copy with the same misalignment of the first element relative to 16 bytes as ``t``."""
    es = t.element_size()
    shift = (t.data_ptr() % 16) // es
    buf = torch.empty(t.numel() + shift, dtype=t.dtype, device=t.device)
    out = buf[shift:].view(t.shape)
    out.copy_(t)
    return out


def reference_ops(op="swiglu"):
    """The reference's launch wrappers (Triton kernels underneath) from the copy under baseline/_ref."""
    try:
        import fetch_reference
    except ImportError:
        from benchmarks import fetch_reference
    return fetch_reference.load(op)


def unavailable_row(name, provider, exc):
    text = (str(exc).strip().splitlines() or [type(exc).__name__])[-1]
    return {"config": name, "provider": provider, "unavailable": f"{type(exc).__name__}: {text}"[:300]}


def run_case(name, args, device, rank, world):
    import kernels.swiglu as own_ops
    from kernels.swiglu import torch_swiglu_reference

    w, gate0, up0, dh = make_case(name, device, rank, world, args.strong, args.max_rows)
    rows, width = gate0.shape
    es = gate0.element_size()
    n = rows * width
    byte_model = {"forward": 3 * n * es, "backward": 5 * n * es, "full": 8 * n * es}
    out_rows = []
    for provider in args.providers:
        ops = own_ops
        if provider.startswith("ref-triton-"):
            try:
                ops = reference_ops("geglu" if provider.startswith("ref-triton-geglu-") else "swiglu")
            except Exception as exc:  # copy absent, or triton not importable
                out_rows.append(unavailable_row(name, provider, exc))
                continue
        packed = provider in ("b200-packed", "ref-triton-packed")
        preserve = provider in ("b200-safe", "ref-triton-safe")
        gate, up = clone_like(gate0), clone_like(up0)
        gate_up0 = torch.cat([gate0, up0], dim=-1) if packed else None
        gate_up = gate_up0.clone() if packed else None

        def restore():
            # untimed: undo the in-place backward, then stream dh once (read-only, larger than L2
            # for every configuration but c1) so the copies' dirty L2 lines are written back
            # before the timed kernels start
            if packed:
                gate_up.copy_(gate_up0)
            elif (provider in ("b200", "b200-perseq", "ref-triton-fast", "liger") or provider.startswith("geglu-")
                  or provider.startswith("ref-triton-geglu-")):
                gate.copy_(gate0)
                up.copy_(up0)
            else:
                return
            dh.sum()

        if provider == "torch-eager":
            g = gate0.clone().requires_grad_(True)
            u = up0.clone().requires_grad_(True)
            state = {}

            def fwd():
                state["h"] = torch_swiglu_reference(g, u)

            def bwd():
                torch.autograd.grad(state["h"], (g, u), dh)

            def full():
                fwd()
                bwd()
                state.clear()

            setups = {"forward": state.clear, "backward": fwd, "full": state.clear}
        elif provider == "liger":
            try:
                import importlib

                importlib.import_module("torch.distributed.tensor")  # liger looks the submodule up as an attribute
                from liger_kernel.ops.swiglu import LigerSiLUMulFunction
            except Exception as exc:
                out_rows.append(unavailable_row(name, provider, exc))
                continue
            state = {}
            g = gate.requires_grad_(True)
            u = up.requires_grad_(True)

            def fwd():
                state["h"] = LigerSiLUMulFunction.apply(g, u)

            def bwd():
                torch.autograd.grad(state["h"], (g, u), dh)

            def full():
                fwd()
                bwd()
                state.clear()

            def liger_restore():
                state.clear()
                with torch.no_grad():
                    restore()

            def liger_bwd_setup():
                liger_restore()
                fwd()

            setups = {"forward": liger_restore, "backward": liger_bwd_setup, "full": liger_restore}
        elif provider.startswith("geglu-") or provider.startswith("ref-triton-geglu-"):
            if provider.startswith("ref-triton-"):  # the reference's own Triton GeGLU, in-place backward
                geglu_backward, geglu_forward = ops.geglu_backward, ops.geglu_forward
            else:
                from kernels.geglu import geglu_backward, geglu_forward

            approximate = "tanh" if provider.endswith("-tanh") else "none"

            def fwd():
                geglu_forward(gate, up, approximate)

            def bwd():
                geglu_backward(dh, gate, up, approximate)

            def full():
                fwd()
                bwd()

            setups = {m: restore for m in ("forward", "backward", "full")}
        elif packed:
            def fwd():
                ops.swiglu_packed_forward(gate_up)

            def bwd():
                ops.swiglu_packed_backward(dh, gate_up, gate_up.shape, preserve_inputs=False)

            def full():
                fwd()
                bwd()

            setups = {m: restore for m in ("forward", "backward", "full")}
        elif provider == "b200-graph":
            # the same launches (preserve_inputs, so that a replay needs no restore) captured once in CUDA graphs
            # and replayed: what a launch-bound loop over small shapes gains
            def capture(step):
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    for _ in range(3):
                        step()
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step()
                return graph

            def both():
                own_ops.swiglu_forward(gate, up)
                own_ops.swiglu_backward(dh, gate, up, preserve_inputs=True)

            graphs = {"forward": capture(lambda: own_ops.swiglu_forward(gate, up)),
                      "backward": capture(lambda: own_ops.swiglu_backward(dh, gate, up, preserve_inputs=True)),
                      "full": capture(both)}
            fwd, bwd, full = graphs["forward"].replay, graphs["backward"].replay, graphs["full"].replay
            setups = {m: (lambda: None) for m in ("forward", "backward", "full")}
        elif provider == "b200-perseq":
            # one call per sequence of the variable-length batch (row slices of the packed token axis): what a
            # caller that walks cu_seqlens does; the op is row-independent, so the results are those of one call
            lens = W.varlen_lengths()
            if sum(lens) != rows:
                continue  # only the whole var-len batch (c3 and its variants, unsharded) has these boundaries
            bounds = [(sum(lens[:i]), sum(lens[:i + 1])) for i in range(len(lens))]

            def fwd():
                for a, b in bounds:
                    ops.swiglu_forward(gate[a:b], up[a:b])

            def bwd():
                for a, b in bounds:
                    ops.swiglu_backward(dh[a:b], gate[a:b], up[a:b])

            def full():
                fwd()
                bwd()

            setups = {m: restore for m in ("forward", "backward", "full")}
        else:
            def fwd():
                ops.swiglu_forward(gate, up)

            def bwd():
                ops.swiglu_backward(dh, gate, up, preserve_inputs=preserve)

            def full():
                fwd()
                bwd()

            setups = {m: restore for m in ("forward", "backward", "full")}

        fns = {"forward": fwd, "backward": bwd, "full": full}
        for mode in args.modes:
            try:
                mean, med, best = time_cuda(fns[mode], setups[mode], args.warmup, args.rep)
                peak_bytes, extra_bytes = peak_memory(fns[mode], setups[mode])
            except Exception as exc:
                if ops is own_ops and provider != "liger":
                    raise  # this library's own providers never fail quietly
                out_rows.append(unavailable_row(name, provider, exc))
                break
            t = torch.tensor([mean, med, best], dtype=torch.float64, device=device)
            if world > 1:
                import torch.distributed as dist

                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            mean, med, best = t.tolist()
            out_rows.append({
                "config": name, "provider": provider, "mode": mode, "dtype": str(w.dtype).split(".")[-1],
                "tokens_per_gpu": rows, "width": width, "gpus": world,
                "ms_mean_trimmed": mean, "ms_median": med, "ms_min": best,
                "algorithmic_bytes_per_gpu": byte_model[mode],
                "gbs_per_gpu": byte_model[mode] / (mean * 1e-3) / 1e9,
                "tokens_per_s": (w.tokens if args.strong else rows * world) / (mean * 1e-3),
                "peak_mib": peak_bytes / 2**20, "call_allocates_mib": extra_bytes / 2**20,
            })
        del gate, up, gate_up, gate_up0
        torch.cuda.empty_cache()
    return out_rows


C4 = {"m": 16384, "n": 14336, "k": 4096, "seed": 3}
FALLBACK_BF16_TFLOPS = 1590.0


def tensor_peak():
    try:
        d = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    except Exception:
        return FALLBACK_BF16_TFLOPS, 1400.0, "fallback"


def run_c4(args, device):
    """Fused gate/up projection + SwiGLU (benchmark configuration c4): X [16384, 4096] ~ N(0,1),
    W_gate, W_up [14336, 4096] ~ N(0, 0.02^2), bf16, seed 3; dh ~ N(0,1) for the backward.
    FLOPs: forward 4*M*N*K (two GEMMs), backward 8*M*N*K (dX: two GEMMs, dW_gate, dW_up)."""
    from kernel_pocs_b200.fused_mlp import check_status, fused_gate_up_swiglu, gate_up_swiglu_forward
    from kernels.swiglu import swiglu, swiglu_forward

    m = min(C4["m"], args.max_rows) if args.max_rows else C4["m"]
    n, k = C4["n"], C4["k"]
    g = torch.Generator(device=device).manual_seed(C4["seed"])
    x = torch.randn(m, k, generator=g, device=device).bfloat16()
    wg = (0.02 * torch.randn(n, k, generator=g, device=device)).bfloat16()
    wu = (0.02 * torch.randn(n, k, generator=g, device=device)).bfloat16()
    dh = torch.randn(m, n, generator=g, device=device).bfloat16()
    flops = {"forward": 4.0 * m * n * k, "full": 12.0 * m * n * k}
    xg, wgg, wug = (t.clone().requires_grad_(True) for t in (x, wg, wu))

    def fused_fwd():
        gate_up_swiglu_forward(x, wg, wu)

    def fused_full():
        h = fused_gate_up_swiglu(xg, wgg, wug)
        torch.autograd.grad(h, (xg, wgg, wug), dh)

    def unfused_fwd():
        swiglu_forward(x @ wg.t(), x @ wu.t())

    def unfused_full():
        h = swiglu(xg @ wgg.t(), xg @ wug.t())
        torch.autograd.grad(h, (xg, wgg, wug), dh)

    def cublas_fwd():
        x @ wg.t()
        x @ wu.t()

    burst, sustained, kind = tensor_peak()
    rows = []
    # the reference's own attempt at this fusion: its autotuned Triton dual GEMM (experiments/v2), without adapters
    ref_providers = ()
    try:
        ref_v2 = reference_ops("lora_v2")

        def ref_dual_gemm():
            ref_v2.fused_gate_up_swiglu(x, wg, None, None, 1.0, wu, None, None, 1.0)

        ref_dual_gemm()  # JIT and autotuning
        torch.cuda.synchronize()
        ref_providers = (("ref-triton-dual-gemm", {"forward": ref_dual_gemm}),)
    except Exception as exc:
        rows.append(unavailable_row("c4", "ref-triton-dual-gemm", exc))
        print(f"{'c4':>16} {'ref-triton-dual-gemm':>18} unavailable: {rows[-1]['unavailable']}", flush=True)
    for provider, fns in (("b200-fused-gemm", {"forward": fused_fwd, "full": fused_full}),
                          ("cublas+b200-swiglu", {"forward": unfused_fwd, "full": unfused_full}),
                          ("cublas-2gemm-only", {"forward": cublas_fwd}), *ref_providers):
        for mode, fn in fns.items():
            if mode not in args.modes:
                continue
            mean, med, best = time_cuda(fn, lambda: None, args.warmup, args.rep)
            check_status(device)
            r = {"config": "c4", "provider": provider, "mode": mode, "dtype": "bfloat16", "m": m, "n": n, "k": k,
                 "ms_mean_trimmed": mean, "ms_median": med, "ms_min": best, "flops": flops[mode],
                 "tflops": flops[mode] / (mean * 1e-3) / 1e12,
                 "frac_of_measured_bf16_burst": flops[mode] / (mean * 1e-3) / 1e12 / burst,
                 "tokens_per_s": m / (mean * 1e-3)}
            rows.append(r)
            print(f"{'c4':>16} {provider:>18} {mode:>8} bf16 M{m} N{n} K{k} {mean:9.4f} ms  {r['tflops']:8.1f} TFLOP/s  "
                  f"{100 * r['frac_of_measured_bf16_burst']:5.1f}% of {kind} cuBLAS burst {burst:.0f} "
                  f"({100 * r['tflops'] / 2250:4.1f}% of nominal 2250)  {r['tokens_per_s'] / 1e6:8.3f} Mtok/s", flush=True)
    return rows


def run_lora(args, device):
    """LoRA + SwiGLU epilogue on the c4 activation shape: E, G bf16 [16384, 14336], rank 16 adapters.
    Algorithmic bytes: read E and G, write h (3*M*N*2), plus e and g written back when saved for the backward
    (5*M*N*2); the rank-r operands are negligible.  Comparator: the unfused sequence the reference's fusion
    replaces, two in-place addmm_ (cuBLAS) followed by this library's SwiGLU kernel."""
    from kernel_pocs_b200.fused_mlp import check_status
    from kernel_pocs_b200.lora_mlp import fused_lora_swiglu
    from kernels.swiglu import swiglu_forward

    m = min(C4["m"], args.max_rows) if args.max_rows else C4["m"]
    n, r = C4["n"], 16
    g = torch.Generator(device=device).manual_seed(7)
    mk = lambda *shape, std=1.0: (std * torch.randn(*shape, generator=g, device=device)).bfloat16()
    e, gg, xag, xau, bg, bu = mk(m, n), mk(m, n), mk(m, r), mk(m, r), mk(n, r, std=0.3), mk(n, r, std=0.3)
    e2, g2 = e.clone(), gg.clone()
    peak, kind = hbm_peak()
    rows = []

    def fused():
        fused_lora_swiglu(e, gg, xag, xau, bg, bu, 2.0, 2.0)

    def fused_save():
        fused_lora_swiglu(e, gg, xag, xau, bg, bu, 2.0, 2.0, save_eg=True)

    def unfused():
        e2.addmm_(xag, bg.t(), alpha=2.0)
        g2.addmm_(xau, bu.t(), alpha=2.0)
        swiglu_forward(e2, g2)

    # backward elementwise step of the LoRA MLP: (dh, e, g) -> (h, de, dg) in place, 6*M*N*2 bytes, against
    # the two kernels that give the same three tensors (forward: 3 passes, backward in place: 5 passes)
    from kernel_pocs_b200.swiglu import swiglu_backward, swiglu_backward_recompute

    dh = mk(m, n)

    def recompute():
        swiglu_backward_recompute(dh, e2, g2)

    def fwd_then_bwd():
        swiglu_forward(e2, g2)
        swiglu_backward(dh, e2, g2)

    def reseed():
        # in-place results feed the next repetition; keep the values in the range of the first
        e2.copy_(e)
        g2.copy_(gg)

    # the reference's own Triton kernel for this step (experiments/v3, fused_lora_swiglu), when its copy is there
    try:
        ref_v3 = reference_ops("lora_v3")
        ref_v3.fused_lora_swiglu(e[:256], gg[:256], xag[:256], xau[:256], bg, bu, 2.0, 2.0)  # first JIT
        torch.cuda.synchronize()
        ref_rows = (
            ("ref-triton-lora-epilogue", lambda: ref_v3.fused_lora_swiglu(e, gg, xag, xau, bg, bu, 2.0, 2.0),
             3 * m * n * 2, "forward", lambda: None),
            ("ref-triton-lora-epilogue+save",
             lambda: ref_v3.fused_lora_swiglu(e, gg, xag, xau, bg, bu, 2.0, 2.0, save_eg=True),
             5 * m * n * 2, "forward", lambda: None))
    except Exception as exc:
        ref_rows = ()
        rows.append(unavailable_row("lora", "ref-triton-lora-epilogue", exc))
        print(f"{'lora':>16} {'ref-triton-lora-epilogue':>24} unavailable: {rows[-1]['unavailable']}", flush=True)

    for provider, fn, nbytes, mode, setup in (
            ("b200-lora-epilogue", fused, 3 * m * n * 2, "forward", lambda: None),
            ("b200-lora-epilogue+save", fused_save, 5 * m * n * 2, "forward", lambda: None),
            *ref_rows,
            ("addmm_x2+b200-swiglu", unfused, 3 * m * n * 2, "forward", lambda: None),
            ("b200-bwd-recompute", recompute, 6 * m * n * 2, "backward", reseed),
            ("b200-fwd+b200-bwd", fwd_then_bwd, 8 * m * n * 2, "backward", reseed)):
        mean, med, best = time_cuda(fn, setup, args.warmup, args.rep)
        check_status(device)
        r_ = {"config": "lora", "provider": provider, "mode": mode, "dtype": "bfloat16", "m": m, "n": n, "r": r,
              "ms_mean_trimmed": mean, "ms_median": med, "ms_min": best, "algorithmic_bytes_per_gpu": nbytes,
              "gbs_per_gpu": nbytes / (mean * 1e-3) / 1e9, "tokens_per_s": m / (mean * 1e-3)}
        r_["frac_of_measured_copy"] = r_["gbs_per_gpu"] / peak
        rows.append(r_)
        print(f"{'lora':>16} {provider:>24} {mode:>8} bf16 M{m} N{n} r{r} {mean:9.4f} ms  {r_['gbs_per_gpu']:8.1f} GB/s  "
              f"{100 * r_['frac_of_measured_copy']:6.1f}% of {kind} {peak:.0f}  {r_['tokens_per_s'] / 1e6:8.3f} Mtok/s", flush=True)
        if "lora-epilogue" in provider:
            ms = time_back_to_back(fn)
            check_status(device)
            r_["ms_back_to_back"] = ms
            r_["gbs_back_to_back"] = nbytes / (ms * 1e-3) / 1e9
            r_["frac_of_measured_copy_back_to_back"] = r_["gbs_back_to_back"] / peak
            print(f"{'':>16} {'ten calls back to back':>24} {mode:>8} bf16 M{m} N{n} r{r} {ms:9.4f} ms  "
                  f"{r_['gbs_back_to_back']:8.1f} GB/s  {100 * r_['frac_of_measured_copy_back_to_back']:6.1f}% of {kind} {peak:.0f}",
                  flush=True)
    # the whole gate/up stage of a LoRA MLP from X: one launch (projections + adapters + SwiGLU) against two
    # cuBLAS GEMMs, two skinny GEMMs and the epilogue kernel above
    from kernel_pocs_b200.fused_mlp import lora_gate_up_swiglu_forward

    k = C4["k"]
    x = mk(m, k)
    wg, wu = mk(n, k, std=0.02), mk(n, k, std=0.02)
    ag, au = mk(r, k, std=0.02), mk(r, k, std=0.02)
    burst, _, kind_t = tensor_peak()

    def one_launch():
        lora_gate_up_swiglu_forward(x, wg, wu, ag, bg, 2.0, au, bu, 2.0)

    def gemms_then_epilogue():
        fused_lora_swiglu(x @ wg.t(), x @ wu.t(), x @ ag.t(), x @ au.t(), bg, bu, 2.0, 2.0)

    flops = 4.0 * m * n * k
    for provider, fn in (("b200-lora-gemm-1-launch", one_launch), ("cublas-x2+b200-lora-epilogue", gemms_then_epilogue)):
        mean, med, best = time_cuda(fn, lambda: None, args.warmup, args.rep)
        check_status(device)
        r_ = {"config": "lora", "provider": provider, "mode": "forward-from-x", "dtype": "bfloat16", "m": m, "n": n,
              "k": k, "r": r, "ms_mean_trimmed": mean, "ms_median": med, "ms_min": best, "flops": flops,
              "tflops": flops / (mean * 1e-3) / 1e12, "tokens_per_s": m / (mean * 1e-3)}
        r_["frac_of_measured_bf16_burst"] = r_["tflops"] / burst
        rows.append(r_)
        print(f"{'lora':>16} {provider:>28} from-x bf16 M{m} N{n} K{k} r{r} {mean:9.4f} ms  {r_['tflops']:8.1f} TFLOP/s  "
              f"{100 * r_['frac_of_measured_bf16_burst']:5.1f}% of {kind_t} cuBLAS burst {burst:.0f}  "
              f"{r_['tokens_per_s'] / 1e6:8.3f} Mtok/s", flush=True)
    # whole LoRA MLP, forward + backward (gradients for X and the six adapter matrices, base weights frozen):
    # this library's LoRAMLP against the same block written with PyTorch operators under autograd
    from kernel_pocs_b200.lora_mlp import LoRAMLP

    wd = mk(k, n, std=0.02)
    ad, bd = mk(r, n, std=0.02), mk(k, r, std=0.3)
    dy = mk(m, k)
    train = [t.clone().requires_grad_(True) for t in (x, ag, bg, au, bu, ad, bd)]

    def own_mlp():
        xx, a1, b1, a2, b2, a3, b3 = train
        y = LoRAMLP.apply(xx, wg, a1, b1, 2.0, wu, a2, b2, 2.0, wd, a3, b3, 2.0)
        torch.autograd.grad(y, train, dy)

    def torch_mlp():
        xx, a1, b1, a2, b2, a3, b3 = train
        proj = lambda t, w, a, b_: torch.addmm(t @ w.t(), t @ a.t(), b_.t(), alpha=2.0)
        y = proj(torch.nn.functional.silu(proj(xx, wg, a1, b1)) * proj(xx, wu, a2, b2), wd, a3, b3)
        torch.autograd.grad(y, train, dy)

    for provider, fn in (("b200-lora-mlp", own_mlp), ("torch-autograd-lora-mlp", torch_mlp)):
        mean, med, best = time_cuda(fn, lambda: None, max(2, args.warmup // 2), max(5, args.rep // 2))
        check_status(device)
        r_ = {"config": "lora", "provider": provider, "mode": "mlp-fwd+bwd", "dtype": "bfloat16", "m": m, "n": n, "k": k,
              "r": r, "ms_mean_trimmed": mean, "ms_median": med, "ms_min": best, "tokens_per_s": m / (mean * 1e-3)}
        rows.append(r_)
        print(f"{'lora':>16} {provider:>28} mlp fwd+bwd bf16 M{m} N{n} K{k} r{r} {mean:9.4f} ms  "
              f"{r_['tokens_per_s'] / 1e6:8.3f} Mtok/s", flush=True)
    return rows


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--configs", nargs="+", default=["c1", "c2", "c3", "c3-fp32", "c3+w11009", "c3+w11009-off1"])
    ap.add_argument("--providers", nargs="+", default=["b200", "b200-safe", "ref-triton-fast", "torch-eager"],
                    choices=["b200", "b200-safe", "b200-graph", "b200-packed", "b200-perseq", "torch-eager", "geglu-tanh", "geglu-erf",
                             "ref-triton-fast", "ref-triton-safe", "ref-triton-packed", "ref-triton-geglu-tanh",
                             "ref-triton-geglu-erf", "liger"])
    ap.add_argument("--modes", nargs="+", default=["forward", "backward", "full"],
                    choices=["forward", "backward", "full"])
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--rep", type=int, default=50)
    ap.add_argument("--strong", action="store_true", help="split each configuration's token rows across the ranks")
    ap.add_argument("--max-rows", type=int, default=0,
                    help="cap the token rows of every configuration (small cases for profiler captures)")
    ap.add_argument("--save", default="")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("CUDA is required: the SwiGLU path has no CPU fallback")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    peak, kind = hbm_peak()
    rows = []
    for name in args.configs:
        if name == "c4":
            if world == 1:
                rows.extend(run_c4(args, device))
            continue
        if name == "lora":
            if world == 1:
                rows.extend(run_lora(args, device))
            continue
        for r in run_case(name, args, device, rank, world):
            if "unavailable" in r:
                rows.append(r)
                if rank == 0:
                    print(f"{r['config']:>16} {r['provider']:>17} unavailable: {r['unavailable']}", flush=True)
                continue
            r["frac_of_measured_copy"] = r["gbs_per_gpu"] / peak
            r["frac_of_nominal_8TBs"] = r["gbs_per_gpu"] / NOMINAL_HBM_GBS
            rows.append(r)
            if rank == 0:
                print(f"{r['config']:>16} {r['provider']:>17} {r['mode']:>8} {r['dtype']:>8} "
                      f"{r['ms_mean_trimmed']:9.4f} ms  {r['gbs_per_gpu']:8.1f} GB/s/GPU  "
                      f"{100 * r['frac_of_measured_copy']:6.1f}% of {kind} {peak:.0f}  "
                      f"{100 * r['frac_of_nominal_8TBs']:5.1f}% of 8000  {r['tokens_per_s'] / 1e6:9.3f} Mtok/s "
                      f"x{world}  peak {r['peak_mib']:8.0f} MiB (+{r['call_allocates_mib']:.0f})", flush=True)
    if rank == 0 and args.save:
        Path(args.save).parent.mkdir(parents=True, exist_ok=True)
        Path(args.save).write_text(json.dumps({"hbm_peak_gbs": peak, "hbm_peak_kind": kind, "rows": rows}, indent=1))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Fused gate/up projection + SwiGLU epilogue (tcgen05 kernel) against a PyTorch fp32 reference.

This is a floating-point contraction, so the comparator is plain PyTorch in fp32 on the same bf16
operands: g = x @ w_gate.T, u = x @ w_up.T (fp32 accumulation, TF32 off), h = silu(g*gm) * u * dm.
The kernel accumulates in fp32 in a different order and rounds once to bf16, so the bound is one
bf16 rounding plus accumulation noise:  |h - ref| <= 2^-7 * |ref| + 2^-9 * rms(ref).
The optional pre-activation outputs must be the bf16 rounding of g and u to the same bound, and the
epilogue must agree with the CPU oracle applied to those pre-activations.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from kernel_pocs_b200 import _lib
from kernel_pocs_b200 import fused_mlp as F
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
DEVICE = "cuda"


def reference(x, wg, wu, gm=1.0, dm=1.0):
    g = x.float() @ wg.float().t()
    u = x.float() @ wu.float().t()
    return torch.nn.functional.silu(g * gm) * u * dm, g, u


def assert_close_bf16(got, ref, what):
    ref = ref.float()
    tol = 2.0 ** -7 * ref.abs() + 2.0 ** -9 * ref.pow(2).mean().sqrt()
    err = (got.float() - ref).abs()
    bad = err > tol
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} of {bad.numel()} outside tolerance, worst {float((err / tol).max()):.2f}x"


def make(m, n, k, seed=3, w_std=0.05):
    g = torch.Generator(device=DEVICE).manual_seed(seed)
    x = torch.randn(m, k, generator=g, device=DEVICE).bfloat16()
    wg = (w_std * torch.randn(n, k, generator=g, device=DEVICE)).bfloat16()
    wu = (w_std * torch.randn(n, k, generator=g, device=DEVICE)).bfloat16()
    return x, wg, wu


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 64), (256, 128, 64), (1, 16, 8), (7, 48, 24), (200, 144, 72), (257, 272, 200),
    (384, 1024, 512), (1000, 2064, 1032), (2048, 1408, 4096), (4500, 384, 256),
])
@pytest.mark.parametrize("gm,dm", [(1.0, 1.0), (0.7, 1.3)])
def test_forward_matches_fp32_reference(m, n, k, gm, dm):
    x, wg, wu = make(m, n, k)
    before = _lib.lib.swiglu_b200_gemm_launch_count()
    h, gate, up = F.gate_up_swiglu_forward(x, wg, wu, gm, dm, save_preactivations=True)
    F.check_status(x.device)
    assert _lib.lib.swiglu_b200_gemm_launch_count() == before + 1
    ref_h, ref_g, ref_u = reference(x, wg, wu, gm, dm)
    assert h.shape == (m, n) and h.dtype == torch.bfloat16
    assert_close_bf16(gate, ref_g, "gate pre-activation")
    assert_close_bf16(up, ref_u, "up pre-activation")
    assert_close_bf16(h, ref_h, "h")
    # the epilogue is the SwiGLU forward of the fp32 accumulators; from the bf16-rounded pre-activations the
    # CPU oracle must land within 2 bf16 ulp of it almost everywhere (the kernel rounds h from unrounded g, u)
    oh = O.fwd(gate.cpu(), up.cpu(), gm, dm, "once")
    d = O.ulp_distance(h.cpu(), oh)
    assert float((d > 4).double().mean()) < 0.02
    # without the optional outputs the result is bit-identical
    h2 = F.gate_up_swiglu_forward(x, wg, wu, gm, dm)
    F.check_status(x.device)
    assert torch.equal(h, h2)


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (1, 16, 8), (300, 272, 200), (257, 528, 72), (1000, 2064, 1032),
                                   (2048, 1408, 4096), (4500, 384, 256)])
@pytest.mark.parametrize("gm,dm", [(1.0, 1.0), (0.7, 1.3)])
@pytest.mark.parametrize("tile", ["wide", "staggered"])
def test_wide_tile_kernels_agree_with_the_narrow_one(m, n, k, gm, dm, tile, monkeypatch):
    """The two 256 x 256 pair-tile kernels, forced on small and ragged shapes (SWIGLU_B200_GEMM_TILE): `wide`
    (two MMAs per step sharing the X operand, one 512-column accumulator, sixteen epilogue warps) and `staggered`
    (two 256 x 128 streams a few K blocks apart, each issued by its own thread, sharing a ring of X tiles; the
    default where a problem has a tile per resident cluster).  Each output element is accumulated over K in the
    same order by all three kernels, so the bits must agree; the fp32 reference bounds them."""
    x, wg, wu = make(m, n, k, seed=11)
    monkeypatch.setenv("SWIGLU_B200_GEMM_TILE", "narrow")
    want = F.gate_up_swiglu_forward(x, wg, wu, gm, dm, save_preactivations=True)
    monkeypatch.setenv("SWIGLU_B200_GEMM_TILE", tile)
    before = _lib.lib.swiglu_b200_gemm_launch_count()
    got = F.gate_up_swiglu_forward(x, wg, wu, gm, dm, save_preactivations=True)
    F.check_status(x.device)
    assert _lib.lib.swiglu_b200_gemm_launch_count() == before + 1
    for a, b, what in zip(got, want, ("h", "gate", "up")):
        assert torch.equal(a, b), what
    ref_h, ref_g, ref_u = reference(x, wg, wu, gm, dm)
    assert_close_bf16(got[0], ref_h, "h")
    assert_close_bf16(got[1], ref_g, "gate pre-activation")
    h_only = F.gate_up_swiglu_forward(x, wg, wu, gm, dm)
    F.check_status(x.device)
    assert torch.equal(h_only, got[0])


@pytest.mark.parametrize("r", [8, 16, 40, 64])
@pytest.mark.parametrize("activation", ["silu", "gelu_tanh", "gelu_exact"])
@pytest.mark.parametrize("wide", ["wide", "staggered"])
def test_wide_tile_kernels_with_adapters_and_gelu(r, activation, wide, monkeypatch):
    m, n, k = 520, 784, 328
    g = torch.Generator(device=DEVICE).manual_seed(r)
    mk = lambda *s, std=1.0: (std * torch.randn(*s, generator=g, device=DEVICE)).bfloat16()
    x, wg, wu = mk(m, k), mk(n, k, std=k ** -0.5), mk(n, k, std=k ** -0.5)
    ag, au, bg, bu = mk(r, k, std=k ** -0.5), mk(r, k, std=k ** -0.5), mk(n, r, std=0.3), mk(n, r, std=0.3)
    outs = {}
    for tile in ("narrow", wide):
        monkeypatch.setenv("SWIGLU_B200_GEMM_TILE", tile)
        outs["wide" if tile == wide else tile] = F.lora_gate_up_swiglu_forward(x, wg, wu, ag, bg, 2.0, au, bu, 0.5, save_eg=True,
                                                   activation=activation)
        F.check_status(x.device)
    for a, b, what in zip(outs["wide"], outs["narrow"], ("h", "e", "g")):
        assert torch.equal(a, b), what
    e_ref = x.float() @ wg.float().t() + (x @ (ag * 2.0).t()).float() @ bg.float().t()
    g_ref = x.float() @ wu.float().t() + (x @ (au * 0.5).t()).float() @ bu.float().t()
    assert_close_bf16(outs["wide"][1], e_ref, "e")
    assert_close_bf16(outs["wide"][2], g_ref, "g")
    act = {"silu": torch.nn.functional.silu, "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
           "gelu_exact": torch.nn.functional.gelu}[activation]
    assert_close_bf16(outs["wide"][0], act(e_ref) * g_ref, "h")


def test_leading_dimensions_and_errors():
    x, wg, wu = make(6 * 20, 64, 32)
    h = F.gate_up_swiglu_forward(x.view(6, 20, 32), wg, wu)
    assert h.shape == (6, 20, 64)
    with pytest.raises(ValueError, match="features"):
        F.gate_up_swiglu_forward(x[:, :16].contiguous(), wg, wu)
    with pytest.raises(ValueError, match="k % 8"):
        F.gate_up_swiglu_forward(x[:, :20].contiguous(), wg[:, :20].contiguous(), wu[:, :20].contiguous())
    with pytest.raises(TypeError, match="bf16"):
        F.gate_up_swiglu_forward(x.float(), wg.float(), wu.float())
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        F.gate_up_swiglu_forward(x.cpu(), wg.cpu(), wu.cpu())
    c = _lib.lib.swiglu_b200_gemm_fwd
    p = h.data_ptr()
    st = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    assert c(p, None, None, x.data_ptr(), wg.data_ptr(), wu.data_ptr(), 4, 64, 20, 1.0, 1.0, st.data_ptr(), 0, None) == 3
    assert c(p, p, None, x.data_ptr(), wg.data_ptr(), wu.data_ptr(), 4, 64, 32, 1.0, 1.0, st.data_ptr(), 0, None) == 2
    assert c(p, None, None, x.data_ptr(), wg.data_ptr(), wu.data_ptr(), 4, 64, 32, 1.0, 1.0, None, 0, None) == 2
    assert c(p, None, None, x.data_ptr(), wg.data_ptr(), wu.data_ptr(), 0, 64, 32, 1.0, 1.0, st.data_ptr(), 0, None) == 0
    F.check_status(x.device)


def test_autograd_matches_reference():
    m, n, k = 512, 768, 256
    x, wg, wu = make(m, n, k, seed=9)
    dh = torch.randn(m, n, device=DEVICE).bfloat16()
    xs = [t.clone().requires_grad_(True) for t in (x, wg, wu)]
    h = F.fused_gate_up_swiglu(*xs, 0.9, 1.1)
    dx, dwg, dwu = torch.autograd.grad(h, xs, dh)
    F.check_status(x.device)
    rs = [t.float().clone().requires_grad_(True) for t in (x, wg, wu)]
    g = rs[0] @ rs[1].t()
    u = rs[0] @ rs[2].t()
    rh = torch.nn.functional.silu(g * 0.9) * u * 1.1
    rdx, rdwg, rdwu = torch.autograd.grad(rh, rs, dh.float())
    assert_close_bf16(h, rh.detach(), "h")
    # gradients go through bf16 dgate/dup and bf16 GEMMs: bound them by the spread of the reference
    for got, ref, what in ((dx, rdx, "dx"), (dwg, rdwg, "dw_gate"), (dwu, rdwu, "dw_up")):
        assert got.dtype == torch.bfloat16 and got.shape == ref.shape
        err = (got.float() - ref).abs()
        assert float(err.max()) <= 0.03 * float(ref.abs().max()), what
        assert float(err.pow(2).mean().sqrt()) <= 0.01 * float(ref.pow(2).mean().sqrt()), what


def test_single_cta_kernel_variant_agrees():
    """The one-CTA-per-tile kernel (selected by SWIGLU_B200_GEMM=single at process start) must give the
    same bits as the CTA-pair kernel: both accumulate each output over K in the same order."""
    code = (
        "import sys, torch; sys.path.insert(0, %r)\n"
        "from kernel_pocs_b200 import fused_mlp as F\n"
        "g = torch.Generator(device='cuda').manual_seed(3)\n"
        "x = torch.randn(300, 200, generator=g, device='cuda').bfloat16()\n"
        "wg = (0.05 * torch.randn(272, 200, generator=g, device='cuda')).bfloat16()\n"
        "wu = (0.05 * torch.randn(272, 200, generator=g, device='cuda')).bfloat16()\n"
        "h = F.gate_up_swiglu_forward(x, wg, wu, 0.7, 1.3); F.check_status(x.device)\n"
        "torch.save(h.cpu(), sys.argv[1])\n" % str(ROOT)
    )
    outs = []
    for variant in ("single", "pair"):
        path = f"/tmp/swiglu_gemm_{variant}_{os.getpid()}.pt"
        env = dict(os.environ, SWIGLU_B200_GEMM=variant)
        subprocess.run([sys.executable, "-c", code, path], check=True, env=env, timeout=300)
        outs.append(torch.load(path))
        os.unlink(path)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("tile", ["auto", "256", "512"])
@pytest.mark.parametrize("m,n,k", [(256, 128, 256), (512, 256, 512), (300, 136, 80), (1000, 2064, 1040),
                                   (4096, 1408, 1024), (8192, 1024, 2048),
                                   (6400, 3456, 1536)])  # the last: 75 and 81 wide tiles, so the tail of the
                                                         # last wave is handed out as 256-column halves
def test_backward_gemms_match_fp32_reference(m, n, k, tile, monkeypatch):
    """dx, dw_gate, dw_up from the tcgen05 backward kernels (operands whose contiguous dimension is not the
    contraction dimension, i.e. MN-major shared-memory descriptors) against fp32 matmuls of the same bf16
    operands; one bf16 rounding plus accumulation noise relative to the spread of the result.  Both tile
    widths (256 columns with two accumulators, 512 columns with one) are forced in turn, besides the
    library's own choice."""
    if tile == "auto":
        monkeypatch.delenv("SWIGLU_B200_GEMM_BWD_TILE", raising=False)
    else:
        monkeypatch.setenv("SWIGLU_B200_GEMM_BWD_TILE", tile)
    g = torch.Generator(device=DEVICE).manual_seed(5)
    x = torch.randn(m, k, generator=g, device=DEVICE).bfloat16()
    wg = (0.05 * torch.randn(n, k, generator=g, device=DEVICE)).bfloat16()
    wu = (0.05 * torch.randn(n, k, generator=g, device=DEVICE)).bfloat16()
    dgate = torch.randn(m, n, generator=g, device=DEVICE).bfloat16()
    dup = torch.randn(m, n, generator=g, device=DEVICE).bfloat16()
    before = _lib.lib.swiglu_b200_gemm_bwd_launch_count()
    dx, dwg, dwu = F.gate_up_swiglu_backward_gemms(dgate, dup, x, wg, wu)
    F.check_status(x.device)
    assert _lib.lib.swiglu_b200_gemm_bwd_launch_count() == before + 2
    assert_close_bf16(dx, dgate.float() @ wg.float() + dup.float() @ wu.float(), "dx")
    assert_close_bf16(dwg, dgate.float().t() @ x.float(), "dw_gate")
    assert_close_bf16(dwu, dup.float().t() @ x.float(), "dw_up")
    # either half on its own
    dx2, none_g, none_u = F.gate_up_swiglu_backward_gemms(dgate, dup, x, wg, wu, need_dw=False)
    assert none_g is None and none_u is None and torch.equal(dx2, dx)
    none_x, dwg2, dwu2 = F.gate_up_swiglu_backward_gemms(dgate, dup, x, wg, wu, need_dx=False)
    F.check_status(x.device)
    assert none_x is None and torch.equal(dwg2, dwg) and torch.equal(dwu2, dwu)


def test_full_size_projection_workload():
    """Benchmark configuration c4 at its FULL size: X bf16 [16384, 4096] ~ N(0,1), W_gate and W_up bf16
    [14336, 4096] ~ N(0, 0.02^2) (seed 3), dh ~ N(0,1).  Sixty-four sampled token rows (first, last and tile
    edges among them) of h, of both pre-activations and of dX over ALL their columns, and sixty-four sampled
    rows of dW_gate and dW_up over all theirs, against fp32 matmuls of the same bf16 operands; then the
    autograd wrapper must reproduce the step-by-step results bit for bit."""
    from kernels.swiglu import swiglu_backward

    m, n, k = 16384, 14336, 4096
    g = torch.Generator(device=DEVICE).manual_seed(3)
    x = torch.randn(m, k, generator=g, device=DEVICE).bfloat16()
    wg = (0.02 * torch.randn(n, k, generator=g, device=DEVICE)).bfloat16()
    wu = (0.02 * torch.randn(n, k, generator=g, device=DEVICE)).bfloat16()
    dh = torch.randn(m, n, generator=g, device=DEVICE).bfloat16()
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        pick = torch.Generator().manual_seed(33)
        rows = torch.cat([torch.tensor([0, 1, 127, 128, 255, 256, m - 257, m - 256, m - 2, m - 1]),
                          torch.randint(0, m, (54,), generator=pick)]).to(DEVICE)
        cols = torch.cat([torch.tensor([0, 1, 127, 128, 255, 256, n - 257, n - 256, n - 2, n - 1]),
                          torch.randint(0, n, (54,), generator=pick)]).to(DEVICE)
        h, gate, up = F.gate_up_swiglu_forward(x, wg, wu, save_preactivations=True)
        F.check_status(x.device)
        xr = x[rows].float()
        g_ref, u_ref = xr @ wg.float().t(), xr @ wu.float().t()
        assert_close_bf16(gate[rows], g_ref, "gate pre-activation rows")
        assert_close_bf16(up[rows], u_ref, "up pre-activation rows")
        assert_close_bf16(h[rows], torch.nn.functional.silu(g_ref) * u_ref, "h rows")
        del g_ref, u_ref
        h_keep = h[rows].clone()
        # the activation backward on the saved pre-activations (in place: they become dgate, dup), then the GEMMs
        dgate, dup = swiglu_backward(dh, gate, up)
        dx, dwg, dwu = F.gate_up_swiglu_backward_gemms(dgate, dup, x, wg, wu)
        F.check_status(x.device)
        assert_close_bf16(dx[rows], dgate[rows].float() @ wg.float() + dup[rows].float() @ wu.float(), "dx rows")
        xf = x.float()
        assert_close_bf16(dwg[cols], dgate[:, cols].float().t() @ xf, "dw_gate rows")
        assert_close_bf16(dwu[cols], dup[:, cols].float().t() @ xf, "dw_up rows")
        del xf, dgate, dup, gate, up, h
        # the same through autograd
        leaves = [t.clone().requires_grad_(True) for t in (x, wg, wu)]
        h2 = F.fused_gate_up_swiglu(*leaves)
        dx2, dwg2, dwu2 = torch.autograd.grad(h2, leaves, dh)
        F.check_status(x.device)
        assert torch.equal(h2[rows], h_keep)
        assert torch.equal(dx2, dx) and torch.equal(dwg2, dwg) and torch.equal(dwu2, dwu)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_tensor_core_kernels_on_random_shapes():
    """Forward projection (plain, with adapters, with a GELU gate) and both backward GEMMs on 48 seeded random
    shapes: ragged row counts, widths that end inside a tile, contractions that end inside a K block, every rank
    layout of the adapter steps, both backward tile widths, and the forward by its default choice of kernel, by
    the staggered two-stream kernel and by the 256 x 128 one in turn."""
    import os
    import random

    from kernel_pocs_b200.geglu import gate_up_geglu_forward

    rng = random.Random(20240607)
    g = torch.Generator(device=DEVICE).manual_seed(77)
    mk = lambda *s, std=1.0: (std * torch.randn(*s, generator=g, device=DEVICE)).bfloat16()
    saved = os.environ.get("SWIGLU_B200_GEMM_BWD_TILE")
    saved_fwd = os.environ.get("SWIGLU_B200_GEMM_TILE")
    try:
        for case in range(48):
            forward_tile = (None, "staggered", "narrow")[case % 3]
            if forward_tile is None:
                os.environ.pop("SWIGLU_B200_GEMM_TILE", None)
            else:
                os.environ["SWIGLU_B200_GEMM_TILE"] = forward_tile
            m = rng.choice([1, 7, 127, 128, 129, 255, 257, 300, 511, 777, 1024, 1500])
            n = 16 * rng.randint(1, 75)
            k = 16 * rng.randint(1, 50)
            r = rng.choice([0, 8, 16, 24, 32, 40, 48, 56, 64])
            what = f"case {case}: m={m} n={n} k={k} r={r}"
            x, wg, wu = mk(m, k), mk(n, k, std=k ** -0.5), mk(n, k, std=k ** -0.5)
            xf, wgf, wuf = x.float(), wg.float(), wu.float()
            e_ref, u_ref = xf @ wgf.t(), xf @ wuf.t()
            if r:
                ag, au, bg, bu = mk(r, k, std=k ** -0.5), mk(r, k, std=k ** -0.5), mk(n, r, std=0.3), mk(n, r, std=0.3)
                h, e, u = F.lora_gate_up_swiglu_forward(x, wg, wu, ag, bg, 2.0, au, bu, 0.5, save_eg=True)
                e_ref = e_ref + (x @ (ag * 2.0).t()).float() @ bg.float().t()
                u_ref = u_ref + (x @ (au * 0.5).t()).float() @ bu.float().t()
            else:
                h, e, u = F.gate_up_swiglu_forward(x, wg, wu, save_preactivations=True)
            F.check_status(x.device)
            assert_close_bf16(e, e_ref, what + " gate")
            assert_close_bf16(u, u_ref, what + " up")
            assert_close_bf16(h, torch.nn.functional.silu(e_ref) * u_ref, what + " h")
            if case % 3 == 0:
                approximate = "tanh" if case % 2 else "none"
                hg = gate_up_geglu_forward(x, wg, wu, approximate)
                F.check_status(x.device)
                assert_close_bf16(hg, torch.nn.functional.gelu(xf @ wgf.t(), approximate=approximate) * (xf @ wuf.t()),
                                  what + " geglu h")
            dgate, dup = mk(m, n), mk(m, n)
            os.environ["SWIGLU_B200_GEMM_BWD_TILE"] = ("256", "512")[case % 2]
            dx, dwg, dwu = F.gate_up_swiglu_backward_gemms(dgate, dup, x, wg, wu)
            F.check_status(x.device)
            assert_close_bf16(dx, dgate.float() @ wgf + dup.float() @ wuf, what + " dx")
            assert_close_bf16(dwg, dgate.float().t() @ xf, what + " dw_gate")
            assert_close_bf16(dwu, dup.float().t() @ xf, what + " dw_up")
    finally:
        for name, value in (("SWIGLU_B200_GEMM_BWD_TILE", saved), ("SWIGLU_B200_GEMM_TILE", saved_fwd)):
            if value is None:
                os.environ.pop(name, None)
            else:
                os.environ[name] = value


def test_status_ring_reports_a_failed_launch():
    """A kernel that gives up on a wait leaves a code in its status word.  Made on the host here (the word is
    filled by hand after a good launch; no kernel is made to fail): the code must surface as a RuntimeError
    within one turn of the ring, once, and an explicit check afterwards must be clean."""
    x, wg, wu = make(256, 128, 64)
    F.gate_up_swiglu_forward(x, wg, wu)
    F.check_status(x.device)
    word = F._status(x.device)           # a word of the ring, as a launch would get it
    word.fill_(321)
    with pytest.raises(RuntimeError, match="code 321"):
        for _ in range(F._StatusRing.SLOTS + 1):
            F.gate_up_swiglu_forward(x, wg, wu)
    F.check_status(x.device)              # reported once: nothing is left behind
    for _ in range(2 * F._StatusRing.SLOTS):
        h = F.gate_up_swiglu_forward(x, wg, wu)
    F.check_status(x.device)
    assert bool(torch.isfinite(h).all())
    # the explicit check sees a code at once
    F._status(x.device).fill_(77)
    with pytest.raises(RuntimeError, match="code 77"):
        F.check_status(x.device)
    F.check_status(x.device)


def test_status_ring_keeps_a_code_whose_half_was_already_copied():
    """The window between the copy of a half of the ring and the reuse of its words: a code that sits in a
    half when that half is sent to the host must still be found by an explicit check made before the ring
    comes back to it, and by the ring itself when it does; a reused word must not hide it."""
    x, wg, wu = make(256, 128, 64)
    F.check_status(x.device)
    ring = F._ring(x.device)
    half = F._StatusRing.HALF
    # walk to the start of a half so that the scenario below is the same wherever the ring stood
    while ring.next % half:
        F.gate_up_swiglu_forward(x, wg, wu)
    F._status(x.device).fill_(555)                     # first word of this half
    for _ in range(half):                              # the rest of this half and the first launch of the other:
        F.gate_up_swiglu_forward(x, wg, wu)            # the half with the code is now on its way to the host
    first = ring.next // half
    assert ring.pending[1 - first] is not None
    with pytest.raises(RuntimeError, match="code 555"):
        F.check_status(x.device)
    F.check_status(x.device)
    # same again, but let the ring find it: launches on a side stream, so the copy has to wait for that stream
    side = torch.cuda.Stream()
    while ring.next % half:
        F.gate_up_swiglu_forward(x, wg, wu)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        F.selftest_wait_timeout(x.device, 0, 200_000, 556)   # a real kernel leaves the code, on the side stream
    with pytest.raises(RuntimeError, match="code 556"):
        for _ in range(F._StatusRing.SLOTS):
            F.gate_up_swiglu_forward(x, wg, wu)
    F.check_status(x.device)


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
def test_bounded_wait_runs_out_and_reports(mode):
    """The failure path of the tensor-core kernels on a real GPU, in the one form that harms nothing: a
    one-warp kernel waits, with the kernels' own wait functions and a limit of about a millisecond, on a
    barrier nothing arrives at.  The wait must give up (the call returns, the device stays usable), the
    status word must hold the code, the status ring must raise once, and an ordinary fused GEMM right after
    must be correct."""
    x, wg, wu = make(512, 256, 128, seed=21)
    want = F.gate_up_swiglu_forward(x, wg, wu)
    F.check_status(x.device)
    code = 900 + mode
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    word = F.selftest_wait_timeout(x.device, mode, 2_000_000, code)
    t1.record()
    torch.cuda.synchronize()
    assert int(word.item()) == code
    assert t0.elapsed_time(t1) < 100.0, "the wait is limited to about a millisecond"
    with pytest.raises(RuntimeError, match=f"code {code}"):
        F.check_status(x.device)
    F.check_status(x.device)  # reported once
    got = F.gate_up_swiglu_forward(x, wg, wu)
    F.check_status(x.device)
    assert torch.equal(got, want)
    # straight through the C ABI with a word of the caller's own
    st = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    lib = _lib.lib
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.swiglu_b200_selftest_wait_timeout(st.data_ptr(), mode, 2_000_000, 7, 0, stream) == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 7
    # argument checks: limit beyond the cap, zero code, unknown mode, null word
    assert lib.swiglu_b200_selftest_wait_timeout(st.data_ptr(), mode, 10**9, 7, 0, stream) == 3
    assert lib.swiglu_b200_selftest_wait_timeout(st.data_ptr(), mode, 1000, 0, 0, stream) == 3
    assert lib.swiglu_b200_selftest_wait_timeout(st.data_ptr(), 9, 1000, 7, 0, stream) == 3
    assert lib.swiglu_b200_selftest_wait_timeout(None, mode, 1000, 7, 0, stream) == 2

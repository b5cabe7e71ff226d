"""LoRA MLP (library GEMMs + the fused LoRA/SwiGLU epilogue + the backward-with-recompute kernel) against a
plain PyTorch composite under autograd, with the structure of the reference's own tests for its LoRAMLPv3
(kernels/lora_mlp/tests/test_lora_mlp.py:428-560: fp32 backward against the PyTorch reference, bf16 with its
loose tolerances), and the recompute kernel against this library's forward and backward kernels, bit for bit."""
import pytest
import torch

from kernel_pocs_b200 import _lib
from kernel_pocs_b200.fused_mlp import check_status
from kernel_pocs_b200.lora_mlp import LoRAMLP, lora_mlp, swiglu_DWf_DW_dfg_kernel
from kernel_pocs_b200.swiglu import swiglu_backward, swiglu_backward_recompute, swiglu_forward

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def rand3(shape, dtype, seed, offset=0):
    g = torch.Generator(device=DEVICE).manual_seed(seed)
    n = 1
    for d in shape:
        n *= d
    out = []
    for _ in range(3):
        buf = (1.5 * torch.randn(n + 16, generator=g, device=DEVICE)).to(dtype)
        out.append(buf[offset:offset + n].view(*shape))
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1,), (7,), (3, 5, 257), (64, 1024), (1000, 1101), (2048, 14336)])
@pytest.mark.parametrize("multipliers", [(1.0, 1.0), (0.7, 1.3)])
def test_recompute_equals_forward_and_backward(dtype, shape, multipliers):
    gm, dm = multipliers
    dh, gate, up = rand3(shape, dtype, seed=21)
    h_ref = swiglu_forward(gate, up, gm, dm)[0]
    dgate_ref, dup_ref = swiglu_backward(dh, gate, up, gm, dm, preserve_inputs=True)
    before = _lib.launch_count()
    h, dgate, dup = swiglu_backward_recompute(dh, gate, up, gm, dm, preserve_inputs=True)
    assert _lib.launch_count() == before + 1
    assert torch.equal(h.view(torch.uint8), h_ref.view(torch.uint8))
    assert torch.equal(dgate.view(torch.uint8), dgate_ref.view(torch.uint8))
    assert torch.equal(dup.view(torch.uint8), dup_ref.view(torch.uint8))
    # in place: h over dh, dgate over gate, dup over up
    dh2, gate2, up2 = dh.clone(), gate.clone(), up.clone()
    h2, dgate2, dup2 = swiglu_backward_recompute(dh2, gate2, up2, gm, dm)
    assert h2.data_ptr() == dh2.data_ptr() and dgate2.data_ptr() == gate2.data_ptr() and dup2.data_ptr() == up2.data_ptr()
    assert torch.equal(h2.view(torch.uint8), h_ref.view(torch.uint8))
    assert torch.equal(dgate2.view(torch.uint8), dgate_ref.view(torch.uint8))
    assert torch.equal(dup2.view(torch.uint8), dup_ref.view(torch.uint8))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("offset", [1, 2, 4])
def test_recompute_misaligned_buffers(dtype, offset):
    dh, gate, up = rand3((33, 1001), dtype, seed=22, offset=offset)
    h_ref = swiglu_forward(gate.clone(), up.clone())[0]
    dgate_ref, dup_ref = swiglu_backward(dh.clone(), gate.clone(), up.clone(), preserve_inputs=True)
    h, dgate, dup = swiglu_backward_recompute(dh, gate, up)   # in place, on the misaligned views
    assert torch.equal(h.view(torch.uint8), h_ref.view(torch.uint8))
    assert torch.equal(dgate.view(torch.uint8), dgate_ref.view(torch.uint8))
    assert torch.equal(dup.view(torch.uint8), dup_ref.view(torch.uint8))


def test_reference_buffer_convention():
    """DW <- h, e <- gradient of g, g <- gradient of e (the cross pairing of the reference's backward step)."""
    dw, e, g = rand3((256, 1536), torch.bfloat16, seed=23)
    h_ref = swiglu_forward(e, g)[0]
    de_ref, dg_ref = swiglu_backward(dw, e, g, preserve_inputs=True)
    a, b, c = swiglu_DWf_DW_dfg_kernel(dw, e, g)
    assert a is dw and b is e and c is g
    assert torch.equal(dw, h_ref) and torch.equal(e, dg_ref) and torch.equal(g, de_ref)


def test_recompute_alias_errors():
    dh, gate, up = rand3((4, 64), torch.bfloat16, seed=24)
    lib, st = _lib.lib, torch.cuda.current_stream().cuda_stream
    out = torch.empty(3, 4 * 64, dtype=torch.bfloat16, device=DEVICE)
    args = (4 * 64, 2, 1.0, 1.0, 0, st)
    # two outputs on one buffer; an output overlapping an input at an offset
    assert lib.swiglu_b200_bwd_recompute(out[0].data_ptr(), out[0].data_ptr(), out[2].data_ptr(), dh.data_ptr(),
                                         gate.data_ptr(), up.data_ptr(), *args) == 5
    assert lib.swiglu_b200_bwd_recompute(out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                         out[0].data_ptr() + 32, gate.data_ptr(), up.data_ptr(), *args) == 5
    assert lib.swiglu_b200_bwd_recompute(None, out[1].data_ptr(), out[2].data_ptr(), dh.data_ptr(),
                                         gate.data_ptr(), up.data_ptr(), *args) == 2
    assert lib.swiglu_b200_bwd_recompute(out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), dh.data_ptr(),
                                         gate.data_ptr(), up.data_ptr(), 0, 2, 1.0, 1.0, 0, st) == 0
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        swiglu_backward_recompute(dh.cpu(), gate.cpu(), up.cpu())


# ------------------------------------------------------------------------------------------------ the MLP

def make_params(hidden, inter, rank, dtype, seed=42):
    g = torch.Generator(device=DEVICE).manual_seed(seed)
    mk = lambda *s, std: (std * torch.randn(*s, generator=g, device=DEVICE)).to(dtype)
    p = {}
    for name, (o, i) in dict(gate=(inter, hidden), up=(inter, hidden), down=(hidden, inter)).items():
        p[f"W_{name}"] = mk(o, i, std=i ** -0.5)
        p[f"A_{name}"] = mk(rank, i, std=i ** -0.5)
        p[f"B_{name}"] = mk(o, rank, std=0.3)      # non-zero, so that every gradient is exercised
        p[f"s_{name}"] = 2.0
    return p


def composite(X, p):
    proj = lambda x, n: x @ p[f"W_{n}"].t() + p[f"s_{n}"] * ((x @ p[f"A_{n}"].t()) @ p[f"B_{n}"].t())
    return proj(torch.nn.functional.silu(proj(X, "gate")) * proj(X, "up"), "down")


def args_of(X, p):
    return (X, p["W_gate"], p["A_gate"], p["B_gate"], p["s_gate"], p["W_up"], p["A_up"], p["B_up"], p["s_up"],
            p["W_down"], p["A_down"], p["B_down"], p["s_down"])


GRADS = ["A_gate", "B_gate", "A_up", "B_up", "A_down", "B_down"]


def run_with_grads(fn, X, p, dY):
    X = X.detach().clone().requires_grad_(True)
    q = {k: (v.detach().clone().requires_grad_(k in GRADS) if isinstance(v, torch.Tensor) else v)
         for k, v in p.items()}
    out = fn(X, q)
    out.backward(dY)
    return out.detach(), [X.grad] + [q[k].grad for k in GRADS]


@pytest.mark.parametrize("shape,rank", [((2, 32, 128, 256), 8), ((1, 100, 192, 520), 16), ((3, 17, 64, 136), 24)])
def test_mlp_fp32_matches_composite(shape, rank):
    b, s, hidden, inter = shape
    p = make_params(hidden, inter, rank, torch.float32)
    X = torch.randn(b, s, hidden, device=DEVICE)
    dY = torch.randn(b, s, hidden, device=DEVICE)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        out_ref, grads_ref = run_with_grads(composite, X, p, dY)
        out, grads = run_with_grads(lambda x, q: LoRAMLP.apply(*args_of(x, q)), X, p, dY)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    torch.testing.assert_close(out, out_ref, rtol=1e-4, atol=1e-4)
    for name, a, r in zip(["X"] + GRADS, grads, grads_ref):
        torch.testing.assert_close(a, r, rtol=1e-3, atol=1e-3 * float(r.abs().max()), msg=lambda m: f"d{name}: {m}")


@pytest.mark.parametrize("shape,rank", [((2, 32, 128, 256), 8), ((2, 256, 512, 1408), 16), ((1, 333, 256, 1096), 32),
                                        ((4, 512, 1024, 2816), 64), ((1, 64, 128, 264), 12)])
def test_mlp_bf16_matches_fp32_composite(shape, rank):
    """bf16 run against the fp32 composite of the same bf16 parameters; bound per tensor: 3 % of its largest
    magnitude (the reference's own bf16 check uses rtol 5e-2 with atol 2.0, test_lora_mlp.py:907-933)."""
    b, s, hidden, inter = shape
    p = make_params(hidden, inter, rank, torch.bfloat16)
    g = torch.Generator(device=DEVICE).manual_seed(7)
    X = torch.randn(b, s, hidden, generator=g, device=DEVICE).bfloat16()
    dY = torch.randn(b, s, hidden, generator=g, device=DEVICE).bfloat16()
    p32 = {k: (v.float() if isinstance(v, torch.Tensor) else v) for k, v in p.items()}
    out_ref, grads_ref = run_with_grads(composite, X.float(), p32, dY.float())
    before = _lib.lib.swiglu_b200_gemm_launch_count()
    out, grads = run_with_grads(lambda x, q: LoRAMLP.apply(*args_of(x, q)), X, p, dY)
    check_status(X.device)
    fused = rank % 8 == 0 and inter % 16 == 0
    assert _lib.lib.swiglu_b200_gemm_launch_count() == before + (1 if fused else 0)
    assert out.dtype == torch.bfloat16 and out.shape == X.shape
    for name, a, r in zip(["out", "X"] + GRADS, [out] + grads, [out_ref] + grads_ref):
        assert a.shape == r.shape and a.dtype == torch.bfloat16, name
        err = (a.float() - r).abs().max().item()
        assert err <= 0.03 * r.abs().max().item(), f"{name}: max err {err} against max |ref| {r.abs().max().item()}"
    # inference entry: same forward, 2-D input, no autograd graph
    out2 = lora_mlp(*args_of(X.view(-1, hidden), p))
    assert out2.shape == (b * s, hidden) and not out2.requires_grad
    assert torch.equal(out2.view_as(out), out)


def test_mlp_without_adapters_and_determinism():
    p = make_params(128, 256, 8, torch.bfloat16)
    X = torch.randn(2, 16, 128, device=DEVICE).bfloat16()
    q = dict(p, A_gate=None, B_gate=None, A_up=None, B_up=None, A_down=None, B_down=None)
    out = lora_mlp(*args_of(X, q))
    ref = (torch.nn.functional.silu(X.float() @ p["W_gate"].float().t()) * (X.float() @ p["W_up"].float().t())) \
        @ p["W_down"].float().t()
    assert (out.float() - ref).abs().max() <= 0.03 * ref.abs().max()
    a, b = lora_mlp(*args_of(X, p)), lora_mlp(*args_of(X, p))
    assert torch.equal(a, b) and torch.isfinite(a).all()


# ------------------------------------------------------------------- vectors produced by the reference itself

def golden_cases(golden_dir):
    import numpy as np

    from tests.test_oracle_golden import _cases, load_lora_case
    from tests._util import DTYPES as BY_NAME

    z = np.load(golden_dir / "lora_mlp.npz")
    for key in _cases(z):
        dtype = BY_NAME[key.split("|")[0]]
        t, p = load_lora_case(z, key, dtype)
        yield key, dtype, {k: v.to(DEVICE) for k, v in t.items()}, \
            {k: (v.to(DEVICE) if isinstance(v, torch.Tensor) else v) for k, v in p.items()}


def test_mlp_matches_reference_vectors(golden_dir):
    """LoRAMLP on the inputs of tests/golden/lora_mlp.npz against what the reference's own LoRAMLP (its PyTorch
    ground truth, kernels/lora_mlp/reference/lora_mlp_pytorch.py:113-236) returned for them, and against the
    float64 oracle: fp32 to 1e-4 of each tensor's largest magnitude, bf16 to 3 %."""
    from oracle import lora_oracle as L

    seen = 0
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for key, dtype, t, p in golden_cases(golden_dir):
            out, grads = run_with_grads(lambda x, q: LoRAMLP.apply(*args_of(x, q)), t["X"], p, t["dY"])
            check_status(t["X"].device)
            truth = L.lora_mlp_fwd_bwd(t["X"].double().cpu().numpy(),
                                       {k: (v.double().cpu().numpy() if isinstance(v, torch.Tensor) else v)
                                        for k, v in p.items()}, t["dY"].double().cpu().numpy())
            bound = 1e-4 if dtype == torch.float32 else 3e-2
            names = ["out", "dX"] + ["d" + n for n in GRADS]
            for name, got in zip(names, [out] + grads):
                ref = t[name].double().reshape(got.shape)
                assert got.dtype == dtype
                err = (got.double() - ref).abs().max().item()
                assert err <= bound * ref.abs().max().item(), f"{key} {name} vs reference vectors: {err}"
                tr = torch.from_numpy(truth[name]).to(DEVICE).reshape(got.shape)
                err = (got.double() - tr).abs().max().item()
                assert err <= bound * tr.abs().max().item(), f"{key} {name} vs float64 oracle: {err}"
            seen += 1
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    assert seen == 4


def test_epilogue_and_fused_projection_match_reference_vectors(golden_dir):
    """bf16 vectors: the LoRA epilogue fed with cuBLAS base projections against the reference's e, g, h, and the
    fused gate/up GEMM against its adapter-free h.  e and g carry one bf16 rounding on either side:
    2^-7 |ref| + 2^-7 rms(ref).  The reference's h is computed from its ROUNDED e and g and rounded again (three
    roundings, each up to 2^-9 relative, plus one here, and the roundings of e and g are relative to THEIR magnitude,
    not to that of h), so h gets 2^-6 |ref| + 2^-6 rms(ref)."""
    from kernel_pocs_b200.fused_mlp import gate_up_swiglu_forward
    from kernel_pocs_b200.lora_mlp import fused_lora_swiglu

    def close(got, ref, what, rel=2.0 ** -7):
        ref = ref.float().reshape(got.shape)
        err = (got.float() - ref).abs()
        tol = rel * (ref.abs() + ref.pow(2).mean().sqrt())
        assert bool((err <= tol).all()), f"{what}: worst excess {(err - tol).max().item()}"

    seen = 0
    for key, dtype, t, p in golden_cases(golden_dir):
        if dtype != torch.bfloat16:
            continue
        x2 = t["X"].reshape(-1, t["X"].shape[-1])
        h, e, g = fused_lora_swiglu(x2 @ p["W_gate"].t(), x2 @ p["W_up"].t(), x2 @ p["A_gate"].t(), x2 @ p["A_up"].t(),
                                    p["B_gate"], p["B_up"], p["s_gate"], p["s_up"], save_eg=True)
        check_status(x2.device)
        close(e, t["e"], f"{key} e")
        close(g, t["g"], f"{key} g")
        close(h, t["h"], f"{key} h", rel=2.0 ** -6)
        h0 = gate_up_swiglu_forward(x2, p["W_gate"], p["W_up"])
        check_status(x2.device)
        close(h0, t["h_noadapter"], f"{key} fused projection h", rel=2.0 ** -6)
        seen += 1
    assert seen == 2


@pytest.mark.parametrize("m,n,k,r", [(256, 128, 64, 8), (300, 272, 200, 16), (1000, 1040, 520, 24), (512, 512, 256, 32),
                                     (777, 2064, 1024, 40), (2048, 1408, 512, 64), (4096, 14336, 4096, 16)])
@pytest.mark.parametrize("save_eg", [False, True])
def test_one_launch_projection_with_adapters(m, n, k, r, save_eg):
    """swiglu_b200_lora_gemm_fwd against fp32 PyTorch on the same bf16 operands: the adapter terms enter as extra
    contraction steps (tiles loaded at column 64 j for the gate half, 64 j - r for the up half, zero-filled
    outside the adapter matrix), for every rank layout: 2r below, at and above one 64-wide step."""
    from kernel_pocs_b200.fused_mlp import lora_gate_up_swiglu_forward
    from tests.test_fused_gemm import assert_close_bf16

    g = torch.Generator(device=DEVICE).manual_seed(31)
    mk = lambda *s, std: (std * torch.randn(*s, generator=g, device=DEVICE)).bfloat16()
    x, wg, wu = mk(m, k, std=1.0), mk(n, k, std=k ** -0.5), mk(n, k, std=k ** -0.5)
    ag, au, bg, bu = mk(r, k, std=k ** -0.5), mk(r, k, std=k ** -0.5), mk(n, r, std=0.3), mk(n, r, std=0.3)
    sg, su = 2.0, 0.75
    before = _lib.lib.swiglu_b200_gemm_launch_count()
    h, e, gg = lora_gate_up_swiglu_forward(x, wg, wu, ag, bg, sg, au, bu, su, save_eg=save_eg)
    check_status(x.device)
    assert _lib.lib.swiglu_b200_gemm_launch_count() == before + 1
    # x (s A)^T is a bf16 tensor on its way into the kernel (as x A^T is in the reference, whose xa_gate / xa_up
    # are bf16 matmul results): the comparison starts from those values
    xf = x.float()
    xa_g = (x @ (ag * sg).t()).float()
    xa_u = (x @ (au * su).t()).float()
    e_ref = xf @ wg.float().t() + xa_g @ bg.float().t()
    g_ref = xf @ wu.float().t() + xa_u @ bu.float().t()
    assert_close_bf16(h, torch.nn.functional.silu(e_ref) * g_ref, "h")
    if save_eg:
        assert_close_bf16(e, e_ref, "e")
        assert_close_bf16(gg, g_ref, "g")
    else:
        assert e is None and gg is None
    # zero second factors reduce to the plain fused projection, bit for bit
    from kernel_pocs_b200.fused_mlp import gate_up_swiglu_forward

    h0, _, _ = lora_gate_up_swiglu_forward(x, wg, wu, ag, torch.zeros_like(bg), sg, au, torch.zeros_like(bu), su)
    check_status(x.device)
    assert torch.equal(h0, gate_up_swiglu_forward(x, wg, wu))


# ------------------------------------------------------------------------------------------ GELU-gated blocks

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("approximate", ["tanh", "none"])
@pytest.mark.parametrize("shape", [(7,), (3, 5, 257), (1000, 1101)])
def test_geglu_recompute_equals_forward_and_backward(dtype, approximate, shape):
    from kernel_pocs_b200.geglu import geglu_backward, geglu_backward_recompute, geglu_forward

    dh, gate, up = rand3(shape, dtype, seed=41)
    h_ref = geglu_forward(gate, up, approximate)[0]
    dgate_ref, dup_ref = geglu_backward(dh, gate, up, approximate, preserve_inputs=True)
    h, dgate, dup = geglu_backward_recompute(dh, gate, up, approximate, preserve_inputs=True)
    for got, ref in ((h, h_ref), (dgate, dgate_ref), (dup, dup_ref)):
        assert torch.equal(got.reshape(-1).view(torch.uint8), ref.reshape(-1).view(torch.uint8))
    dh2, gate2, up2 = dh.clone(), gate.clone(), up.clone()
    h2, dgate2, dup2 = geglu_backward_recompute(dh2, gate2, up2, approximate)
    assert h2.data_ptr() == dh2.data_ptr() and dgate2.data_ptr() == gate2.data_ptr()
    assert torch.equal(h2, h) and torch.equal(dgate2, dgate) and torch.equal(dup2, dup)


def composite_act(X, p, activation):
    proj = lambda x, n: x @ p[f"W_{n}"].t() + p[f"s_{n}"] * ((x @ p[f"A_{n}"].t()) @ p[f"B_{n}"].t())
    e = proj(X, "gate")
    act = torch.nn.functional.silu(e) if activation == "silu" else torch.nn.functional.gelu(
        e, approximate="tanh" if activation == "gelu_tanh" else "none")
    return proj(act * proj(X, "up"), "down")


@pytest.mark.parametrize("activation", ["gelu_tanh", "gelu_exact"])
@pytest.mark.parametrize("dtype,shape,rank", [(torch.float32, (2, 32, 128, 256), 8), (torch.bfloat16, (2, 256, 512, 1408), 16),
                                              (torch.bfloat16, (1, 100, 128, 264), 12)])
def test_mlp_with_gelu_gate_matches_composite(activation, dtype, shape, rank):
    """LoRAMLP with the GELU gates of the Gemma family (no fused kernel for it exists in the reference) against the
    PyTorch composite under autograd: fp32 tightly, bf16 within 3 % of each tensor's largest magnitude against the
    fp32 composite of the same bf16 parameters."""
    b, s, hidden, inter = shape
    p = make_params(hidden, inter, rank, dtype)
    g = torch.Generator(device=DEVICE).manual_seed(9)
    X = torch.randn(b, s, hidden, generator=g, device=DEVICE).to(dtype)
    dY = torch.randn(b, s, hidden, generator=g, device=DEVICE).to(dtype)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        p32 = {k: (v.float() if isinstance(v, torch.Tensor) else v) for k, v in p.items()}
        out_ref, grads_ref = run_with_grads(lambda x, q: composite_act(x, q, activation), X.float(), p32, dY.float())
        before = _lib.lib.swiglu_b200_gemm_launch_count()
        out, grads = run_with_grads(lambda x, q: LoRAMLP.apply(*args_of(x, q), activation), X, p, dY)
        check_status(X.device)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    one_launch = dtype == torch.bfloat16 and rank % 8 == 0 and inter % 16 == 0
    assert _lib.lib.swiglu_b200_gemm_launch_count() == before + (1 if one_launch else 0)
    bound = 1e-3 if dtype == torch.float32 else 3e-2
    for name, a, r in zip(["out", "X"] + GRADS, [out] + grads, [out_ref] + grads_ref):
        assert a.dtype == dtype and a.shape == r.shape, name
        err = (a.float() - r).abs().max().item()
        assert err <= bound * r.abs().max().item(), f"{name}: max err {err} against max |ref| {r.abs().max().item()}"
    assert torch.equal(lora_mlp(*args_of(X, p), activation), out)

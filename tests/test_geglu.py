"""GeGLU, the sibling operator: oracle pin on the CPU, parity of the CUDA path on the GPU.

CPU: the C restatement (oracle "chain") against vectors produced by the reference's own geglu() /
geglu_packed() CPU path (tests/golden/geglu.npz, written by tests/golden/make_golden.py).
GPU: the reference's parametrisation (tests/test_geglu.py:32-118: shapes, both GELU forms, preserve_inputs,
dtypes with their tolerances, seeds) through the same call signature, then the tight contract used for
SwiGLU: 16-bit outputs within one ulp of the fp32 closed form rounded once and a correct rounding of the
float64 truth; fp32 within 2e-6 (scaled by |dh*up| for dgate, whose derivative factor crosses zero near
x = -0.75).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests._util import DTYPES, assert_rel_scaled, assert_rounded_once, assert_ulp

DEVICE = "cuda"


def _names(npz):
    return sorted({k.rsplit("|", 1)[0] for k in npz.files})


def test_oracle_matches_reference_vectors(golden_dir):
    z = np.load(golden_dir / "geglu.npz")
    keys = _names(z)
    assert len(keys) == 18
    for key in keys:
        dname, shape, approximate = key.split("|")
        dtype = DTYPES[dname]
        if shape == "packed":
            gate_up, dout, h, dgate_up = (O.from_numpy_bits(z[f"{key}|{n}"], dtype) for n in ("gate_up", "dout", "h", "dgate_up"))
            gate, up = O.packed_split(gate_up)
            dgate, dup = O.packed_split(dgate_up)
        else:
            gate, up, dout, h, dgate, dup = (O.from_numpy_bits(z[f"{key}|{n}"], dtype)
                                             for n in ("gate", "up", "dout", "h", "dgate", "dup"))
        oh = O.geglu_fwd(gate, up, approximate, "chain")
        odg, odu = O.geglu_bwd(dout, gate, up, approximate, "chain")
        if dtype == torch.float32:
            # libm's tanhf/erff against ATen's vectorised ones (its erf carries ~1e-7 absolute error): errors
            # are bounded relative to the operands, |gate*up| for h, |gate*dh| for dup, |dh*up| for dgate
            g64, u64, d64 = gate.double().abs(), up.double().abs(), dout.double().abs()
            assert_rel_scaled(oh, h.double(), 2e-6, f"{key} h", scale=g64 * u64)
            assert_rel_scaled(odu, dup.double(), 2e-6, f"{key} dup", scale=g64 * d64)
            assert_rel_scaled(odg, dgate.double(), 2e-6, f"{key} dgate", scale=d64 * u64)
        else:
            # tanh form: bit-identical but for rounding boundaries.  erf form: ATen evaluates erf on the CPU by
            # a vectorised approximation with ~1e-7 absolute error; for gate < -2, where 1 + erf cancels, that
            # is a sizeable fraction of a 16-bit ulp of the activation (libm's erff is accurate there), so the
            # two implementations round the intermediate differently and the results part by a few ulp
            for got, want, n in ((oh, h, "h"), (odu, dup, "dup"), (odg, dgate, "dgate")):
                d = O.ulp_distance(got, want)
                assert float((d == 0).double().mean()) >= (0.999 if approximate == "tanh" else 0.98), f"{key} {n}"
                bad = (d > 8) | ((d > 1) & (gate.float() > -2.0))
                assert not bool(bad.any()), f"{key} {n}: {int(bad.sum())} elements differ from the reference"


def test_round_once_variant_is_a_correct_rounding_of_the_truth():
    g = torch.Generator().manual_seed(17)
    for dname in ("bf16", "fp16"):
        dtype = DTYPES[dname]
        gate, up, dout = ((2.0 * torch.randn(32, 1000, generator=g)).to(dtype) for _ in range(3))
        for approximate in ("tanh", "none"):
            h = O.geglu_fwd(gate, up, approximate, "once")
            dg, du = O.geglu_bwd(dout, gate, up, approximate, "once")
            th, tdg, tdu, scale = O.geglu_f64(dout, gate, up, approximate)
            assert_rounded_once(h, th, f"{dname} {approximate} h", extra=1e-6 * up.double().abs())
            assert_rounded_once(du, tdu, f"{dname} {approximate} dup", extra=1e-6 * dout.double().abs())
            assert_rounded_once(dg, tdg, f"{dname} {approximate} dgate", extra=1e-6 * scale)


def test_host_api_without_gpu():
    import kernels.geglu as dropin

    with pytest.raises(ValueError, match="same shape"):
        dropin.geglu(torch.randn(2, 3), torch.randn(2, 4))
    with pytest.raises(ValueError, match="approximate must be"):
        dropin.geglu(torch.randn(2, 3), torch.randn(2, 3), approximate="fast")
    with pytest.raises(ValueError, match="even"):
        dropin.geglu_packed(torch.randn(2, 5))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        dropin.geglu(torch.randn(2, 3), torch.randn(2, 3))
    g, u = torch.randn(4, 9), torch.randn(4, 9)
    assert torch.equal(dropin.torch_geglu_reference(g, u, "none"), torch.nn.functional.gelu(g) * u)
    # MLP-level helpers (reference tests/test_geglu.py:289-297 and the packing rules of geglu.py:275-308)
    with pytest.raises(ValueError, match="either packed_gate_up_weight or separate"):
        dropin.geglu_mlp(torch.randn(2, 3), torch.randn(3, 4), gate_weight=torch.randn(4, 3), up_weight=torch.randn(4, 3),
                         packed_gate_up_weight=torch.randn(8, 3))
    with pytest.raises(ValueError, match="separate path requires"):
        dropin.geglu_mlp(torch.randn(2, 3), torch.randn(3, 4), gate_weight=torch.randn(4, 3))
    with pytest.raises(ValueError, match="must be even"):
        dropin.geglu_mlp(torch.randn(2, 3), torch.randn(3, 4), packed_gate_up_weight=torch.randn(7, 3))
    with pytest.raises(ValueError, match="use packed_gate_up_bias"):
        dropin.geglu_mlp(torch.randn(2, 3), torch.randn(3, 4), packed_gate_up_weight=torch.randn(8, 3),
                         gate_bias=torch.randn(4))
    with pytest.raises(TypeError, match="dtype"):
        dropin.geglu_mlp(torch.randn(2, 3), torch.randn(3, 4), gate_weight=torch.randn(4, 3).half(),
                         up_weight=torch.randn(4, 3).half())
    with pytest.raises(ValueError, match="same shape"):
        dropin.pack_geglu_gate_up_weight(torch.randn(4, 3), torch.randn(5, 3))
    with pytest.raises(ValueError, match="both be None or both be tensors"):
        dropin.pack_geglu_gate_up_bias(torch.randn(4), None)
    wg, wu = torch.randn(4, 3), torch.randn(4, 3)
    packed = dropin.pack_geglu_gate_up_weight(wg, wu)
    assert packed.shape == (8, 3) and torch.equal(packed[:4], wg) and torch.equal(packed[4:], wu)
    assert dropin.pack_geglu_gate_up_bias(None, None) is None
    assert torch.equal(dropin.pack_geglu_gate_up_bias(torch.ones(4), torch.zeros(4)), torch.tensor([1.0] * 4 + [0.0] * 4))
    x, wd = torch.randn(2, 5, 3), torch.randn(3, 4)
    ref = dropin.torch_geglu_mlp_reference(x, wg, wu, wd, approximate="none")
    assert torch.allclose(ref, (torch.nn.functional.gelu(x @ wg.t()) * (x @ wu.t())) @ wd.t(), atol=1e-6)


def _check(h, dgate, dup, gate, up, dout, approximate, what):
    gate, up, dout = gate.detach().cpu(), up.detach().cpu(), dout.detach().cpu()
    dtype = gate.dtype
    th, tdg, tdu, scale = O.geglu_f64(dout, gate, up, approximate)
    if dtype == torch.float32:
        # |gelu(x)| has no floor in the negative tail; bound the error by the operand scale there.  2e-6: the
        # sigmoid's argument q(x) reaches |q| ~ 10 where gelu is still 1e-3 of x, and exp(-q) turns the fp32
        # rounding of q (~1e-7 |q|) into that relative error; measured worst case 1.02e-6 on N(0, 2^2) data
        assert_rel_scaled(h, th, 2e-6, f"{what} h", scale=1e-3 * up.double().abs())
        assert_rel_scaled(dup, tdu, 2e-6, f"{what} dup", scale=1e-3 * dout.double().abs())
        assert_rel_scaled(dgate, tdg, 2e-6, f"{what} dgate", scale=scale)
        return
    oh = O.geglu_fwd(gate, up, approximate, "once")
    odg, odu = O.geglu_bwd(dout, gate, up, approximate, "once")
    assert_ulp(h, oh, 1, f"{what} h vs once", min_exact=0.99)
    assert_ulp(dup, odu, 1, f"{what} dup vs once", min_exact=0.99)
    assert_ulp(dgate, odg, 1, f"{what} dgate vs once", min_exact=0.99)
    assert_rounded_once(h, th, f"{what} h", extra=1e-6 * up.double().abs())
    assert_rounded_once(dup, tdu, f"{what} dup", extra=1e-6 * dout.double().abs())
    assert_rounded_once(dgate, tdg, f"{what} dgate", extra=1e-6 * scale)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 8, 128), (1, 3, 257), (4, 5, 1024), (1, 2, 11008)])
@pytest.mark.parametrize("approximate", ["tanh", "none"])
@pytest.mark.parametrize("preserve_inputs", [False, True])
@pytest.mark.parametrize("dtype, atol, rtol", [(torch.float32, 1e-5, 1e-5), (torch.float16, 2e-2, 2e-2),
                                               (torch.bfloat16, 3e-2, 3e-2)])
def test_geglu_forward_backward(shape, approximate, preserve_inputs, dtype, atol, rtol):
    from kernels.geglu import geglu, torch_geglu_reference

    torch.manual_seed(0)
    gate_ref = torch.randn(*shape, device=DEVICE, dtype=dtype, requires_grad=True)
    up_ref = torch.randn(*shape, device=DEVICE, dtype=dtype, requires_grad=True)
    gate_forge = gate_ref.detach().clone().requires_grad_(True)
    up_forge = up_ref.detach().clone().requires_grad_(True)
    gate_before, up_before = gate_forge.detach().clone(), up_forge.detach().clone()

    out_ref = torch_geglu_reference(gate_ref, up_ref, approximate)
    out_forge = geglu(gate_forge, up_forge, approximate, preserve_inputs)
    torch.testing.assert_close(out_forge, out_ref, atol=atol, rtol=rtol)
    grad = torch.randn_like(out_ref)
    out_ref.backward(grad)
    out_forge.backward(grad)
    torch.testing.assert_close(gate_forge.grad, gate_ref.grad, atol=atol, rtol=rtol)
    torch.testing.assert_close(up_forge.grad, up_ref.grad, atol=atol, rtol=rtol)
    if preserve_inputs:
        torch.testing.assert_close(gate_forge.detach(), gate_before, atol=0, rtol=0)
        torch.testing.assert_close(up_forge.detach(), up_before, atol=0, rtol=0)
    _check(out_forge, gate_forge.grad, up_forge.grad, gate_before, up_before, grad, approximate,
           f"geglu {approximate} {dtype} {shape}")


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 8, 256), (1, 3, 514)])
@pytest.mark.parametrize("approximate", ["tanh", "none"])
@pytest.mark.parametrize("preserve_inputs", [False, True])
@pytest.mark.parametrize("dtype, atol, rtol", [(torch.float32, 1e-5, 1e-5), (torch.float16, 2e-2, 2e-2),
                                               (torch.bfloat16, 3e-2, 3e-2)])
def test_geglu_packed_forward_backward(shape, approximate, preserve_inputs, dtype, atol, rtol):
    from kernels.geglu import geglu_packed, torch_geglu_packed_reference

    torch.manual_seed(1)
    gate_up_ref = torch.randn(*shape, device=DEVICE, dtype=dtype, requires_grad=True)
    gate_up_forge = gate_up_ref.detach().clone().requires_grad_(True)
    gate_up_before = gate_up_forge.detach().clone()
    out_ref = torch_geglu_packed_reference(gate_up_ref, approximate)
    out_forge = geglu_packed(gate_up_forge, approximate, preserve_inputs)
    torch.testing.assert_close(out_forge, out_ref, atol=atol, rtol=rtol)
    grad = torch.randn_like(out_ref)
    out_ref.backward(grad)
    out_forge.backward(grad)
    torch.testing.assert_close(gate_up_forge.grad, gate_up_ref.grad, atol=atol, rtol=rtol)
    if preserve_inputs:
        torch.testing.assert_close(gate_up_forge.detach(), gate_up_before, atol=0, rtol=0)
    gate, up = O.packed_split(gate_up_before.cpu())
    dgate, dup = O.packed_split(gate_up_forge.grad.cpu())
    _check(out_forge, dgate, dup, gate, up, grad, approximate, f"geglu packed {approximate} {dtype} {shape}")


@pytest.mark.gpu
@pytest.mark.parametrize("approximate", ["tanh", "none"])
def test_geglu_forward_special_values(approximate):
    from kernels.geglu import geglu, torch_geglu_reference

    gate = torch.tensor([[[0.0, float("inf"), float("-inf"), float("nan"), 20.0, -20.0]]], device=DEVICE)
    up = torch.tensor([[[1.0, 2.0, 3.0, 4.0, -1.0, -2.0]]], device=DEVICE)
    out_ref = torch_geglu_reference(gate, up, approximate)
    out_forge = geglu(gate, up, approximate, preserve_inputs=True)
    # gelu(-inf) is -inf * 0 = NaN in the reference's tanh form and in both forms here, -0 in its erf form;
    # compare the positions where the reference is finite or NaN alike
    same = torch.isnan(out_ref) == torch.isnan(out_forge)
    assert bool(same[..., [0, 1, 3, 4, 5]].all())
    ok = torch.isfinite(out_ref) & torch.isfinite(out_forge)
    torch.testing.assert_close(out_forge[ok], out_ref[ok], atol=1e-12, rtol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dname", ["bf16", "fp32"])
@pytest.mark.parametrize("approximate", ["tanh", "none"])
def test_geglu_wide_rows_and_tails(dname, approximate):
    """Hidden size above the reference's 65536 row limit (its test :122-138) with N(0, 2^2) inputs."""
    from kernels.geglu import geglu_backward, geglu_forward

    dtype = DTYPES[dname]
    g = torch.Generator().manual_seed(2)
    gate0, up0, dout0 = ((2.0 * torch.randn(3, 65537, generator=g)).to(dtype) for _ in range(3))
    gate, up = gate0.to(DEVICE), up0.to(DEVICE)
    h, gate_flat, up_flat = geglu_forward(gate, up, approximate)
    dgate, dup = geglu_backward(dout0.to(DEVICE), gate_flat, up_flat, approximate)
    assert dgate.data_ptr() == gate.data_ptr()
    _check(h, dgate, dup, gate0, up0, dout0, approximate, f"geglu wide {dname} {approximate}")


# ------------------------------------------------------------------------------------------ MLP level

@pytest.mark.gpu
@pytest.mark.parametrize("use_bias", [False, True])
@pytest.mark.parametrize("approximate", ["tanh", "none"])
@pytest.mark.parametrize("intermediate", [257, 272])
@pytest.mark.parametrize("dtype, atol, rtol", [(torch.float32, 2e-5, 2e-5), (torch.float16, 3e-2, 3e-2),
                                               (torch.bfloat16, 4e-2, 4e-2)])
def test_geglu_mlp_packed_matches_separate_and_reference(use_bias, approximate, intermediate, dtype, atol, rtol):
    """Parametrisation, seed, sizes and tolerances of the reference's test of the same name
    (tests/test_geglu.py:160-270); width 272 is added because bias-free bf16 at that width takes the one-launch
    tcgen05 path for the gate/up stage, while 257 (the reference's width) takes library GEMMs + the GeGLU kernels."""
    from kernel_pocs_b200 import _lib
    from kernels.geglu import geglu_mlp, pack_geglu_gate_up_bias, pack_geglu_gate_up_weight, torch_geglu_mlp_reference

    torch.manual_seed(3)
    batch, seq, hidden = 2, 7, 128
    mk = lambda *shape: (torch.randn(*shape, device=DEVICE, dtype=dtype) * 0.02)
    x0 = torch.randn(batch, seq, hidden, device=DEVICE, dtype=dtype)
    wg0, wu0, wd0 = mk(intermediate, hidden), mk(intermediate, hidden), mk(hidden, intermediate)
    bg0, bu0, bd0 = (mk(intermediate), mk(intermediate), mk(hidden)) if use_bias else (None, None, None)
    leaf = lambda t: None if t is None else t.detach().clone().requires_grad_(True)

    x_r, wg_r, wu_r, wd_r, bg_r, bu_r, bd_r = map(leaf, (x0, wg0, wu0, wd0, bg0, bu0, bd0))
    out_ref = torch_geglu_mlp_reference(x_r, wg_r, wu_r, wd_r, bg_r, bu_r, bd_r, approximate)
    x_s, wg_s, wu_s, wd_s, bg_s, bu_s, bd_s = map(leaf, (x0, wg0, wu0, wd0, bg0, bu0, bd0))
    before = _lib.lib.swiglu_b200_gemm_launch_count()
    out_sep = geglu_mlp(x_s, wd_s, gate_weight=wg_s, up_weight=wu_s, gate_bias=bg_s, up_bias=bu_s, down_bias=bd_s,
                        approximate=approximate, preserve_inputs=False)
    x_p, wd_p, bd_p = leaf(x0), leaf(wd0), leaf(bd0)
    w_p = pack_geglu_gate_up_weight(wg0, wu0).requires_grad_(True)
    b_p = pack_geglu_gate_up_bias(bg0, bu0)
    if b_p is not None:
        b_p.requires_grad_(True)
    out_packed = geglu_mlp(x_p, wd_p, packed_gate_up_weight=w_p, packed_gate_up_bias=b_p, down_bias=bd_p,
                           approximate=approximate, preserve_inputs=False)
    one_launch = dtype == torch.bfloat16 and not use_bias and intermediate % 16 == 0
    assert _lib.lib.swiglu_b200_gemm_launch_count() == before + (2 if one_launch else 0)
    torch.testing.assert_close(out_sep, out_ref, atol=atol, rtol=rtol)
    torch.testing.assert_close(out_packed, out_ref, atol=atol, rtol=rtol)

    grad = torch.randn_like(out_ref)
    out_ref.backward(grad)
    out_sep.backward(grad)
    out_packed.backward(grad)
    close = lambda a, b: torch.testing.assert_close(a, b, atol=atol, rtol=rtol)
    close(x_s.grad, x_r.grad)
    close(x_p.grad, x_r.grad)
    close(wg_s.grad, wg_r.grad)
    close(wu_s.grad, wu_r.grad)
    close(wd_s.grad, wd_r.grad)
    close(w_p.grad[:intermediate], wg_r.grad)
    close(w_p.grad[intermediate:], wu_r.grad)
    close(wd_p.grad, wd_r.grad)
    if use_bias:
        close(bg_s.grad, bg_r.grad)
        close(bu_s.grad, bu_r.grad)
        close(bd_s.grad, bd_r.grad)
        close(b_p.grad[:intermediate], bg_r.grad)
        close(b_p.grad[intermediate:], bu_r.grad)
        close(bd_p.grad, bd_r.grad)


@pytest.mark.gpu
@pytest.mark.parametrize("approximate", ["tanh", "none"])
@pytest.mark.parametrize("m,n,k", [(256, 128, 256), (300, 272, 200), (2048, 2064, 1024)])
def test_one_launch_gate_up_geglu(m, n, k, approximate):
    """swiglu_b200_geglu_gemm_fwd against fp32 PyTorch on the same bf16 operands, and its saved projections."""
    from kernel_pocs_b200.fused_mlp import check_status
    from kernel_pocs_b200.geglu import gate_up_geglu_forward
    from tests.test_fused_gemm import assert_close_bf16

    g = torch.Generator(device=DEVICE).manual_seed(17)
    x = torch.randn(m, k, generator=g, device=DEVICE).bfloat16()
    wg = (2.0 * k ** -0.5 * torch.randn(n, k, generator=g, device=DEVICE)).bfloat16()
    wu = (k ** -0.5 * torch.randn(n, k, generator=g, device=DEVICE)).bfloat16()
    h, gate, up = gate_up_geglu_forward(x, wg, wu, approximate, save_preactivations=True)
    check_status(x.device)
    gate_ref, up_ref = x.float() @ wg.float().t(), x.float() @ wu.float().t()
    assert_close_bf16(gate, gate_ref, "gate")
    assert_close_bf16(up, up_ref, "up")
    assert_close_bf16(h, torch.nn.functional.gelu(gate_ref, approximate=approximate) * up_ref, "h")
    assert torch.equal(gate_up_geglu_forward(x, wg, wu, approximate), h)

"""Parity tests of the CUDA path, through the reference's call signature.

The first three tests keep the parametrisation of the reference's tests/test_swiglu.py
(:28-113: shapes, multipliers, preserve_inputs, dtypes with their tolerances, seeds and draw
order) and call ``swiglu`` / ``swiglu_packed`` exactly as it does.  On top of the reference's
``assert_close`` gates every case is held to the tighter contract of this implementation:

* fp16 / bf16: every output is within ONE ulp of the fp32 closed form rounded once into the
  I/O dtype (oracle variant "once"), at least 99.5 % of elements are bit-identical to it, and
  each is a correct rounding (<= 0.51 ulp) of the float64 truth;
* fp32: |error| <= 1e-6 * |truth| for h and dup, and <= 1e-6 * max(|truth|, |dh*dm*up*gm|) for
  dgate, whose derivative factor crosses zero near gate*gm = -1.278 so that a purely relative
  bound is meaningless there (the reference itself is off by 4e-3 relative at such points);
* against the reference's own rounding chain (oracle variant "chain", pinned to vectors made
  by the reference): at most 2 ulp apart in 16-bit types (3 in fewer than 1e-4 of the elements);
* the outer gate of the reference README, rtol = atol = 1e-3 against the float64 truth, which
  a correctly rounded bf16 value (relative error <= 2^-9) meets only together with atol, is
  applied to fp16 and fp32; for bf16 the reference test's own 3e-2 is the outer bound.

The remaining tests extend coverage to what the reference does not test: odd widths and token
counts, widths beyond its 65536-element row limit, misaligned and non-contiguous inputs,
aliasing semantics of the in-place backward, guard bands around outputs, empty tensors,
special values in 16-bit types, saturation tails, and direct calls through the C ABI.
"""
from pathlib import Path
import sys

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from kernels.swiglu import ForgeSwiGLUFunction
from kernels.swiglu import swiglu
from kernels.swiglu import swiglu_backward
from kernels.swiglu import swiglu_forward
from kernels.swiglu import swiglu_packed
from kernels.swiglu import torch_swiglu_packed_reference
from kernels.swiglu import torch_swiglu_reference

from kernel_pocs_b200 import _lib
from oracle import oracle as O
from tests._util import DTYPES, assert_rel_scaled, assert_rounded_once, assert_ulp, guarded

pytestmark = pytest.mark.gpu

DEVICE = "cuda"

REFERENCE_TOLERANCES = [
    (torch.float32, 1e-5, 1e-5),
    (torch.float16, 2e-2, 2e-2),
    (torch.bfloat16, 3e-2, 3e-2),
]


def _loaded_native_library() -> bool:
    return any("libswiglu_b200.so" in line for line in open("/proc/self/maps"))


def check_against_oracle(h, dgate, dup, gate, up, dout, gm, dm, what):
    """The tight contract described in the module docstring.  Inputs are the ORIGINAL gate/up."""
    dtype = gate.dtype
    gate, up, dout = gate.detach().cpu(), up.detach().cpu(), dout.detach().cpu()
    th = O.fwd_f64(gate, up, gm, dm)
    tdg, tdu, scale = O.bwd_f64(dout, gate, up, gm, dm)
    if dtype == torch.float32:
        assert_rel_scaled(h, th, 1e-6, f"{what} h")
        assert_rel_scaled(dup, tdu, 1e-6, f"{what} dup")
        assert_rel_scaled(dgate, tdg, 1e-6, f"{what} dgate", scale=scale)
        return
    oh = O.fwd(gate, up, gm, dm, "once")
    odg, odu = O.bwd(dout, gate, up, gm, dm, "once")
    assert_ulp(h, oh, 1, f"{what} h vs once", min_exact=0.995)
    assert_ulp(dup, odu, 1, f"{what} dup vs once", min_exact=0.995)
    assert_ulp(dgate, odg, 1, f"{what} dgate vs once", min_exact=0.995)
    assert_rounded_once(h, th, f"{what} h")
    assert_rounded_once(dup, tdu, f"{what} dup")
    assert_rounded_once(dgate, tdg, f"{what} dgate", extra=1e-6 * scale)
    ch = O.fwd(gate, up, gm, dm, "chain")
    cdg, cdu = O.bwd(dout, gate, up, gm, dm, "chain")
    for got, want, n in ((h, ch, "h"), (dup, cdu, "dup"), (dgate, cdg, "dgate")):
        # the reference's extra roundings through 16-bit intermediates: 2 ulp, a third only where an
        # intermediate is an fp16 subnormal (seen once in 3e5 elements of N(0, 2^2) data)
        assert_ulp(got, want, 3, f"{what} {n} vs reference chain")
        assert float((O.ulp_distance(got, want) > 2).double().mean()) <= 1e-4, f"{what} {n} vs reference chain"
    if dtype == torch.float16:
        for got, truth, n in ((h, th, "h"), (dup, tdu, "dup"), (dgate, tdg, "dgate")):
            torch.testing.assert_close(got.detach().cpu().double(), truth, rtol=1e-3, atol=1e-3, msg=f"{what} {n} README gate")


# --------------------------------------------------------------------------------------------
# the reference's own parametrisation
# --------------------------------------------------------------------------------------------

@pytest.mark.parametrize("shape", [(2, 8, 128), (1, 3, 257), (4, 5, 1024), (1, 2, 11008)])
@pytest.mark.parametrize("gate_multiplier, down_multiplier", [(1.0, 1.0), (0.7, 1.3)])
@pytest.mark.parametrize("preserve_inputs", [False, True])
@pytest.mark.parametrize("dtype, atol, rtol", REFERENCE_TOLERANCES)
def test_swiglu_forward_backward(shape, gate_multiplier, down_multiplier, preserve_inputs, dtype, atol, rtol):
    torch.manual_seed(0)
    gate_ref = torch.randn(*shape, device=DEVICE, dtype=dtype, requires_grad=True)
    up_ref = torch.randn(*shape, device=DEVICE, dtype=dtype, requires_grad=True)
    gate_forge = gate_ref.detach().clone().requires_grad_(True)
    up_forge = up_ref.detach().clone().requires_grad_(True)
    gate_before = gate_forge.detach().clone()
    up_before = up_forge.detach().clone()

    out_ref = torch_swiglu_reference(gate_ref, up_ref, gate_multiplier, down_multiplier)
    launches = _lib.launch_count()
    out_forge = swiglu(gate_forge, up_forge, gate_multiplier, down_multiplier, preserve_inputs)
    assert _lib.launch_count() == launches + 1, "the forward must be exactly one launch of this library"
    torch.testing.assert_close(out_forge, out_ref, atol=atol, rtol=rtol)

    grad = torch.randn_like(out_ref)
    out_ref.backward(grad)
    out_forge.backward(grad)
    assert _lib.launch_count() == launches + 2, "the backward must be exactly one launch of this library"

    torch.testing.assert_close(gate_forge.grad, gate_ref.grad, atol=atol, rtol=rtol)
    torch.testing.assert_close(up_forge.grad, up_ref.grad, atol=atol, rtol=rtol)

    if preserve_inputs:
        torch.testing.assert_close(gate_forge.detach(), gate_before, atol=0, rtol=0)
        torch.testing.assert_close(up_forge.detach(), up_before, atol=0, rtol=0)
    else:
        # the reference's in-place semantics: the gradients live in the inputs' storage
        assert gate_forge.grad.data_ptr() == gate_forge.data_ptr()
        assert up_forge.grad.data_ptr() == up_forge.data_ptr()

    check_against_oracle(out_forge, gate_forge.grad, up_forge.grad, gate_before, up_before, grad,
                         gate_multiplier, down_multiplier, f"{dtype} {shape}")
    assert _loaded_native_library()


@pytest.mark.parametrize("shape", [(2, 8, 256), (1, 3, 514)])
@pytest.mark.parametrize("gate_multiplier, down_multiplier", [(1.0, 1.0), (1.5, 0.5)])
@pytest.mark.parametrize("preserve_inputs", [False, True])
@pytest.mark.parametrize("dtype, atol, rtol", REFERENCE_TOLERANCES)
def test_swiglu_packed_forward_backward(shape, gate_multiplier, down_multiplier, preserve_inputs, dtype, atol, rtol):
    torch.manual_seed(1)
    gate_up_ref = torch.randn(*shape, device=DEVICE, dtype=dtype, requires_grad=True)
    gate_up_forge = gate_up_ref.detach().clone().requires_grad_(True)
    gate_up_before = gate_up_forge.detach().clone()

    out_ref = torch_swiglu_packed_reference(gate_up_ref, gate_multiplier, down_multiplier)
    out_forge = swiglu_packed(gate_up_forge, gate_multiplier, down_multiplier, preserve_inputs)
    torch.testing.assert_close(out_forge, out_ref, atol=atol, rtol=rtol)

    grad = torch.randn_like(out_ref)
    out_ref.backward(grad)
    out_forge.backward(grad)

    torch.testing.assert_close(gate_up_forge.grad, gate_up_ref.grad, atol=atol, rtol=rtol)
    if preserve_inputs:
        torch.testing.assert_close(gate_up_forge.detach(), gate_up_before, atol=0, rtol=0)

    gate, up = O.packed_split(gate_up_before.cpu())
    dgate, dup = O.packed_split(gate_up_forge.grad.cpu())
    check_against_oracle(out_forge, dgate, dup, gate, up, grad, gate_multiplier, down_multiplier,
                         f"packed {dtype} {shape}")


def test_swiglu_special_values_forward():
    gate = torch.tensor(
        [[[0.0, float("inf"), float("-inf"), float("nan"), 20.0, -20.0]]],
        device=DEVICE,
        dtype=torch.float32,
    )
    up = torch.tensor([[[1.0, 2.0, 3.0, 4.0, -1.0, -2.0]]], device=DEVICE, dtype=torch.float32)

    out_ref = torch_swiglu_reference(gate, up)
    out_forge = swiglu(gate, up, preserve_inputs=True)
    torch.testing.assert_close(out_forge, out_ref, atol=1e-12, rtol=1e-7, equal_nan=True)


# --------------------------------------------------------------------------------------------
# golden vectors produced by the reference itself
# --------------------------------------------------------------------------------------------

def test_matches_reference_vectors(golden_dir):
    z = np.load(golden_dir / "separate.npz")
    for key in sorted({k.rsplit("|", 1)[0] for k in z.files}):
        dname, _, gm, dm = key.split("|")
        dtype, gm, dm = DTYPES[dname], float(gm), float(dm)
        t = {n: O.from_numpy_bits(z[f"{key}|{n}"], dtype) for n in ["gate", "up", "dout", "h", "dgate", "dup"]}
        gate = t["gate"].to(DEVICE).requires_grad_(True)
        up = t["up"].to(DEVICE).requires_grad_(True)
        h = swiglu(gate, up, gm, dm, True)
        h.backward(t["dout"].to(DEVICE))
        if dtype == torch.float32:
            assert_ulp(h, t["h"], 8, f"{key} h")
            assert_ulp(up.grad, t["dup"], 8, f"{key} dup")
            scale = (t["dout"].double() * dm * t["up"].double() * gm).abs()
            assert_rel_scaled(gate.grad, t["dgate"].double(), 1e-6, f"{key} dgate", scale=scale)
        else:
            assert_ulp(h, t["h"], 2, f"{key} h")
            assert_ulp(up.grad, t["dup"], 2, f"{key} dup")
            assert_ulp(gate.grad, t["dgate"], 2, f"{key} dgate")

    z = np.load(golden_dir / "special.npz")
    for dname, dtype in DTYPES.items():
        gate, up, want = (O.from_numpy_bits(z[f"{dname}|{n}"], dtype) for n in ("gate", "up", "h"))
        got = swiglu_forward(gate.to(DEVICE), up.to(DEVICE))[0].cpu()
        assert torch.equal(torch.isnan(got), torch.isnan(want)), dname
        # fp32: exp and a reciprocal good to 1 ulp each, then two products
        assert_ulp(got, want, 4 if dtype == torch.float32 else 1, f"special values {dname}")


def test_config1_fp32(golden_dir):
    """fp32 [2,128,1024], seed 0, draw order gate, up, dh (the reference's CPU-runnable case)."""
    torch.manual_seed(0)
    gate0, up0, dout = (torch.randn(2, 128, 1024) for _ in range(3))
    gate = gate0.to(DEVICE).requires_grad_(True)
    up = up0.to(DEVICE).requires_grad_(True)
    h = swiglu(gate, up)
    h.backward(dout.to(DEVICE))
    check_against_oracle(h, gate.grad, up.grad, gate0, up0, dout, 1.0, 1.0, "config 1")
    ah, adg, adu = O.aten_fwd_bwd(gate0, up0, dout)
    torch.testing.assert_close(h.cpu(), ah, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(up.grad.cpu(), adu, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(gate.grad.cpu(), adg, rtol=1e-6, atol=1e-6)


# --------------------------------------------------------------------------------------------
# shapes and layouts the reference does not test
# --------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dname", ["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("shape", [(1, 1), (1, 7), (3, 1), (5, 9), (7, 1101), (13, 11009), (2, 65537), (1, 131080),
                                   (257, 1024), (33, 4104)])
@pytest.mark.parametrize("preserve_inputs", [False, True])
def test_odd_shapes_with_guard_bands(dname, shape, preserve_inputs):
    """Ragged widths and token counts, rows wider than the reference's 65536 limit; inputs drawn
    N(0, 2^2) to reach the saturation tails.  Outputs sit between sentinel bands."""
    dtype = DTYPES[dname]
    g = torch.Generator().manual_seed(2)
    gate0, up0, dout0 = ((2.0 * torch.randn(*shape, generator=g)).to(dtype) for _ in range(3))
    gate_buf, gate_guard = guarded(shape, dtype, DEVICE)
    up_buf, up_guard = guarded(shape, dtype, DEVICE)
    gate_buf.copy_(gate0)
    up_buf.copy_(up0)
    h, gate_2d, up_2d = swiglu_forward(gate_buf, up_buf, 0.9, 1.1)
    assert gate_2d.data_ptr() == gate_buf.data_ptr() and up_2d.data_ptr() == up_buf.data_ptr()
    dgate, dup = swiglu_backward(dout0.to(DEVICE), gate_2d, up_2d, 0.9, 1.1, preserve_inputs)
    torch.cuda.synchronize()
    gate_guard("gate/dgate")
    up_guard("up/dup")
    if preserve_inputs:
        assert torch.equal(gate_buf.cpu(), gate0) and torch.equal(up_buf.cpu(), up0)
    else:
        assert dgate.data_ptr() == gate_buf.data_ptr() and dup.data_ptr() == up_buf.data_ptr()
    check_against_oracle(h, dgate, dup, gate0, up0, dout0, 0.9, 1.1, f"{dname} {shape}")


@pytest.mark.parametrize("dname", ["bf16", "fp32"])
@pytest.mark.parametrize("offset", [1, 3, 4, 5, 8])
def test_misaligned_views(dname, offset):
    """Row slices of an odd-width tensor start at addresses that are not 16-byte aligned, and
    the freshly allocated output is aligned differently from the inputs."""
    dtype = DTYPES[dname]
    g = torch.Generator().manual_seed(7)
    width, rows = 1003, 9
    base_gate = torch.randn(rows * width + 16, generator=g).to(dtype).to(DEVICE)
    base_up = torch.randn(rows * width + 16, generator=g).to(dtype).to(DEVICE)
    gate = base_gate[offset:offset + rows * width].view(rows, width)
    up = base_up[offset:offset + rows * width].view(rows, width)
    dout = torch.randn(rows, width, generator=g).to(dtype).to(DEVICE)
    gate0, up0 = gate.cpu().clone(), up.cpu().clone()
    sentinel_gate, sentinel_up = base_gate.cpu().clone(), base_up.cpu().clone()
    h, gate_2d, up_2d = swiglu_forward(gate, up)
    # congruent misalignment of every tensor: dout sliced the same way, in-place gradients
    dout_base = torch.zeros(rows * width + 16, dtype=dtype, device=DEVICE)
    dout_view = dout_base[offset:offset + rows * width].view(rows, width)
    dout_view.copy_(dout)
    dgate, dup = swiglu_backward(dout_view, gate_2d, up_2d)
    check_against_oracle(h, dgate, dup, gate0, up0, dout.cpu(), 1.0, 1.0, f"misaligned {dname} +{offset}")
    # nothing outside the slices was touched
    assert torch.equal(base_gate.cpu()[:offset], sentinel_gate[:offset])
    assert torch.equal(base_gate.cpu()[offset + rows * width:], sentinel_gate[offset + rows * width:])
    assert torch.equal(base_up.cpu()[:offset], sentinel_up[:offset])
    assert torch.equal(base_up.cpu()[offset + rows * width:], sentinel_up[offset + rows * width:])


@pytest.mark.parametrize("dname", ["bf16", "fp32"])
def test_non_contiguous_inputs(dname):
    """Transposed inputs are compacted by the wrapper (as in the reference, swiglu.py:214-215);
    the caller's tensors are then never overwritten, whatever preserve_inputs says."""
    dtype = DTYPES[dname]
    g = torch.Generator().manual_seed(8)
    gate0 = torch.randn(48, 6, 40, generator=g).to(dtype)
    up0 = torch.randn(48, 6, 40, generator=g).to(dtype)
    dout0 = torch.randn(6, 48, 40, generator=g).to(dtype)
    gate = gate0.to(DEVICE).transpose(0, 1).requires_grad_(True)
    up = up0.to(DEVICE).transpose(0, 1).requires_grad_(True)
    assert not gate.is_contiguous()
    h = swiglu(gate, up)
    h.backward(dout0.to(DEVICE))
    assert torch.equal(gate.detach().cpu(), gate0.transpose(0, 1))
    check_against_oracle(h, gate.grad, up.grad, gate0.transpose(0, 1).contiguous(), up0.transpose(0, 1).contiguous(),
                         dout0, 1.0, 1.0, f"non-contiguous {dname}")


@pytest.mark.parametrize("dname", ["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("half_width", [1, 3, 5, 128, 257, 1000, 1001, 5503, 5504])
@pytest.mark.parametrize("preserve_inputs", [False, True])
def test_packed_widths(dname, half_width, preserve_inputs):
    """Packed gate|up with odd half-widths: the up half of every row is misaligned relative to
    the gate half, which the reference only exercises at width 257 (the ragged-row kernels; bases
    that are misaligned as well are in tests/test_ragged_rows.py)."""
    dtype = DTYPES[dname]
    g = torch.Generator().manual_seed(9)
    rows = 11
    gate_up0 = (2.0 * torch.randn(rows, 2 * half_width, generator=g)).to(dtype)
    dout0 = torch.randn(rows, half_width, generator=g).to(dtype)
    buf, guard = guarded((rows, 2 * half_width), dtype, DEVICE)
    buf.copy_(gate_up0)
    gate_up = buf.requires_grad_(True)
    h = swiglu_packed(gate_up, 1.5, 0.5, preserve_inputs)
    assert h.shape == (rows, half_width)
    h.backward(dout0.to(DEVICE))
    torch.cuda.synchronize()
    guard("packed gate_up")
    if preserve_inputs:
        assert torch.equal(gate_up.detach().cpu(), gate_up0)
    gate, up = O.packed_split(gate_up0)
    dgate, dup = O.packed_split(gate_up.grad.cpu())
    check_against_oracle(h, dgate, dup, gate, up, dout0, 1.5, 0.5, f"packed {dname} I={half_width}")


def test_empty_tensors():
    for shape in [(0, 128), (4, 0), (2, 0, 16)]:
        gate = torch.empty(*shape, device=DEVICE, dtype=torch.bfloat16, requires_grad=True)
        up = torch.empty(*shape, device=DEVICE, dtype=torch.bfloat16, requires_grad=True)
        before = _lib.launch_count()
        h = swiglu(gate, up)
        assert h.shape == gate.shape
        h.backward(torch.empty_like(h))
        assert gate.grad.shape == gate.shape and up.grad.shape == up.shape
        assert _lib.launch_count() == before
    gu = torch.empty(3, 0, device=DEVICE, requires_grad=True)
    assert swiglu_packed(gu).shape == (3, 0)


def test_autograd_contract():
    """ctx.save_for_backward(gate_2d, up_2d): contiguous 2-D views, gate first; five gradients."""
    gate = torch.randn(2, 3, 64, device=DEVICE, requires_grad=True)
    up = torch.randn(2, 3, 64, device=DEVICE, requires_grad=True)
    h = ForgeSwiGLUFunction.apply(gate, up, 0.7, 1.3, True)
    fn = h.grad_fn
    saved_gate, saved_up = fn.saved_tensors
    assert saved_gate.shape == (6, 64) and saved_up.shape == (6, 64)
    assert saved_gate.data_ptr() == gate.data_ptr() and saved_up.data_ptr() == up.data_ptr()
    assert fn.gate_multiplier == 0.7 and fn.down_multiplier == 1.3 and fn.preserve_inputs is True
    # multipliers and the flag receive no gradient
    out = ForgeSwiGLUFunction.backward(fn, torch.ones_like(h))
    assert len(out) == 5 and out[2:] == (None, None, None)
    dgate, dup = torch.autograd.grad(h, (gate, up), torch.ones_like(h))
    assert dgate.shape == gate.shape and dup.shape == up.shape
    assert torch.equal(dgate, out[0]) and torch.equal(dup, out[1])
    with pytest.raises(TypeError, match="Python scalar"):
        swiglu(gate, up, down_multiplier=torch.tensor(2.0))


def test_multipliers_are_runtime_values():
    """A new multiplier value must not change which kernel runs (the reference recompiles per
    value because its multipliers are compile-time constants, swiglu.py:65-67)."""
    gate = torch.randn(4, 512, device=DEVICE)
    up = torch.randn(4, 512, device=DEVICE)
    for gm, dm in [(1.0, 1.0), (0.31, 2.7), (-1.25, 1e-3), (3.0, -0.5)]:
        h = swiglu_forward(gate, up, gm, dm)[0]
        assert_rel_scaled(h, O.fwd_f64(gate.cpu(), up.cpu(), gm, dm), 1e-6, f"multipliers {gm},{dm}")


def test_saturation_tails_bf16():
    """|gate| up to ~90: sigmoid saturates to 0 and 1, exp over- and underflows."""
    g = torch.Generator().manual_seed(12)
    gate0 = (30.0 * torch.randn(64, 2048, generator=g)).to(torch.bfloat16)
    up0 = torch.randn(64, 2048, generator=g).to(torch.bfloat16)
    dout0 = torch.randn(64, 2048, generator=g).to(torch.bfloat16)
    gate = gate0.to(DEVICE).requires_grad_(True)
    up = up0.to(DEVICE).requires_grad_(True)
    h = swiglu(gate, up, 1.0, 1.0, True)
    h.backward(dout0.to(DEVICE))
    assert bool(torch.isfinite(h).all()) and bool(torch.isfinite(gate.grad).all())
    check_against_oracle(h, gate.grad, up.grad, gate0, up0, dout0, 1.0, 1.0, "saturation bf16")


def test_direct_c_abi_strided_call():
    """Calls swiglu_b200_fwd/bwd directly with row strides larger than the width (a column
    window of a wider matrix), a layout the Python wrappers never produce."""
    rows, cols, pitch = 17, 96, 160
    g = torch.Generator().manual_seed(13)
    big_gate = torch.randn(rows, pitch, generator=g).bfloat16().to(DEVICE)
    big_up = torch.randn(rows, pitch, generator=g).bfloat16().to(DEVICE)
    big_dout = torch.randn(rows, pitch, generator=g).bfloat16().to(DEVICE)
    out = torch.full((rows, pitch), 7.0, dtype=torch.bfloat16, device=DEVICE)
    dgate = torch.full((rows, pitch), 7.0, dtype=torch.bfloat16, device=DEVICE)
    dup = torch.full((rows, pitch), 7.0, dtype=torch.bfloat16, device=DEVICE)
    col0 = 32
    es = 2
    stream = torch.cuda.current_stream().cuda_stream
    off = col0 * es
    rc = _lib.lib.swiglu_b200_fwd(out.data_ptr() + off, big_gate.data_ptr() + off, big_up.data_ptr() + off, rows, cols,
                                  pitch, pitch, _lib.BF16, 1.0, 1.0, 0, stream)
    assert rc == 0
    rc = _lib.lib.swiglu_b200_bwd(dgate.data_ptr() + off, dup.data_ptr() + off, big_dout.data_ptr() + off,
                                  big_gate.data_ptr() + off, big_up.data_ptr() + off, rows, cols, pitch, pitch, pitch,
                                  _lib.BF16, 1.0, 1.0, 0, stream)
    assert rc == 0
    torch.cuda.synchronize()
    win = slice(col0, col0 + cols)
    check_against_oracle(out[:, win].cpu(), dgate[:, win].cpu(), dup[:, win].cpu(), big_gate[:, win].cpu(),
                         big_up[:, win].cpu(), big_dout[:, win].cpu(), 1.0, 1.0, "strided C ABI")
    for t in (out, dgate, dup):
        outside = torch.cat([t[:, :col0], t[:, col0 + cols:]], dim=1)
        assert bool((outside == 7.0).all())


def test_large_shape_properties():
    """Llama-3-8B MLP width at a token count that still checks in seconds on the host:
    row-permutation equivariance and bit-equality of split-by-rows against the whole."""
    g = torch.Generator(device=DEVICE).manual_seed(1)
    rows, width = 4096, 14336
    gate = torch.randn(rows, width, generator=g, device=DEVICE).bfloat16()
    up = torch.randn(rows, width, generator=g, device=DEVICE).bfloat16()
    dout = torch.randn(rows, width, generator=g, device=DEVICE).bfloat16()
    h = swiglu_forward(gate, up)[0]
    dgate, dup = swiglu_backward(dout, gate, up, preserve_inputs=True)
    # split by contiguous token rows (the multi-GPU partition) == whole
    for lo, hi in [(0, 1000), (1000, 1001), (1001, 4096)]:
        hp = swiglu_forward(gate[lo:hi], up[lo:hi])[0]
        dgp, dup_p = swiglu_backward(dout[lo:hi], gate[lo:hi], up[lo:hi], preserve_inputs=True)
        assert torch.equal(hp, h[lo:hi]) and torch.equal(dgp, dgate[lo:hi]) and torch.equal(dup_p, dup[lo:hi])
    # in place == out of place
    g2, u2 = gate.clone(), up.clone()
    dg2, du2 = swiglu_backward(dout, g2, u2)
    assert dg2.data_ptr() == g2.data_ptr() and torch.equal(dg2, dgate) and torch.equal(du2, dup)
    # a sample of rows against the oracle
    idx = torch.tensor([0, 1, 2047, 4095])
    check_against_oracle(h[idx], dgate[idx], dup[idx], gate[idx].cpu(), up[idx].cpu(), dout[idx].cpu(), 1.0, 1.0,
                         "14336-wide rows")
    # dup is linear in dh: doubling dh doubles dup exactly (power-of-two scaling is exact in bf16)
    _, dup2 = swiglu_backward(dout * 2, gate, up, preserve_inputs=True)
    assert torch.equal(dup2, dup * 2)


# --------------------------------------------------------------------------------------------
# host-buffer entry point
# --------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dname", ["bf16", "fp32"])
@pytest.mark.parametrize("rows,cols,ws_rows", [(1, 8, 1), (37, 1003, 5), (1000, 512, 64), (4096, 1024, 0)])
def test_host_buffer_pipeline_matches_device_path(dname, rows, cols, ws_rows):
    """Host tensors streamed through a small workspace (many chunks, ragged last chunk) give
    bit-identical results to the device-resident path, and leave the inputs untouched."""
    from kernel_pocs_b200.host_path import swiglu_fwd_bwd_host, workspace_bytes

    dtype = DTYPES[dname]
    g = torch.Generator().manual_seed(21)
    gate, up, dout = (torch.randn(rows, cols, generator=g).to(dtype).pin_memory() for _ in range(3))
    gate0, up0 = gate.clone(), up.clone()
    if ws_rows:
        # room for exactly ws_rows token rows per staged buffer: 3 slots x 4 buffers
        per = (ws_rows * cols * gate.element_size() + 255) // 256 * 256
        ws = torch.empty(12 * per, dtype=torch.uint8, device=DEVICE)
    else:
        ws = torch.empty(workspace_bytes(rows, cols, dtype), dtype=torch.uint8, device=DEVICE)
    before = _lib.launch_count()
    h, dgate, dup = swiglu_fwd_bwd_host(gate, up, dout, 0.9, 1.1, workspace=ws)
    torch.cuda.synchronize()
    chunks = -(-rows // ws_rows) if ws_rows else 1
    assert _lib.launch_count() - before == 2 * chunks
    assert torch.equal(gate, gate0) and torch.equal(up, up0)
    dh, dgate_ref, dup_ref = swiglu_forward(gate.to(DEVICE), up.to(DEVICE), 0.9, 1.1)[0], None, None
    dgate_ref, dup_ref = swiglu_backward(dout.to(DEVICE), gate.to(DEVICE), up.to(DEVICE), 0.9, 1.1, True)
    assert torch.equal(h, dh.cpu()) and torch.equal(dgate, dgate_ref.cpu()) and torch.equal(dup, dup_ref.cpu())
    check_against_oracle(h, dgate, dup, gate0, up0, dout, 0.9, 1.1, f"host path {dname} {rows}x{cols}")


def test_host_buffer_pipeline_rejects_bad_arguments():
    from kernel_pocs_b200.host_path import swiglu_fwd_bwd_host

    gate, up, dout = (torch.randn(4, 64).pin_memory() for _ in range(3))
    with pytest.raises(_lib.SwigluB200Error, match="workspace too small"):
        swiglu_fwd_bwd_host(gate, up, dout, workspace=torch.empty(256, dtype=torch.uint8, device=DEVICE))
    with pytest.raises(ValueError, match="host tensors"):
        swiglu_fwd_bwd_host(gate.to(DEVICE), up.to(DEVICE), dout.to(DEVICE))
    with pytest.raises(ValueError, match="shape and dtype"):
        swiglu_fwd_bwd_host(gate, up, dout[:2])
    torch.cuda.synchronize()


@pytest.mark.parametrize("dname", ["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("offsets", [(1, 0, 0), (0, 3, 5), (7, 2, 6), (4, 4, 1), (3, 3, 3)])
@pytest.mark.parametrize("n", [5, 24, 4099, 2 * 512 * 8 * 4 + 13, 300001])
def test_inputs_skewed_against_each_other(dname, offsets, n):
    """gate, up and dh each start a different number of elements past a 16-byte boundary while the
    freshly allocated outputs are aligned: the loads are realigned in registers (16-byte accesses
    plus a funnel shift), and nothing before or after any slice may be touched."""
    dtype = DTYPES[dname]
    g = torch.Generator().manual_seed(14)
    pad = 16
    bases = [(2.0 * torch.randn(n + 2 * pad, generator=g)).to(dtype).to(DEVICE) for _ in range(3)]
    snapshots = [b.clone() for b in bases]
    gate, up, dout = (b[pad + o: pad + o + n].view(1, n) for b, o in zip(bases, offsets))
    h, gate_2d, up_2d = swiglu_forward(gate, up, 0.8, 1.25)
    assert gate_2d.data_ptr() == gate.data_ptr()
    dgate, dup = swiglu_backward(dout, gate_2d, up_2d, 0.8, 1.25, preserve_inputs=True)
    torch.cuda.synchronize()
    for b, s in zip(bases, snapshots):
        assert torch.equal(b.view(torch.uint8), s.view(torch.uint8)), "an input buffer was modified"
    check_against_oracle(h, dgate, dup, gate.cpu(), up.cpu(), dout.cpu(), 0.8, 1.25, f"skew {offsets} {dname} n={n}")
    # in place: gradients over gate/up, dh skewed against them
    if offsets[0] == offsets[1]:
        g2, u2 = gate.clone(), up.clone()  # clones are aligned; dh keeps its offset
        dg2, du2 = swiglu_backward(dout, g2, u2, 0.8, 1.25)
        assert dg2.data_ptr() == g2.data_ptr()
        assert torch.equal(dg2, dgate) and torch.equal(du2, dup)


@pytest.mark.parametrize("name", ["c2", "c3", "c3-fp32", "c5"])
def test_full_size_workloads(name):
    """The benchmark configurations at their FULL sizes (c2: bf16 [32768, 14336]; c3: the 16 packed
    variable-length sequences, [68298, 11008], N(0, 2^2), in bf16 and in fp32; c5: bf16 [65536, 28672],
    3.76 GB per tensor, so byte offsets pass 2^32): sampled token rows from the start, the middle and the very
    end (for c3 also the first and last token of several sequences) against the oracle, and size-independent
    properties -- in place == out of place, a row range computed on its own == the same rows of the whole
    (the multi-GPU partition), dup linear in dh."""
    from kernel_pocs_b200 import workloads as W

    w = W.workloads()[name]
    need = 7 * w.tokens * w.width * torch.empty((), dtype=w.dtype).element_size()
    free, _total = torch.cuda.mem_get_info()
    if free < need + (4 << 30):
        pytest.skip(f"needs {need / 2**30:.0f} GiB of device memory")
    gate, up, dh = W.generate_rows(w, 0, w.tokens, DEVICE)
    h = swiglu_forward(gate, up)[0]
    dgate, dup = swiglu_backward(dh, gate, up, preserve_inputs=True)
    picks = [0, 1, w.tokens // 2 - 1, w.tokens // 2, w.tokens - 2, w.tokens - 1]
    if name.startswith("c3"):
        lens = W.varlen_lengths()
        assert sum(lens) == w.tokens
        starts = [sum(lens[:i]) for i in range(len(lens))]
        for i in (0, 3, 7, 11, 12, 15):  # sequence 11 is the shortest (434 tokens)
            picks += [starts[i], starts[i] + lens[i] - 1]
    rows = torch.tensor(sorted(set(picks)), device=DEVICE)
    check_against_oracle(h[rows], dgate[rows], dup[rows], gate[rows].cpu(), up[rows].cpu(), dh[rows].cpu(), 1.0, 1.0,
                         f"{name} sampled rows")
    # a shard of rows that starts beyond the 4 GiB mark (for c5) computed on its own
    lo, hi = W.row_shard(w.tokens, 8, 7)
    hs = swiglu_forward(gate[lo:hi], up[lo:hi])[0]
    dgs, dus = swiglu_backward(dh[lo:hi], gate[lo:hi], up[lo:hi], preserve_inputs=True)
    assert torch.equal(hs, h[lo:hi]) and torch.equal(dgs, dgate[lo:hi]) and torch.equal(dus, dup[lo:hi])
    del hs, dgs, dus
    # the generator reproduces the shard bit for bit on its own (what each GPU of a multi-GPU run holds)
    g2, u2, d2 = W.generate_rows(w, lo, hi, DEVICE)
    assert torch.equal(g2, gate[lo:hi]) and torch.equal(u2, up[lo:hi]) and torch.equal(d2, dh[lo:hi])
    del g2, u2, d2
    # linearity of dup in dh (exact for a power-of-two factor), then in place == out of place
    dh.mul_(2)
    _, dup2 = swiglu_backward(dh, gate, up, preserve_inputs=True)
    dh.mul_(0.5)
    assert torch.equal(dup2, dup * 2)
    del dup2
    dg_inplace, du_inplace = swiglu_backward(dh, gate, up)  # overwrites gate/up
    assert dg_inplace.data_ptr() == gate.data_ptr()
    assert torch.equal(dg_inplace, dgate) and torch.equal(du_inplace, dup)


def test_randomised_shapes_alignments_and_modes():
    """300 seeded random cases over dtype, element count (around tile, warp and vector boundaries),
    per-tensor misalignment, multipliers and backward mode, each compared bit for bit with a run of the same
    data from aligned, freshly allocated tensors (the plain vector path, itself checked against the oracle
    elsewhere) and, every tenth case, with the oracle directly."""
    rng = np.random.default_rng(1234)
    specials = [1, 2, 7, 8, 9, 15, 16, 17, 31, 32, 33, 255, 256, 257, 511, 512, 513, 2047, 2048, 2049, 4095, 4096, 4097,
                8 * 512 * 4 - 1, 8 * 512 * 4, 8 * 512 * 4 + 1, 8 * 512 * 2 * 3 + 5, 4 * 512 * 4 * 2 + 3, 100003]
    for case in range(300):
        dtype = [torch.bfloat16, torch.float16, torch.float32][case % 3]
        n = int(rng.choice(specials)) if rng.random() < 0.7 else int(rng.integers(1, 60000))
        offs = [int(o) for o in rng.integers(0, 9, size=3)]
        if rng.random() < 0.3:
            offs = [offs[0]] * 3
        gm, dm = (1.0, 1.0) if rng.random() < 0.5 else (float(rng.uniform(0.5, 1.5)), float(rng.uniform(0.5, 1.5)))
        g = torch.Generator().manual_seed(case)
        src = [(1.5 * torch.randn(n, generator=g)).to(dtype) for _ in range(3)]
        pad = 16
        bufs = [torch.zeros(n + 2 * pad, dtype=dtype, device=DEVICE) for _ in range(3)]
        views = []
        for b, o, t in zip(bufs, offs, src):
            v = b[pad + o: pad + o + n]
            v.copy_(t)
            views.append(v.view(1, n))
        gate, up, dout = views
        what = f"case {case}: {dtype} n={n} offsets={offs} gm={gm:.3f} dm={dm:.3f}"
        # reference run from aligned tensors
        ag, au, ad = (t.to(DEVICE).view(1, n) for t in src)
        h_ref = swiglu_forward(ag, au, gm, dm)[0]
        dg_ref, du_ref = swiglu_backward(ad, ag, au, gm, dm, preserve_inputs=True)
        # misaligned inputs, aligned outputs
        h = swiglu_forward(gate, up, gm, dm)[0]
        dg, du = swiglu_backward(dout, gate, up, gm, dm, preserve_inputs=True)
        assert torch.equal(h, h_ref) and torch.equal(dg, dg_ref) and torch.equal(du, du_ref), what
        if case % 10 == 0:
            check_against_oracle(h, dg, du, src[0].view(1, n), src[1].view(1, n), src[2].view(1, n), gm, dm, what)
        # in place over the misaligned gate/up (needs gate and up aligned alike to stay on a vector path, but
        # must be right either way), then the guard bands around all three buffers
        dg2, du2 = swiglu_backward(dout, gate, up, gm, dm)
        assert dg2.data_ptr() == gate.data_ptr(), what
        assert torch.equal(dg2, dg_ref) and torch.equal(du2, du_ref), what
        for b, o in zip(bufs, offs):
            assert bool((b[: pad + o] == 0).all()) and bool((b[pad + o + n:] == 0).all()), what + " wrote outside"

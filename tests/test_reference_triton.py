"""This library against the reference's own Triton kernels on the same GPU, same seeded inputs.

The comparator is the unmodified copy of the reference's ``kernels/swiglu/swiglu.py`` that
``benchmarks/fetch_reference.py`` places under ``baseline/_ref`` (git-ignored).  When the copy is
absent, or Triton cannot compile for this GPU, the tests skip: the parity of record is the one
against the CPU oracle, which is pinned to vectors produced by the reference itself.

Shapes, seeds, draw order and multipliers are those of the reference's tests/test_swiglu.py:28-99.
With unit multipliers the two implementations differ only in how often they round (once here;
twice or three times through 16-bit intermediates in the Triton kernels, swiglu.py:75-82 and
:102-116), so they are held to 2 ulp in fp16/bf16 (a third ulp, where an intermediate of the
reference is an fp16 subnormal, in at most one element in ten thousand) and to the reference's
1e-5 in fp32.  With multipliers (0.7, 1.3) the Triton in this image also rounds the multiplier
itself to the tile's 16-bit type, so only the reference test file's own tolerances (2e-2 fp16,
3e-2 bf16) apply.
"""
from __future__ import annotations

import pytest
import torch

from benchmarks import fetch_reference
from oracle import oracle as O
from tests._util import assert_ulp

pytestmark = pytest.mark.gpu

SHAPES = [(2, 8, 128), (1, 3, 257), (4, 5, 1024), (1, 2, 11008)]
PACKED_SHAPES = [(2, 8, 256), (1, 3, 514)]
DTYPE_TOL = [(torch.float32, 1e-5), (torch.float16, 2e-2), (torch.bfloat16, 3e-2)]


@pytest.fixture(scope="module")
def ref():
    if not fetch_reference.available():
        pytest.skip("baseline/_ref is absent (benchmarks/fetch_reference.py --reference <checkout> creates it)")
    try:
        module = fetch_reference.load()
        x = torch.randn(4, 64, device="cuda")
        module.swiglu(x, x.clone())  # first JIT: proves that Triton can compile for this GPU
        torch.cuda.synchronize()
    except Exception as exc:  # no Triton for this architecture, no host compiler, ...
        pytest.skip(f"the reference's Triton kernels do not run here: {type(exc).__name__}: {exc}")
    return module


def assert_two_ulp(got, want, what):
    assert_ulp(got, want, 3, what)
    beyond = int((O.ulp_distance(got, want) > 2).sum())
    assert beyond <= max(1, got.numel() // 10000), f"{what}: {beyond} elements more than 2 ulp apart"


def _run(op, inputs, dout, *args):
    leaves = [t.detach().clone().requires_grad_(True) for t in inputs]
    out = op(*leaves, *args)
    grads = torch.autograd.grad(out, leaves, dout)
    return (out.detach(), *grads)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("preserve_inputs", [False, True])
@pytest.mark.parametrize("dtype,tol", DTYPE_TOL)
def test_unit_multipliers_within_two_ulp_of_the_triton_kernels(ref, shape, preserve_inputs, dtype, tol):
    from kernels.swiglu import swiglu

    torch.manual_seed(0)
    gate = torch.randn(*shape, device="cuda", dtype=dtype)
    up = torch.randn(*shape, device="cuda", dtype=dtype)
    dout = torch.randn(*shape, device="cuda", dtype=dtype)
    want = _run(ref.swiglu, (gate, up), dout, 1.0, 1.0, preserve_inputs)
    got = _run(swiglu, (gate, up), dout, 1.0, 1.0, preserve_inputs)
    for name, g, w in zip(("h", "dgate", "dup"), got, want):
        if dtype == torch.float32:
            torch.testing.assert_close(g, w, rtol=tol, atol=tol, msg=lambda m: f"{name}: {m}")
        else:
            assert_two_ulp(g, w, f"{name} vs the reference's Triton kernel")


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype,tol", DTYPE_TOL)
def test_scaled_multipliers_within_the_reference_tolerances(ref, shape, dtype, tol):
    from kernels.swiglu import swiglu

    torch.manual_seed(0)
    gate = torch.randn(*shape, device="cuda", dtype=dtype)
    up = torch.randn(*shape, device="cuda", dtype=dtype)
    dout = torch.randn(*shape, device="cuda", dtype=dtype)
    want = _run(ref.swiglu, (gate, up), dout, 0.7, 1.3, True)
    got = _run(swiglu, (gate, up), dout, 0.7, 1.3, True)
    for name, g, w in zip(("h", "dgate", "dup"), got, want):
        torch.testing.assert_close(g, w, rtol=tol, atol=tol, msg=lambda m: f"{name}: {m}")


@pytest.mark.parametrize("shape", PACKED_SHAPES)
@pytest.mark.parametrize("multipliers", [(1.0, 1.0), (1.5, 0.5)])
@pytest.mark.parametrize("dtype,tol", DTYPE_TOL)
def test_packed_layout_against_the_triton_kernels(ref, shape, multipliers, dtype, tol):
    from kernels.swiglu import swiglu_packed

    torch.manual_seed(1)
    gate_up = torch.randn(*shape, device="cuda", dtype=dtype)
    dout = torch.randn(*shape[:-1], shape[-1] // 2, device="cuda", dtype=dtype)
    want = _run(ref.swiglu_packed, (gate_up,), dout, *multipliers, True)
    got = _run(swiglu_packed, (gate_up,), dout, *multipliers, True)
    for name, g, w in zip(("h", "dgate_up"), got, want):
        if multipliers == (1.0, 1.0) and dtype != torch.float32:
            assert_two_ulp(g, w, f"packed {name} vs the reference's Triton kernel")
        else:
            torch.testing.assert_close(g, w, rtol=tol, atol=tol, msg=lambda m: f"{name}: {m}")


def test_large_bf16_block_against_the_triton_kernels(ref):
    """4096 token rows of the Llama-3-8B width, N(0,1): every element within 2 ulp, in-place mode."""
    from kernels.swiglu import swiglu_backward, swiglu_forward

    g = torch.Generator(device="cuda").manual_seed(11)
    gate, up, dout = (torch.randn(4096, 14336, generator=g, device="cuda").bfloat16() for _ in range(3))
    h_ref, gate_r, up_r = ref.swiglu_forward(gate.clone(), up.clone())
    dgate_ref, dup_ref = ref.swiglu_backward(dout, gate_r, up_r)
    h, gate_o, up_o = swiglu_forward(gate.clone(), up.clone())
    dgate, dup = swiglu_backward(dout, gate_o, up_o)
    for name, got, want in (("h", h, h_ref), ("dgate", dgate, dgate_ref), ("dup", dup, dup_ref)):
        assert_two_ulp(got, want, f"{name} vs the reference's Triton kernel")


# ---- the sibling operator: GeGLU (reference kernels/geglu/geglu.py, tests/test_geglu.py:32-69) ----

@pytest.fixture(scope="module")
def ref_geglu():
    if not fetch_reference.available("geglu"):
        pytest.skip("baseline/_ref/kernels/geglu is absent (benchmarks/fetch_reference.py creates it)")
    try:
        module = fetch_reference.load("geglu")
        x = torch.randn(4, 64, device="cuda")
        module.geglu(x, x.clone())
        torch.cuda.synchronize()
    except Exception as exc:
        pytest.skip(f"the reference's Triton GeGLU kernels do not run here: {type(exc).__name__}: {exc}")
    return module


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("approximate", ["tanh", "none"])
@pytest.mark.parametrize("preserve_inputs", [False, True])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float16, 2e-2), (torch.bfloat16, 3e-2)])
def test_geglu_within_the_reference_tolerances_of_its_triton_kernels(ref_geglu, shape, approximate, preserve_inputs,
                                                                      dtype, tol):
    """Shapes, seed, draw order and tolerances of the reference's own GeGLU test; the comparator there is the
    PyTorch composite, here it is the reference's Triton kernel itself."""
    from kernels.geglu import geglu

    torch.manual_seed(0)
    gate = torch.randn(*shape, device="cuda", dtype=dtype)
    up = torch.randn(*shape, device="cuda", dtype=dtype)
    dout = torch.randn(*shape, device="cuda", dtype=dtype)
    want = _run(ref_geglu.geglu, (gate, up), dout, approximate, preserve_inputs)
    got = _run(geglu, (gate, up), dout, approximate, preserve_inputs)
    for name, g, w in zip(("h", "dgate", "dup"), got, want):
        torch.testing.assert_close(g, w, rtol=tol, atol=tol, msg=lambda m: f"{name}: {m}")


@pytest.mark.parametrize("approximate", ["tanh", "none"])
def test_geglu_large_bf16_block_against_the_triton_kernels(ref_geglu, approximate):
    """4096 token rows of the Llama-3-8B width, N(0,1), in-place mode, both implementations beside the float64
    value of the formula.  This library is within one bf16 ulp of it everywhere.  The reference's kernels evaluate
    0.5 * (1 + tanh(.)) and 0.5 * (1 + erf(.)), which cancel for gates below about -4.5: there (a hundred-odd
    elements of 59 million) they are tens to thousands of ulp off, down to a flushed zero.  So the two are compared
    where the reference is itself within 2 ulp of the formula (3 ulp apart at most), and the elements where it is
    not must stay that rare."""
    from kernels.geglu import geglu_backward, geglu_forward

    g = torch.Generator(device="cuda").manual_seed(12)
    gate, up, dout = (torch.randn(4096, 14336, generator=g, device="cuda").bfloat16() for _ in range(3))
    h_ref, gate_r, up_r = ref_geglu.geglu_forward(gate.clone(), up.clone(), approximate)
    dgate_ref, dup_ref = ref_geglu.geglu_backward(dout, gate_r, up_r, approximate)
    h, gate_o, up_o = geglu_forward(gate.clone(), up.clone(), approximate)
    dgate, dup = geglu_backward(dout, gate_o, up_o, approximate)
    x, u, d = gate.double(), up.double(), dout.double()
    if approximate == "tanh":
        c = 0.7978845608028654
        t = torch.tanh(c * (x + 0.044715 * x ** 3))
        cdf, dcdf = 0.5 * (1 + t), 0.5 * (1 - t * t) * c * (1 + 3 * 0.044715 * x * x)
        # 1 + tanh in float64 still cancels below -19; N(0,1) bf16 draws stay far above that
    else:
        cdf = 0.5 * torch.special.erfc(-x / 2 ** 0.5)
        dcdf = torch.exp(-0.5 * x * x) / (2 * 3.141592653589793) ** 0.5
    truth = {"h": x * cdf * u, "dgate": d * u * (cdf + x * dcdf), "dup": d * x * cdf}
    del x, u, d, cdf, dcdf
    for name, got, want in (("h", h, h_ref), ("dgate", dgate, dgate_ref), ("dup", dup, dup_ref)):
        exact = truth.pop(name).bfloat16()
        got, want = got.reshape(exact.shape), want.reshape(exact.shape)
        assert_ulp(got, exact, 1, f"geglu[{approximate}] {name} vs the float64 formula")
        ref_ok = O.ulp_distance(want, exact) <= 2
        assert int((~ref_ok).sum()) <= got.numel() // 100000, f"{name}: the reference is off in too many elements"
        apart = O.ulp_distance(got, want)
        assert int(apart[ref_ok].max()) <= 3, f"geglu[{approximate}] {name} vs the reference's Triton kernel"


# ---- the LoRA + SwiGLU epilogue (reference kernels/lora_mlp/experiments/v3/lora_mlp_kernel_v3.py:141-200) ----

@pytest.fixture(scope="module")
def ref_lora():
    if not fetch_reference.available("lora_v3"):
        pytest.skip("baseline/_ref/kernels/lora_mlp/experiments/v3 is absent (benchmarks/fetch_reference.py creates it)")
    try:
        module = fetch_reference.load("lora_v3")
        e = torch.randn(64, 64, device="cuda").bfloat16()
        a = torch.randn(64, 16, device="cuda").bfloat16()
        module.fused_lora_swiglu(e, e.clone(), a, a.clone(), a.clone(), a.clone())
        torch.cuda.synchronize()
    except Exception as exc:
        pytest.skip(f"the reference's Triton LoRA epilogue does not run here: {type(exc).__name__}: {exc}")
    return module


@pytest.mark.parametrize("m,n,r", [(128, 64, 16), (200, 200, 24), (333, 1096, 32), (1000, 4104, 64), (4096, 14336, 16)])
@pytest.mark.parametrize("save_eg", [False, True])
def test_lora_epilogue_against_the_triton_kernel(ref_lora, m, n, r, save_eg):
    """Same bf16 operands through the reference's fused_lora_swiglu and this library's.  Both accumulate the rank-r
    products in fp32 and round e, g and h once, but sum the ranks in different orders, so they are held to one
    bf16 rounding of each other plus accumulation noise (the bound the fused-GEMM tests use against fp32)."""
    from kernel_pocs_b200.fused_mlp import check_status
    from kernel_pocs_b200.lora_mlp import fused_lora_swiglu
    from tests.test_fused_gemm import assert_close_bf16

    g = torch.Generator(device="cuda").manual_seed(41)
    mk = lambda *shape, std=1.0: (std * torch.randn(*shape, generator=g, device="cuda")).bfloat16()
    e, gg, xag, xau, bg, bu = mk(m, n, std=1.5), mk(m, n), mk(m, r), mk(m, r), mk(n, r, std=0.3), mk(n, r, std=0.3)
    want = ref_lora.fused_lora_swiglu(e, gg, xag, xau, bg, bu, 2.0, 0.5, save_eg=save_eg)
    got = fused_lora_swiglu(e, gg, xag, xau, bg, bu, 2.0, 0.5, save_eg=save_eg)
    check_status(e.device)
    for name, a, b in zip(("h", "e", "g"), got, want):
        if b is None:
            assert a is None
        else:
            assert_close_bf16(a, b.float(), f"{name} vs the reference's Triton kernel")


# ---- the fused gate/up projection (reference kernels/lora_mlp/experiments/v2/lora_mlp_kernel_v2.py:145-209) ----

@pytest.mark.parametrize("with_adapters", [False, True])
def test_fused_projection_against_the_triton_dual_gemm(with_adapters):
    """The reference's own attempt at this fusion, an autotuned Triton dual GEMM with the adapters and SwiGLU in its
    epilogue, on the same bf16 operands: both accumulate in fp32 and round h, e and g once, in different orders
    of summation, so they are held to the bound the fused-GEMM tests use against the fp32 product."""
    if not fetch_reference.available("lora_v2"):
        pytest.skip("baseline/_ref/kernels/lora_mlp/experiments/v2 is absent (benchmarks/fetch_reference.py creates it)")
    from kernel_pocs_b200 import fused_mlp as F
    from tests.test_fused_gemm import assert_close_bf16

    m, n, k, r = 640, 1040, 520, 16
    g = torch.Generator(device="cuda").manual_seed(43)
    mk = lambda *shape, std=1.0: (std * torch.randn(*shape, generator=g, device="cuda")).bfloat16()
    x, wg, wu = mk(m, k), mk(n, k, std=k ** -0.5), mk(n, k, std=k ** -0.5)
    ag, au, bg, bu = mk(r, k, std=k ** -0.5), mk(r, k, std=k ** -0.5), mk(n, r, std=0.3), mk(n, r, std=0.3)
    try:
        ref = fetch_reference.load("lora_v2")
        if with_adapters:
            want = ref.fused_gate_up_swiglu(x, wg, ag, bg, 2.0, wu, au, bu, 0.5, save_pre_act=True)
        else:
            want = ref.fused_gate_up_swiglu(x, wg, None, None, 1.0, wu, None, None, 1.0, save_pre_act=True)
        torch.cuda.synchronize()
    except Exception as exc:
        pytest.skip(f"the reference's Triton dual GEMM does not run here: {type(exc).__name__}: {exc}")
    if with_adapters:
        got = F.lora_gate_up_swiglu_forward(x, wg, wu, ag, bg, 2.0, au, bu, 0.5, save_eg=True)
    else:
        got = F.gate_up_swiglu_forward(x, wg, wu, save_preactivations=True)
    F.check_status(x.device)
    for name, a, b in zip(("h", "e", "g"), got, want):
        assert_close_bf16(a, b.float(), f"{name} vs the reference's Triton dual GEMM")

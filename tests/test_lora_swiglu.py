"""LoRA + SwiGLU epilogue (TMA-fed tcgen05 kernel) against the formula of the reference's fused_lora_swiglu
(kernels/lora_mlp/experiments/v3/lora_mlp_kernel_v3.py:141-200), evaluated in fp32 PyTorch on the same bf16
operands:  e = E + s_gate * (XAg @ Bg^T),  g = G + s_up * (XAu @ Bu^T),  h = silu(e) * g.
The reference's own implementation of this step is a Triton kernel and cannot run without a GPU, so no
vectors produced by it exist (tests/test_reference_triton.py compares with it directly where its copy and a
GPU are there): parity for this operator is against the formula (as in the reference's own test,
kernels/lora_mlp/tests/test_lora_mlp.py, which compares with a PyTorch composite), with the bound used for
the fused GEMM: one bf16 rounding plus accumulation noise,  |err| <= 2^-7 |ref| + 2^-9 rms(ref)."""
import pytest
import torch

from kernel_pocs_b200 import _lib
from kernel_pocs_b200.fused_mlp import check_status
from kernel_pocs_b200.lora_mlp import fused_lora_swiglu, fused_lora_swiglu_inplace
from tests.test_fused_gemm import assert_close_bf16

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def operands(m, n, r, seed=4):
    g = torch.Generator(device=DEVICE).manual_seed(seed)
    mk = lambda *shape, std=1.0: (std * torch.randn(*shape, generator=g, device=DEVICE)).bfloat16()
    return mk(m, n, std=1.5), mk(m, n), mk(m, r), mk(m, r), mk(n, r, std=0.3), mk(n, r, std=0.3)


def reference(e, g, xag, xau, bg, bu, sg, su):
    ef = e.float() + sg * (xag.float() @ bg.float().t())
    gf = g.float() + su * (xau.float() @ bu.float().t())
    return torch.nn.functional.silu(ef) * gf, ef, gf


# The last four shapes have enough tiles for the kernel's longer runs of tiles per CTA (two at every rank, eight
# at rank 64 with e and g written, four on the 8192 x 11008 case) and for rows of tiles that end inside a run.
@pytest.mark.parametrize("m,n,r", [(128, 64, 16), (128, 1024, 16), (256, 2048, 8), (1, 8, 8), (200, 200, 24),
                                   (333, 1096, 32), (1000, 4104, 64), (4096, 14336, 16), (4100, 14344, 32),
                                   (8192, 11008, 64), (16384, 14336, 64), (16300, 9480, 16)])
@pytest.mark.parametrize("save_eg", [False, True])
def test_matches_formula(m, n, r, save_eg):
    e, g, xag, xau, bg, bu = operands(m, n, r)
    e0, g0 = e.clone(), g.clone()
    before = _lib.lib.swiglu_b200_lora_launch_count()
    h, e_full, g_full = fused_lora_swiglu(e, g, xag, xau, bg, bu, 2.0, 0.5, save_eg=save_eg)
    check_status(e.device)
    assert _lib.lib.swiglu_b200_lora_launch_count() == before + 1
    assert torch.equal(e, e0) and torch.equal(g, g0), "inputs must not be modified"
    rh, re, rg = reference(e, g, xag, xau, bg, bu, 2.0, 0.5)
    assert h.shape == (m, n) and h.dtype == torch.bfloat16
    assert_close_bf16(h, rh, "h")
    if save_eg:
        assert_close_bf16(e_full, re, "e_full")
        assert_close_bf16(g_full, rg, "g_full")
    else:
        assert e_full is None and g_full is None


def test_two_calls_and_no_adapter_path():
    e, g, xag, xau, bg, bu = operands(384, 1152, 16, seed=8)
    h1, _, _ = fused_lora_swiglu(e, g, xag, xau, bg, bu, 1.0, 1.0)
    h2, e_full, g_full = fused_lora_swiglu(e, g, xag, xau, bg, bu, 1.0, 1.0, save_eg=True)
    check_status(e.device)
    assert torch.equal(h1, h2)
    # zero adapters reduce to plain SwiGLU of the base projections, bit for bit with the streaming kernel
    from kernels.swiglu import swiglu_forward

    h0, _, _ = fused_lora_swiglu(e, g, torch.zeros_like(xag), torch.zeros_like(xau), bg, bu)
    check_status(e.device)
    assert torch.equal(h0, swiglu_forward(e, g)[0])
    hn, en, gn = fused_lora_swiglu(e, g, None, None, None, None, save_eg=True)
    assert torch.equal(hn, h0) and en is e and gn is g


def test_argument_errors():
    e, g, xag, xau, bg, bu = operands(128, 64, 16)
    with pytest.raises(TypeError, match="one dtype"):
        fused_lora_swiglu(e, g, xag.float(), xau.float(), bg, bu)
    with pytest.raises(ValueError, match="shape"):
        fused_lora_swiglu(e, g, xag, xau, bg[:32].contiguous(), bu)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fused_lora_swiglu(e.cpu(), g.cpu(), xag.cpu(), xau.cpu(), bg.cpu(), bu.cpu())


@pytest.mark.parametrize("dtype,r,n", [(torch.float32, 16, 64), (torch.float16, 8, 200), (torch.bfloat16, 12, 64),
                                       (torch.bfloat16, 16, 36), (torch.bfloat16, 72, 128)])
def test_other_dtypes_and_ranks_take_library_gemms(dtype, r, n):
    """fp32 / fp16 (the reference's kernel takes them, lora_mlp_kernel_v3.py:141-200 has no dtype check) and ranks
    or widths outside what the tensor-core epilogue handles: same results, no launch of that kernel."""
    e, g, xag, xau, bg, bu = (t.to(dtype) for t in operands(160, n, 80, seed=13))
    xag, xau, bg, bu = (t[:, :r].contiguous() for t in (xag, xau, bg, bu))
    e0 = e.clone()
    before = _lib.lib.swiglu_b200_lora_launch_count()
    h, e_full, g_full = fused_lora_swiglu(e, g, xag, xau, bg, bu, 2.0, 0.5, save_eg=True)
    assert _lib.lib.swiglu_b200_lora_launch_count() == before
    assert torch.equal(e, e0), "inputs must not be modified"
    rh, re, rg = reference(e, g, xag, xau, bg, bu, 2.0, 0.5)
    if dtype == torch.float32:
        torch.testing.assert_close(h, rh, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(e_full, re, rtol=1e-4, atol=1e-4)
    else:
        # h is computed from the ROUNDED e and g here (they are materialised in the I/O dtype)
        rh16 = torch.nn.functional.silu(e_full.float()) * g_full.float()
        # the library's 16-bit addmm_ may round the product before it adds e: errors scale with the terms, not the sum
        eps = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
        assert bool(((e_full.float() - re).abs() <= eps * (re.abs() + re.pow(2).mean().sqrt())).all()), "e_full"
        torch.testing.assert_close(h.float(), rh16, rtol=2.0 ** -7, atol=1e-3)
    e2 = e.clone()
    h2, e_in, _ = fused_lora_swiglu_inplace(e2, g.clone(), xag, xau, bg, bu, 2.0, 0.5, save_eg=True)
    assert e_in.data_ptr() == e2.data_ptr() and torch.equal(h2, h) and torch.equal(e_in, e_full)


@pytest.mark.parametrize("m,n,r", [(200, 200, 24), (1024, 4104, 16)])
def test_inplace_variant(m, n, r):
    """e_full / g_full written over e_base / g_base (reference v6:81-160) equal the out-of-place results."""
    e, g, xag, xau, bg, bu = operands(m, n, r, seed=11)
    h_ref, e_ref, g_ref = fused_lora_swiglu(e, g, xag, xau, bg, bu, 2.0, 0.5, save_eg=True)
    e2, g2 = e.clone(), g.clone()
    h, e_full, g_full = fused_lora_swiglu_inplace(e2, g2, xag, xau, bg, bu, 2.0, 0.5, save_eg=True)
    check_status(e.device)
    assert e_full.data_ptr() == e2.data_ptr() and g_full.data_ptr() == g2.data_ptr()
    assert torch.equal(h, h_ref) and torch.equal(e_full, e_ref) and torch.equal(g_full, g_ref)
    # without save_eg nothing is overwritten
    e3 = e.clone()
    h3, none_e, none_g = fused_lora_swiglu_inplace(e3, g.clone(), xag, xau, bg, bu, 2.0, 0.5)
    check_status(e.device)
    assert none_e is None and none_g is None and torch.equal(e3, e) and torch.equal(h3, h_ref)

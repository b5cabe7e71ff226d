"""LoRA + SwiGLU epilogue: ``h = silu(e_base + s_gate * xa_gate @ B_gate.T) * (g_base + s_up * xa_up @ B_up.T)``.

Mirrors ``fused_lora_swiglu`` of the reference (kernels/lora_mlp/experiments/v3/lora_mlp_kernel_v3.py:141-200;
same argument order, same return triple), the one kernel of its LoRA-MLP forward that is not a library GEMM:
the base projections and the skinny ``x @ A.T`` products stay with cuBLAS, and this step adds the rank-r
adapter terms and applies SwiGLU in one pass over e and g.  Here it is a TMA-fed tcgen05 kernel
(``swiglu_b200_lora_swiglu_fwd``) for bf16 with a rank that is a multiple of 8 up to 64; other dtypes and
ranks take library GEMMs for the adapter terms followed by the streaming SwiGLU kernel.

``LoRAMLP`` / ``lora_mlp`` are the whole block with the interface of the reference's ``LoRAMLPv3`` /
``lora_mlp_v3`` (same file, :244-357).  Forward: for bf16 the gate and up projections, both adapters and SwiGLU
are ONE tcgen05 launch (``swiglu_b200_lora_gemm_fwd``, what the reference's v2 attempted in Triton); other
dtypes and ranks take library GEMMs and the epilogue above, in place over the base projections as in the
reference's v6.  Backward: library GEMMs around one elementwise pass (``swiglu_b200_bwd_recompute``) that turns
(dh, e, g) into (h, de, dg).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .fused_mlp import _launching
from .swiglu import _as_float, swiglu_backward_recompute, swiglu_forward


def fused_lora_swiglu_inplace(
    e_base: torch.Tensor,
    g_base: torch.Tensor,
    xa_gate: Optional[torch.Tensor],
    xa_up: Optional[torch.Tensor],
    B_gate: Optional[torch.Tensor],
    B_up: Optional[torch.Tensor],
    s_gate: float = 1.0,
    s_up: float = 1.0,
    save_eg: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """``fused_lora_swiglu`` that, with ``save_eg``, writes e_full / g_full over ``e_base`` / ``g_base`` instead
    of into fresh tensors (the reference's ``fused_lora_swiglu_inplace``,
    kernels/lora_mlp/experiments/v6/lora_mlp_kernel_v6.py:81-160: it saves two M x N buffers of peak memory).
    Safe because a tile of e_base / g_base is staged in shared memory in full before its e / g are stored."""
    return fused_lora_swiglu(e_base, g_base, xa_gate, xa_up, B_gate, B_up, s_gate, s_up, save_eg, _inplace=True)


def fused_lora_swiglu(
    e_base: torch.Tensor,
    g_base: torch.Tensor,
    xa_gate: Optional[torch.Tensor],
    xa_up: Optional[torch.Tensor],
    B_gate: Optional[torch.Tensor],
    B_up: Optional[torch.Tensor],
    s_gate: float = 1.0,
    s_up: float = 1.0,
    save_eg: bool = False,
    _inplace: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Returns ``(h, e_full, g_full)`` with ``save_eg``, else ``(h, None, None)``; e_full/g_full are e and g
    with the adapter terms added, as the backward needs them."""
    if not e_base.is_cuda:
        raise RuntimeError("fused_lora_swiglu has a CUDA (sm_100a) kernel only; there is no CPU fallback")
    if e_base.shape != g_base.shape or e_base.dim() != 2:
        raise ValueError(f"e_base and g_base must be [M, N] matrices of one shape, got {e_base.shape} and {g_base.shape}")
    if xa_gate is None:
        # no adapters: plain SwiGLU of the base projections
        h = swiglu_forward(e_base, g_base)[0]
        return (h, e_base, g_base) if save_eg else (h, None, None)
    if any(t.dtype != e_base.dtype for t in (g_base, xa_gate, xa_up, B_gate, B_up)):
        raise TypeError("fused_lora_swiglu needs all tensors in one dtype")
    m, n = e_base.shape
    r = xa_gate.shape[1]
    if xa_gate.shape != (m, r) or xa_up.shape != (m, r) or B_gate.shape != (n, r) or B_up.shape != (n, r):
        raise ValueError("expected xa_gate, xa_up of shape [M, r] and B_gate, B_up of shape [N, r]")
    if e_base.dtype != torch.bfloat16 or r % 8 or not 8 <= r <= 64 or n % 8:
        # fp16 / fp32, or a shape the tensor-core epilogue does not take (rank not a multiple of 8 in
        # [8, 64], N not a multiple of 8): adapter terms by library GEMMs, then the streaming SwiGLU kernel
        sg, su = _as_float("s_gate", s_gate), _as_float("s_up", s_up)
        e = e_base if _inplace else e_base.clone()
        g = g_base if _inplace else g_base.clone()
        e.addmm_(xa_gate, B_gate.t(), alpha=sg)
        g.addmm_(xa_up, B_up.t(), alpha=su)
        h = swiglu_forward(e, g)[0]
        return (h, e, g) if save_eg else (h, None, None)
    sg, su = _as_float("s_gate", s_gate), _as_float("s_up", s_up)
    if _inplace and not (e_base.is_contiguous() and g_base.is_contiguous()):
        raise ValueError("the in-place variant needs contiguous e_base and g_base")
    e_base, g_base = e_base.contiguous(), g_base.contiguous()
    xa_gate, xa_up, B_gate, B_up = (t.contiguous() for t in (xa_gate, xa_up, B_gate, B_up))
    h = torch.empty_like(e_base)
    e_out = (e_base if _inplace else torch.empty_like(e_base)) if save_eg else None
    g_out = (g_base if _inplace else torch.empty_like(e_base)) if save_eg else None
    with _launching(e_base.device) as status:
        rc = _lib.lib.swiglu_b200_lora_swiglu_fwd(
            h.data_ptr(), e_out.data_ptr() if save_eg else None, g_out.data_ptr() if save_eg else None,
            e_base.data_ptr(), g_base.data_ptr(), xa_gate.data_ptr(), xa_up.data_ptr(), B_gate.data_ptr(),
            B_up.data_ptr(), m, n, r, sg, su, status.data_ptr(), e_base.device.index,
            torch.cuda.current_stream(e_base.device).cuda_stream,
        )
    _lib.check("fused_lora_swiglu", rc)
    return h, e_out, g_out


def swiglu_DWf_DW_dfg_kernel(DW: torch.Tensor, e: torch.Tensor, g: torch.Tensor):
    """The elementwise step of the reference's LoRA-MLP backward under its own name and buffer convention
    (kernels/lora_mlp/reference/unsloth_baseline.py:155-170, called at experiments/v3/lora_mlp_kernel_v3.py:324):
    overwrites ``DW`` with ``h = silu(e) * g``, ``e`` with ``DW * silu(e)`` (the gradient of g) and ``g`` with
    ``DW * g * silu'(e)`` (the gradient of e), and returns the three buffers in that order."""
    if not (DW.is_contiguous() and e.is_contiguous() and g.is_contiguous()):
        raise ValueError("DW, e and g must be contiguous: they are overwritten in place")
    if DW.shape != e.shape or e.shape != g.shape or DW.dtype != e.dtype or g.dtype != e.dtype:
        raise ValueError("DW, e and g must share one shape and dtype")
    if not e.is_cuda:
        raise RuntimeError("swiglu_DWf_DW_dfg_kernel has a CUDA (sm_100a) kernel only; there is no CPU fallback")
    from .swiglu import _DTYPE_CODE, _check_cuda_dtype, _stream

    _check_cuda_dtype(e)
    _lib.check(
        "swiglu_DWf_DW_dfg_kernel",
        _lib.lib.swiglu_b200_bwd_recompute(
            DW.data_ptr(), g.data_ptr(), e.data_ptr(), DW.data_ptr(), e.data_ptr(), g.data_ptr(),
            e.numel(), _DTYPE_CODE[e.dtype], 1.0, 1.0, e.device.index, _stream(e.device),
        ),
    )
    return DW, e, g


def _one_launch_ok(X, W_gate, A_gate) -> bool:
    """Shapes and dtypes the fused projection + adapters + SwiGLU kernel takes."""
    if A_gate is None or X.dtype != torch.bfloat16:
        return False
    n, k = W_gate.shape
    r = A_gate.shape[0]
    return r % 8 == 0 and 8 <= r <= 64 and k % 8 == 0 and n % 16 == 0


ACTIVATIONS = ("silu", "gelu_tanh", "gelu_exact")


def _approximate(activation: str) -> str:
    return "tanh" if activation == "gelu_tanh" else "none"


def _lora_mlp_forward(X, W_gate, A_gate, B_gate, s_gate, W_up, A_up, B_up, s_up, W_down, A_down, B_down, s_down,
                      save_eg, activation="silu"):
    if activation not in ACTIVATIONS:
        raise ValueError(f"activation must be one of {ACTIVATIONS}, got {activation!r}")
    x2 = X.reshape(-1, X.shape[-1])
    if _one_launch_ok(X, W_gate, A_gate):
        # gate and up projections, both adapters and the gated activation in one tcgen05 launch; e and g leave
        # the chip only when a backward pass needs them
        from .fused_mlp import lora_gate_up_swiglu_forward

        h, e, g = lora_gate_up_swiglu_forward(x2, W_gate, W_up, A_gate, B_gate, s_gate, A_up, B_up, s_up, save_eg,
                                              activation)
    else:
        e = x2 @ W_gate.t()
        g = x2 @ W_up.t()
        if A_gate is not None and activation == "silu":
            h, e, g = fused_lora_swiglu_inplace(e, g, x2 @ A_gate.t(), x2 @ A_up.t(), B_gate, B_up, s_gate, s_up,
                                                save_eg=save_eg)
        else:
            if A_gate is not None:
                e.addmm_(x2 @ A_gate.t(), B_gate.t(), alpha=s_gate)
                g.addmm_(x2 @ A_up.t(), B_up.t(), alpha=s_up)
            if activation == "silu":
                h = swiglu_forward(e, g)[0]
            else:
                from .geglu import geglu_forward

                h = geglu_forward(e, g, _approximate(activation))[0]
    out = h @ W_down.t()
    if A_down is not None:
        out.addmm_(h @ A_down.t(), B_down.t(), alpha=s_down)
    return out.view(*X.shape[:-1], out.shape[-1]), e, g


def lora_mlp(X, W_gate, A_gate, B_gate, s_gate, W_up, A_up, B_up, s_up, W_down, A_down, B_down, s_down,
             activation: str = "silu"):
    """LoRA MLP forward without autograd: ``down(act(gate(X)) * up(X))``, every projection ``X W^T + s (X A^T) B^T``
    with W ``[out, in]``, A ``[r, in]``, B ``[out, r]``.  Argument order of the reference's ``lora_mlp_v3``
    (kernels/lora_mlp/experiments/v3/lora_mlp_kernel_v3.py:244-256); adapters may be ``None``.  ``activation`` (not in
    the reference, whose block is SiLU only): ``"silu"``, ``"gelu_tanh"`` or ``"gelu_exact"``."""
    with torch.no_grad():
        return _lora_mlp_forward(X, W_gate, A_gate, B_gate, s_gate, W_up, A_up, B_up, s_up, W_down, A_down, B_down,
                                 s_down, save_eg=False, activation=activation)[0]


class LoRAMLP(torch.autograd.Function):
    """Trainable LoRA MLP: gradients for X and the six adapter matrices, base weights frozen.  Same ``apply``
    arguments and gradient tuple as the reference's ``LoRAMLPv3`` (lora_mlp_kernel_v3.py:259-357), plus an optional
    fourteenth argument ``activation`` (``"silu"``, ``"gelu_tanh"``, ``"gelu_exact"``) for Gemma-style blocks.  The forward
    keeps X and the adapter-corrected e, g (not h); the backward recomputes h and overwrites the saved e and g
    with their gradients, so a graph can be walked once."""

    @staticmethod
    def forward(ctx, X, W_gate, A_gate, B_gate, s_gate, W_up, A_up, B_up, s_up, W_down, A_down, B_down, s_down,
                activation="silu"):
        if any(t is None for t in (A_gate, B_gate, A_up, B_up, A_down, B_down)):
            raise ValueError("LoRAMLP differentiates the six adapter matrices: all of them must be given "
                             "(use lora_mlp() for a forward pass with a projection that has no adapter)")
        out, e, g = _lora_mlp_forward(X, W_gate, A_gate, B_gate, s_gate, W_up, A_up, B_up, s_up, W_down, A_down,
                                      B_down, s_down, save_eg=True, activation=activation)
        ctx.save_for_backward(X, e, g, A_gate, B_gate, A_up, B_up, A_down, B_down)
        ctx.base_weights = (W_gate, W_up, W_down)
        ctx.scales = (s_gate, s_up, s_down)
        ctx.activation = activation
        return out

    @staticmethod
    def backward(ctx, dY):
        X, e, g, A_gate, B_gate, A_up, B_up, A_down, B_down = ctx.saved_tensors
        W_gate, W_up, W_down = ctx.base_weights
        s_gate, s_up, s_down = ctx.scales
        x2 = X.reshape(-1, X.shape[-1])
        dy = dY.reshape(-1, dY.shape[-1])

        # through the down projection: dh = dY W_d + s_d (dY B_d) A_d
        dyB = dy @ B_down                                   # [M, r]
        dh = dy @ W_down
        dh.addmm_(dyB, A_down, alpha=s_down)
        if ctx.activation == "silu":
            h, de, dg = swiglu_backward_recompute(dh, e, g)  # in place: dh <- h, e <- de, g <- dg
        else:
            from .geglu import geglu_backward_recompute

            h, de, dg = geglu_backward_recompute(dh, e, g, _approximate(ctx.activation))
        dA_down = s_down * (dyB.t() @ h)                    # [r, I]
        dB_down = s_down * (dy.t() @ (h @ A_down.t()))      # [H, r]

        deB, dgB = de @ B_gate, dg @ B_up                   # [M, r]
        dA_gate = s_gate * (deB.t() @ x2)                   # [r, H]
        dB_gate = s_gate * (de.t() @ (x2 @ A_gate.t()))     # [I, r]
        dA_up = s_up * (dgB.t() @ x2)
        dB_up = s_up * (dg.t() @ (x2 @ A_up.t()))

        n, k = W_gate.shape
        if X.dtype == torch.bfloat16 and k % 16 == 0 and n % 8 == 0:
            # de W_g + dg W_u as ONE contraction of length 2n on this library's tcgen05 kernel
            from .fused_mlp import gate_up_swiglu_backward_gemms

            dX = gate_up_swiglu_backward_gemms(de, dg, x2, W_gate, W_up, need_dx=True, need_dw=False)[0]
        else:
            dX = de @ W_gate
            dX.addmm_(dg, W_up)
        dX.addmm_(deB, A_gate, alpha=s_gate)
        dX.addmm_(dgB, A_up, alpha=s_up)
        return (dX.view_as(X), None, dA_gate, dB_gate, None, None, dA_up, dB_up, None, None, dA_down, dB_down, None,
                None)

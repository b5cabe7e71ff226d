"""LoRA + SwiGLU epilogue: ``h = silu(e_base + s_gate * xa_gate @ B_gate.T) * (g_base + s_up * xa_up @ B_up.T)``.

Mirrors ``fused_lora_swiglu`` of the reference (kernels/lora_mlp/experiments/v3/lora_mlp_kernel_v3.py:141-200;
same argument order, same return triple), the one kernel of its LoRA-MLP forward that is not a library GEMM:
the base projections and the skinny ``x @ A.T`` products stay with cuBLAS, and this step adds the rank-r
adapter terms and applies SwiGLU in one pass over e and g.  Here it is a TMA-fed tcgen05 kernel
(``swiglu_b200_lora_swiglu_fwd``).  bf16 only; the rank must be a multiple of 8, at most 64.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .fused_mlp import _status
from .swiglu import _as_float, swiglu_forward


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
    if e_base.dtype != torch.bfloat16 or any(t.dtype != torch.bfloat16 for t in (g_base, xa_gate, xa_up, B_gate, B_up)):
        raise TypeError("fused_lora_swiglu supports bf16 tensors only")
    m, n = e_base.shape
    r = xa_gate.shape[1]
    if xa_gate.shape != (m, r) or xa_up.shape != (m, r) or B_gate.shape != (n, r) or B_up.shape != (n, r):
        raise ValueError("expected xa_gate, xa_up of shape [M, r] and B_gate, B_up of shape [N, r]")
    if r % 8 or not 8 <= r <= 64 or n % 8:
        raise ValueError("the kernel needs a rank that is a multiple of 8 in [8, 64] and N % 8 == 0")
    sg, su = _as_float("s_gate", s_gate), _as_float("s_up", s_up)
    if _inplace and not (e_base.is_contiguous() and g_base.is_contiguous()):
        raise ValueError("the in-place variant needs contiguous e_base and g_base")
    e_base, g_base = e_base.contiguous(), g_base.contiguous()
    xa_gate, xa_up, B_gate, B_up = (t.contiguous() for t in (xa_gate, xa_up, B_gate, B_up))
    h = torch.empty_like(e_base)
    e_out = (e_base if _inplace else torch.empty_like(e_base)) if save_eg else None
    g_out = (g_base if _inplace else torch.empty_like(e_base)) if save_eg else None
    _lib.check(
        "fused_lora_swiglu",
        _lib.lib.swiglu_b200_lora_swiglu_fwd(
            h.data_ptr(), e_out.data_ptr() if save_eg else None, g_out.data_ptr() if save_eg else None,
            e_base.data_ptr(), g_base.data_ptr(), xa_gate.data_ptr(), xa_up.data_ptr(), B_gate.data_ptr(),
            B_up.data_ptr(), m, n, r, sg, su, _status(e_base.device).data_ptr(), e_base.device.index,
            torch.cuda.current_stream(e_base.device).cuda_stream,
        ),
    )
    return h, e_out, g_out

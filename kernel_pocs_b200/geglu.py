"""Host side of the GeGLU operator, the sibling of SwiGLU: ``h = gelu(gate) * up``.

Mirrors the activation part of kernels/geglu/geglu.py of Forge-researchlab/kernel-POCs name for name
(``geglu``, ``geglu_packed``, ``ForgeGEGLUFunction``, ``ForgePackedGEGLUFunction``, ``geglu_forward`` /
``geglu_backward``, ``geglu_packed_forward`` / ``geglu_packed_backward``, ``torch_geglu_reference``,
``torch_geglu_packed_reference``; reference :255-272 and :380-575), bound to the same streaming CUDA
kernels as SwiGLU with a GELU functor (``swiglu_b200_geglu_fwd`` / ``_bwd``).  ``approximate`` is ``"tanh"``
or ``"none"`` as in the reference; the in-place backward, the saved tensors (flat gate and up) and the
exception messages are kept.  As for SwiGLU there is no CPU path.

The MLP-level helpers of the reference file (``geglu_mlp``, ``pack_geglu_gate_up_weight`` / ``_bias``,
``torch_geglu_mlp_reference``; reference :275-377) are here too.  Where the reference's ``geglu_mlp`` runs one
or two library GEMMs and then its GeGLU kernel, this one runs the gate/up stage as ONE tcgen05 launch
(``swiglu_b200_geglu_gemm_fwd``: both projections with the GELU in the epilogue) whenever the operands are
bias-free bf16 of a shape that kernel takes; a packed ``[2I, H]`` weight is used in place, as its two halves.
Other cases take library GEMMs and the streaming GeGLU kernels.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib
from .swiglu import _DTYPE_CODE, _check_packed_input, _check_same_shape_inputs, _require_cuda, _stream


def _check_cuda_dtype(x: torch.Tensor) -> None:
    if x.dtype not in _DTYPE_CODE:
        raise TypeError(f"CUDA GEGLU supports fp16, bf16, and fp32, got {x.dtype}")


def _check_approximate(approximate: str) -> bool:
    if approximate not in {"tanh", "none"}:
        raise ValueError(f"approximate must be 'tanh' or 'none', got {approximate!r}")
    return approximate == "tanh"


def torch_geglu_reference(gate: torch.Tensor, up: torch.Tensor, approximate: str = "tanh") -> torch.Tensor:
    _check_same_shape_inputs(gate, up)
    _check_approximate(approximate)
    return torch.nn.functional.gelu(gate.to(torch.float32), approximate=approximate).to(gate.dtype) * up


def torch_geglu_packed_reference(gate_up: torch.Tensor, approximate: str = "tanh") -> torch.Tensor:
    _check_packed_input(gate_up)
    half = gate_up.shape[-1] // 2
    return torch_geglu_reference(gate_up[..., :half], gate_up[..., half:], approximate)


def geglu_forward(gate: torch.Tensor, up: torch.Tensor, approximate: str = "tanh"):
    """Returns ``(h, gate_flat, up_flat)``."""
    _check_same_shape_inputs(gate, up)
    _check_cuda_dtype(gate)
    tanh = _check_approximate(approximate)
    _require_cuda(gate, "gate")
    gate_flat = gate.contiguous().view(-1)
    up_flat = up.contiguous().view(-1)
    out = torch.empty_like(gate_flat)
    n = gate_flat.numel()
    _lib.check(
        "geglu_forward",
        _lib.lib.swiglu_b200_geglu_fwd(out.data_ptr(), gate_flat.data_ptr(), up_flat.data_ptr(), 1, n, n, n,
                                       _DTYPE_CODE[gate.dtype], int(tanh), gate.device.index, _stream(gate.device)),
    )
    return out.view(gate.shape), gate_flat, up_flat


def geglu_backward(dout: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, approximate: str = "tanh",
                   preserve_inputs: bool = False):
    """Returns ``(dgate, dup)`` shaped like ``dout``; written over gate/up unless ``preserve_inputs``."""
    _check_same_shape_inputs(gate, up)
    _check_cuda_dtype(gate)
    tanh = _check_approximate(approximate)
    _require_cuda(gate, "gate")
    if dout.dtype != gate.dtype or dout.device != gate.device:
        raise TypeError("dout must have the dtype and device of gate and up")
    if dout.numel() != gate.numel():
        raise ValueError(f"dout of shape {tuple(dout.shape)} does not match gate of shape {tuple(gate.shape)}")
    dout_flat = dout.contiguous().view(-1)
    if preserve_inputs:
        gate, up = gate.contiguous(), up.contiguous()
        dgate, dup = torch.empty_like(gate), torch.empty_like(up)
    else:
        if not (gate.is_contiguous() and up.is_contiguous()):
            raise ValueError("the in-place backward needs contiguous gate and up; pass preserve_inputs=True")
        dgate, dup = gate, up
    n = dout_flat.numel()
    _lib.check(
        "geglu_backward",
        _lib.lib.swiglu_b200_geglu_bwd(dgate.data_ptr(), dup.data_ptr(), dout_flat.data_ptr(), gate.data_ptr(),
                                       up.data_ptr(), 1, n, n, n, n, _DTYPE_CODE[gate.dtype], int(tanh),
                                       gate.device.index, _stream(gate.device)),
    )
    return dgate.view(dout.shape), dup.view(dout.shape)


def geglu_backward_recompute(dout: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, approximate: str = "tanh",
                             preserve_inputs: bool = False):
    """``(h, dgate, dup)`` from one pass over ``(dout, gate, up)``: ``geglu_backward`` together with the forward
    output, for training steps that kept ``gate`` and ``up`` but not ``h``.  Unless ``preserve_inputs`` is set, ``h``
    is written over ``dout``, ``dgate`` over ``gate`` and ``dup`` over ``up``.  No counterpart in the reference."""
    _check_same_shape_inputs(gate, up)
    _check_cuda_dtype(gate)
    tanh = _check_approximate(approximate)
    _require_cuda(gate, "gate")
    if dout.dtype != gate.dtype or dout.device != gate.device or dout.shape != gate.shape:
        raise ValueError("dout must have the shape, dtype and device of gate and up")
    if preserve_inputs:
        dout, gate, up = dout.contiguous(), gate.contiguous(), up.contiguous()
        h, dgate, dup = torch.empty_like(dout), torch.empty_like(gate), torch.empty_like(up)
    else:
        if not (dout.is_contiguous() and gate.is_contiguous() and up.is_contiguous()):
            raise ValueError("the in-place form needs contiguous dout, gate and up; pass preserve_inputs=True")
        h, dgate, dup = dout, gate, up
    _lib.check(
        "geglu_backward_recompute",
        _lib.lib.swiglu_b200_geglu_bwd_recompute(
            h.data_ptr(), dgate.data_ptr(), dup.data_ptr(), dout.data_ptr(), gate.data_ptr(), up.data_ptr(),
            gate.numel(), _DTYPE_CODE[gate.dtype], int(tanh), gate.device.index, _stream(gate.device)),
    )
    return h, dgate, dup


def geglu_packed_forward(gate_up: torch.Tensor, approximate: str = "tanh"):
    _check_packed_input(gate_up)
    _check_cuda_dtype(gate_up)
    tanh = _check_approximate(approximate)
    _require_cuda(gate_up, "gate_up")
    shape = gate_up.shape
    total = shape[-1]
    n_cols = total // 2
    rows = gate_up.numel() // total if total else 0
    gate_up_2d = gate_up.contiguous().view(rows, total)
    out = torch.empty((rows, n_cols), device=gate_up.device, dtype=gate_up.dtype)
    base = gate_up_2d.data_ptr()
    _lib.check(
        "geglu_packed_forward",
        _lib.lib.swiglu_b200_geglu_fwd(out.data_ptr(), base, base + n_cols * gate_up.element_size(), rows, n_cols,
                                       total, n_cols, _DTYPE_CODE[gate_up.dtype], int(tanh), gate_up.device.index,
                                       _stream(gate_up.device)),
    )
    return out.view(*shape[:-1], n_cols), gate_up_2d


def geglu_packed_backward(dout: torch.Tensor, gate_up: torch.Tensor, input_shape: torch.Size,
                          approximate: str = "tanh", preserve_inputs: bool = False):
    _check_packed_input(gate_up)
    _check_cuda_dtype(gate_up)
    tanh = _check_approximate(approximate)
    _require_cuda(gate_up, "gate_up")
    if dout.dtype != gate_up.dtype or dout.device != gate_up.device:
        raise TypeError("dout must have the dtype and device of gate_up")
    n_cols = dout.shape[-1]
    total = input_shape[-1]
    if total != 2 * n_cols or gate_up.numel() != 2 * dout.numel():
        raise ValueError(f"dout of shape {tuple(dout.shape)} does not match packed input {tuple(input_shape)}")
    rows = dout.numel() // n_cols if n_cols else 0
    dout_2d = dout.contiguous().view(rows, n_cols)
    if preserve_inputs:
        gate_up = gate_up.contiguous()
        dgate_up = torch.empty_like(gate_up)
    else:
        if not gate_up.is_contiguous():
            raise ValueError("the in-place backward needs a contiguous gate_up; pass preserve_inputs=True")
        dgate_up = gate_up
    half = n_cols * gate_up.element_size()
    _lib.check(
        "geglu_packed_backward",
        _lib.lib.swiglu_b200_geglu_bwd(dgate_up.data_ptr(), dgate_up.data_ptr() + half, dout_2d.data_ptr(),
                                       gate_up.data_ptr(), gate_up.data_ptr() + half, rows, n_cols, total, total,
                                       n_cols, _DTYPE_CODE[gate_up.dtype], int(tanh), gate_up.device.index,
                                       _stream(gate_up.device)),
    )
    return dgate_up.view(input_shape)


class ForgeGEGLUFunction(torch.autograd.Function):
    """``apply(gate, up, approximate="tanh", preserve_inputs=False)``; saves the flat gate and up."""

    @staticmethod
    def forward(ctx, gate, up, approximate="tanh", preserve_inputs=False):
        h, gate_flat, up_flat = geglu_forward(gate, up, approximate)
        ctx.save_for_backward(gate_flat, up_flat)
        ctx.approximate = approximate
        ctx.preserve_inputs = bool(preserve_inputs)
        return h

    @staticmethod
    def backward(ctx, dout):
        gate_flat, up_flat = ctx.saved_tensors
        dgate, dup = geglu_backward(dout.reshape(-1), gate_flat, up_flat, ctx.approximate, ctx.preserve_inputs)
        return dgate.view(dout.shape), dup.view(dout.shape), None, None


class ForgePackedGEGLUFunction(torch.autograd.Function):
    """``apply(gate_up, approximate="tanh", preserve_inputs=False)``."""

    @staticmethod
    def forward(ctx, gate_up, approximate="tanh", preserve_inputs=False):
        h, gate_up_2d = geglu_packed_forward(gate_up, approximate)
        ctx.save_for_backward(gate_up_2d)
        ctx.input_shape = gate_up.shape
        ctx.approximate = approximate
        ctx.preserve_inputs = bool(preserve_inputs)
        return h

    @staticmethod
    def backward(ctx, dout):
        (gate_up_2d,) = ctx.saved_tensors
        dgate_up = geglu_packed_backward(dout, gate_up_2d, ctx.input_shape, ctx.approximate, ctx.preserve_inputs)
        return dgate_up, None, None


def geglu(gate: torch.Tensor, up: torch.Tensor, approximate: str = "tanh", preserve_inputs: bool = False):
    _check_same_shape_inputs(gate, up)
    _check_approximate(approximate)
    _require_cuda(gate, "gate")
    return ForgeGEGLUFunction.apply(gate, up, approximate, preserve_inputs)


def geglu_packed(gate_up: torch.Tensor, approximate: str = "tanh", preserve_inputs: bool = False):
    _check_packed_input(gate_up)
    _check_approximate(approximate)
    _require_cuda(gate_up, "gate_up")
    return ForgePackedGEGLUFunction.apply(gate_up, approximate, preserve_inputs)


# ------------------------------------------------------------------------------------------ MLP level

def pack_geglu_gate_up_weight(gate_weight: torch.Tensor, up_weight: torch.Tensor) -> torch.Tensor:
    """``[2I, H]`` weight with the gate rows first (reference kernels/geglu/geglu.py:275-286)."""
    if gate_weight.shape != up_weight.shape:
        raise ValueError(
            f"gate_weight and up_weight must have the same shape, got {gate_weight.shape} and {up_weight.shape}")
    if gate_weight.device != up_weight.device:
        raise ValueError("gate_weight and up_weight must be on the same device")
    if gate_weight.dtype != up_weight.dtype:
        raise TypeError(f"gate_weight and up_weight must have the same dtype, got {gate_weight.dtype} and {up_weight.dtype}")
    if gate_weight.dim() != 2:
        raise ValueError(f"gate_weight and up_weight must be 2D, got {gate_weight.dim()}D")
    return torch.cat([gate_weight, up_weight], dim=0).contiguous()


def pack_geglu_gate_up_bias(gate_bias, up_bias):
    """Packed bias matching ``pack_geglu_gate_up_weight``, or ``None`` when there is none (reference :289-308)."""
    if gate_bias is None and up_bias is None:
        return None
    if gate_bias is None or up_bias is None:
        raise ValueError("gate_bias and up_bias must either both be None or both be tensors for packed gate+up")
    if gate_bias.dim() != 1 or up_bias.dim() != 1:
        raise ValueError("gate_bias and up_bias must be 1D tensors")
    if gate_bias.shape != up_bias.shape:
        raise ValueError(f"gate_bias and up_bias must have the same shape, got {gate_bias.shape} and {up_bias.shape}")
    if gate_bias.device != up_bias.device:
        raise ValueError("gate_bias and up_bias must be on the same device")
    if gate_bias.dtype != up_bias.dtype:
        raise TypeError(f"gate_bias and up_bias must have the same dtype, got {gate_bias.dtype} and {up_bias.dtype}")
    return torch.cat([gate_bias, up_bias], dim=0).contiguous()


def torch_geglu_mlp_reference(x, gate_weight, up_weight, down_weight, gate_bias=None, up_bias=None, down_bias=None,
                              approximate: str = "tanh") -> torch.Tensor:
    """``down(gelu(gate(x)) * up(x))`` with PyTorch operators (reference :311-327)."""
    _check_approximate(approximate)
    hidden = torch_geglu_reference(F.linear(x, gate_weight, gate_bias), F.linear(x, up_weight, up_bias), approximate)
    return F.linear(hidden, down_weight, down_bias)


def gate_up_geglu_forward(x, w_gate, w_up, approximate: str = "tanh", save_preactivations: bool = False):
    """``gelu(x @ w_gate.T) * (x @ w_up.T)`` in one launch; with ``save_preactivations`` also the two projections
    (rounded to bf16).  bf16 operands, ``k % 8 == 0``, ``n % 16 == 0``."""
    from .fused_mlp import _check_operands, _launching

    tanh = _check_approximate(approximate)
    _check_operands(x, w_gate, w_up)
    n, k = w_gate.shape
    x2 = x.contiguous().view(-1, k)
    if not (w_gate.is_contiguous() and w_up.is_contiguous()):
        w_gate, w_up = w_gate.contiguous(), w_up.contiguous()
    m = x2.shape[0]
    h = torch.empty((m, n), dtype=x.dtype, device=x.device)
    gate = torch.empty_like(h) if save_preactivations else None
    up = torch.empty_like(h) if save_preactivations else None
    with _launching(x.device) as status:
        rc = _lib.lib.swiglu_b200_geglu_gemm_fwd(
            h.data_ptr(), gate.data_ptr() if save_preactivations else None,
            up.data_ptr() if save_preactivations else None, x2.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(),
            m, n, k, int(tanh), status.data_ptr(), x.device.index, _stream(x.device),
        )
    _lib.check("gate_up_geglu_forward", rc)
    h = h.view(*x.shape[:-1], n)
    return (h, gate, up) if save_preactivations else h


class FusedGateUpGEGLUFunction(torch.autograd.Function):
    """``apply(x, w_gate, w_up, approximate)``: the fused projection + GeGLU with a backward made of this
    library's GeGLU backward kernel on the saved projections and its tcgen05 backward GEMMs."""

    @staticmethod
    def forward(ctx, x, w_gate, w_up, approximate):
        h, gate, up = gate_up_geglu_forward(x, w_gate, w_up, approximate, True)
        ctx.save_for_backward(x, w_gate, w_up, gate, up)
        ctx.approximate = approximate
        return h

    @staticmethod
    def backward(ctx, dh):
        from .fused_mlp import _own_backward_gemms, gate_up_swiglu_backward_gemms

        x, w_gate, w_up, gate, up = ctx.saved_tensors
        n, k = w_gate.shape
        # gate/up are private to this node, so the in-place backward is safe
        dgate, dup = geglu_backward(dh.reshape(-1, n), gate, up, ctx.approximate, False)
        if _own_backward_gemms(n, k):
            need_dw = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
            dx, dw_gate, dw_up = gate_up_swiglu_backward_gemms(dgate, dup, x, w_gate, w_up, ctx.needs_input_grad[0],
                                                               need_dw)
            return dx, dw_gate, dw_up, None
        x2 = x.reshape(-1, k)
        dx = torch.addmm(dgate @ w_gate, dup, w_up).view(x.shape) if ctx.needs_input_grad[0] else None
        dw_gate = dgate.t() @ x2 if ctx.needs_input_grad[1] else None
        dw_up = dup.t() @ x2 if ctx.needs_input_grad[2] else None
        return dx, dw_gate, dw_up, None


def _linear_operand(name, t, expect, x):
    """A weight ``[out, in]`` (``expect`` = in) or bias ``[out]`` (``expect`` = out) that fits ``x``."""
    want_dim = 2 if name.endswith("weight") else 1
    if t.dim() != want_dim or t.shape[-1] != expect:
        kind = f"[out_features, {expect}]" if want_dim == 2 else f"[{expect}]"
        raise ValueError(f"{name} must have shape {kind}, got {tuple(t.shape)}")
    if not t.is_floating_point():
        raise TypeError(f"{name} must be a floating point tensor")
    if t.device != x.device:
        raise ValueError(f"{name} must be on device {x.device}, got {t.device}")
    if t.dtype != x.dtype:
        raise TypeError(f"{name} must have dtype {x.dtype}, got {t.dtype}")


def _takes_one_launch(x, w_gate, biased: bool) -> bool:
    n, k = w_gate.shape
    return x.is_cuda and x.dtype == torch.bfloat16 and not biased and k % 8 == 0 and n % 16 == 0


def geglu_mlp(x, down_weight, gate_weight=None, up_weight=None, packed_gate_up_weight=None, gate_bias=None,
              up_bias=None, packed_gate_up_bias=None, down_bias=None, approximate: str = "tanh",
              preserve_inputs: bool = False) -> torch.Tensor:
    """``down(gelu(gate(x)) * up(x))`` from separate gate/up weights or from one packed ``[2I, H]`` weight:
    the signature and argument rules of the reference's ``geglu_mlp`` (kernels/geglu/geglu.py:330-377).  The gate/up
    stage is one tcgen05 launch for bias-free bf16 operands (``k % 8 == 0``, ``I % 16 == 0``); otherwise library GEMMs
    feed the streaming GeGLU kernels."""
    _check_approximate(approximate)
    if x.dim() < 2:
        raise ValueError(f"x must have at least 2 dimensions, got shape {tuple(x.shape)}")
    if not x.is_floating_point():
        raise TypeError("x must be a floating point tensor")
    hidden_in = x.shape[-1]
    packed = packed_gate_up_weight is not None
    if packed and (gate_weight is not None or up_weight is not None):
        raise ValueError("provide either packed_gate_up_weight or separate gate_weight/up_weight, not both")

    if packed:
        _linear_operand("packed_gate_up_weight", packed_gate_up_weight, hidden_in, x)
        rows = packed_gate_up_weight.shape[0]
        if rows % 2:
            raise ValueError(f"packed_gate_up_weight output dimension must be even, got {rows}")
        if gate_bias is not None or up_bias is not None:
            raise ValueError("use packed_gate_up_bias with packed_gate_up_weight")
        if packed_gate_up_bias is not None:
            _linear_operand("packed_gate_up_bias", packed_gate_up_bias, rows, x)
        inter = rows // 2
        w_gate, w_up = packed_gate_up_weight[:inter], packed_gate_up_weight[inter:]  # views: the halves in place
        biased = packed_gate_up_bias is not None
    else:
        if gate_weight is None or up_weight is None:
            raise ValueError("separate path requires gate_weight and up_weight")
        if packed_gate_up_bias is not None:
            raise ValueError("packed_gate_up_bias requires packed_gate_up_weight")
        _linear_operand("gate_weight", gate_weight, hidden_in, x)
        _linear_operand("up_weight", up_weight, hidden_in, x)
        if gate_weight.shape != up_weight.shape:
            raise ValueError(
                f"gate_weight and up_weight must have the same shape, got {gate_weight.shape} and {up_weight.shape}")
        inter = gate_weight.shape[0]
        for name, b in (("gate_bias", gate_bias), ("up_bias", up_bias)):
            if b is not None:
                _linear_operand(name, b, inter, x)
        w_gate, w_up = gate_weight, up_weight
        biased = gate_bias is not None or up_bias is not None

    if _takes_one_launch(x, w_gate, biased):
        hidden = FusedGateUpGEGLUFunction.apply(x, w_gate, w_up, approximate)
    elif packed:
        hidden = geglu_packed(F.linear(x, packed_gate_up_weight, packed_gate_up_bias), approximate=approximate,
                              preserve_inputs=preserve_inputs)
    else:
        hidden = geglu(F.linear(x, w_gate, gate_bias), F.linear(x, w_up, up_bias), approximate=approximate,
                       preserve_inputs=preserve_inputs)

    _linear_operand("down_weight", down_weight, inter, x)
    if down_bias is not None:
        _linear_operand("down_bias", down_bias, down_weight.shape[0], x)
    return F.linear(hidden, down_weight, down_bias)

"""Host side of the GeGLU operator, the sibling of SwiGLU: ``h = gelu(gate) * up``.

Mirrors the activation part of kernels/geglu/geglu.py of Forge-researchlab/kernel-POCs name for name
(``geglu``, ``geglu_packed``, ``ForgeGEGLUFunction``, ``ForgePackedGEGLUFunction``, ``geglu_forward`` /
``geglu_backward``, ``geglu_packed_forward`` / ``geglu_packed_backward``, ``torch_geglu_reference``,
``torch_geglu_packed_reference``; reference :255-272 and :380-575), bound to the same streaming CUDA
kernels as SwiGLU with a GELU functor (``swiglu_b200_geglu_fwd`` / ``_bwd``).  ``approximate`` is ``"tanh"``
or ``"none"`` as in the reference; the in-place backward, the saved tensors (flat gate and up) and the
exception messages are kept.  As for SwiGLU there is no CPU path.  The MLP-level helpers of the reference
file (``geglu_mlp``, weight packing) are matmul glue and are not part of this package.
"""
from __future__ import annotations

import torch

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

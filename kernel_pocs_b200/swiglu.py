"""Host side of the SwiGLU operator: the reference's public interface, bound to the CUDA library.

Mirrors kernels/swiglu/swiglu.py of Forge-researchlab/kernel-POCs name for name:

    swiglu, swiglu_packed                       (reference :388-410)
    ForgeSwiGLUFunction, ForgePackedSwiGLUFunction   (:326-385)
    swiglu_forward / swiglu_backward            (:201-262)
    swiglu_packed_forward / swiglu_packed_backward   (:265-323)
    torch_swiglu_reference / torch_swiglu_packed_reference   (:179-198)

What is kept: argument names, defaults, exception types and messages (:11-57), the
``ctx.save_for_backward(gate_2d, up_2d)`` contract, the in-place backward that overwrites the
saved gate/up storage unless ``preserve_inputs`` is set, and the shapes of everything returned.

What changes: the four Triton launches become two calls into libswiglu_b200.so
(``swiglu_b200_fwd`` / ``swiglu_b200_bwd``); multipliers are run-time floats rather than
compile-time constants, so a new value costs no recompilation; rows may be wider than 65536
elements (the reference's per-row block limit, :8, :19-25, does not exist in a flat stream);
bf16/fp16 results are rounded once from the fp32 value instead of two or three times.

There is no path for tensors that are not on a CUDA device: ``swiglu`` and ``swiglu_packed``
raise for them (the reference routes them to its PyTorch composite, :396-397, :408-409).
"""
from __future__ import annotations

import numbers

import torch

from . import _lib

_DTYPE_CODE = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


# ------------------------------------------------------------------------------------------
# Argument checks (same exception types and wording as the reference, swiglu.py:11-57)
# ------------------------------------------------------------------------------------------

def _as_float(name: str, value) -> float:
    if isinstance(value, torch.Tensor):
        raise TypeError(f"{name} must be a Python scalar, not a tensor")
    if not isinstance(value, numbers.Real):
        raise TypeError(f"{name} must be a real Python scalar")
    return float(value)


def _check_same_shape_inputs(gate: torch.Tensor, up: torch.Tensor) -> None:
    if gate.shape != up.shape:
        raise ValueError(f"gate and up must have the same shape, got {gate.shape} and {up.shape}")
    if gate.device != up.device:
        raise ValueError("gate and up must be on the same device")
    if gate.dtype != up.dtype:
        raise TypeError(f"gate and up must have the same dtype, got {gate.dtype} and {up.dtype}")
    if not (gate.is_floating_point() and up.is_floating_point()):
        raise TypeError("gate and up must be floating point tensors")


def _check_cuda_dtype(x: torch.Tensor) -> None:
    if x.dtype not in _DTYPE_CODE:
        raise TypeError(f"CUDA SwiGLU supports fp16, bf16, and fp32, got {x.dtype}")


def _check_packed_input(gate_up: torch.Tensor) -> None:
    if gate_up.shape[-1] % 2 != 0:
        raise ValueError(f"packed gate_up last dimension must be even, got {gate_up.shape[-1]}")
    if not gate_up.is_floating_point():
        raise TypeError("gate_up must be a floating point tensor")


def _require_cuda(x: torch.Tensor, what: str) -> None:
    if not x.is_cuda:
        raise RuntimeError(
            f"{what} is on {x.device}: this SwiGLU implementation has CUDA (sm_100a) kernels only "
            "and no CPU fallback; use torch_swiglu_reference for a host computation"
        )


# ------------------------------------------------------------------------------------------
# PyTorch composite, part of the public surface (tests compare against it on any device)
# ------------------------------------------------------------------------------------------

def torch_swiglu_reference(
    gate: torch.Tensor,
    up: torch.Tensor,
    gate_multiplier: float = 1.0,
    down_multiplier: float = 1.0,
) -> torch.Tensor:
    """``silu(gate * gm)`` in fp32, cast to the input dtype, times ``up``, times ``dm``."""
    gm = _as_float("gate_multiplier", gate_multiplier)
    dm = _as_float("down_multiplier", down_multiplier)
    activated = torch.nn.functional.silu(gate.to(torch.float32) * gm).to(gate.dtype)
    return activated * up * dm


def torch_swiglu_packed_reference(
    gate_up: torch.Tensor,
    gate_multiplier: float = 1.0,
    down_multiplier: float = 1.0,
) -> torch.Tensor:
    _check_packed_input(gate_up)
    half = gate_up.shape[-1] // 2
    return torch_swiglu_reference(gate_up[..., :half], gate_up[..., half:], gate_multiplier, down_multiplier)


# ------------------------------------------------------------------------------------------
# Launch wrappers
# ------------------------------------------------------------------------------------------

def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _rows_2d(x: torch.Tensor, n_cols: int) -> torch.Tensor:
    # A view when x is already contiguous, so the backward can overwrite the caller's storage.
    rows = x.numel() // n_cols if n_cols else 0
    return x.contiguous().view(rows, n_cols)


def swiglu_forward(
    gate: torch.Tensor,
    up: torch.Tensor,
    gate_multiplier: float = 1.0,
    down_multiplier: float = 1.0,
):
    """Returns ``(h, gate_2d, up_2d)``; h has the shape of ``gate``."""
    _check_same_shape_inputs(gate, up)
    _check_cuda_dtype(gate)
    _require_cuda(gate, "gate")
    gm = _as_float("gate_multiplier", gate_multiplier)
    dm = _as_float("down_multiplier", down_multiplier)

    shape = gate.shape
    n_cols = shape[-1]
    gate_2d = _rows_2d(gate, n_cols)
    up_2d = _rows_2d(up, n_cols)
    out = torch.empty_like(gate_2d)
    rows = gate_2d.shape[0]
    _lib.check(
        "swiglu_forward",
        _lib.lib.swiglu_b200_fwd(
            out.data_ptr(), gate_2d.data_ptr(), up_2d.data_ptr(), rows, n_cols, n_cols, n_cols,
            _DTYPE_CODE[gate.dtype], gm, dm, gate.device.index, _stream(gate.device),
        ),
    )
    return out.view(shape), gate_2d, up_2d


def swiglu_backward(
    dout: torch.Tensor,
    gate: torch.Tensor,
    up: torch.Tensor,
    gate_multiplier: float = 1.0,
    down_multiplier: float = 1.0,
    preserve_inputs: bool = False,
):
    """Returns ``(dgate, dup)`` shaped like ``dout``.  Unless ``preserve_inputs`` is set they
    are written over ``gate`` and ``up``."""
    _check_same_shape_inputs(gate, up)
    _check_cuda_dtype(gate)
    _require_cuda(gate, "gate")
    gm = _as_float("gate_multiplier", gate_multiplier)
    dm = _as_float("down_multiplier", down_multiplier)
    if dout.dtype != gate.dtype or dout.device != gate.device:
        raise TypeError("dout must have the dtype and device of gate and up")

    shape = dout.shape
    n_cols = shape[-1]
    if dout.numel() != gate.numel() or (gate.dim() > 0 and gate.shape[-1] != n_cols):
        raise ValueError(f"dout of shape {tuple(shape)} does not match gate of shape {tuple(gate.shape)}")
    dout_2d = _rows_2d(dout, n_cols)
    if preserve_inputs:
        gate = gate.contiguous()
        up = up.contiguous()
        dgate = torch.empty_like(gate)
        dup = torch.empty_like(up)
    else:
        if not (gate.is_contiguous() and up.is_contiguous()):
            raise ValueError("the in-place backward needs contiguous gate and up; pass preserve_inputs=True")
        dgate, dup = gate, up
    rows = dout_2d.shape[0]
    _lib.check(
        "swiglu_backward",
        _lib.lib.swiglu_b200_bwd(
            dgate.data_ptr(), dup.data_ptr(), dout_2d.data_ptr(), gate.data_ptr(), up.data_ptr(),
            rows, n_cols, n_cols, n_cols, n_cols, _DTYPE_CODE[gate.dtype], gm, dm,
            gate.device.index, _stream(gate.device),
        ),
    )
    return dgate.view(shape), dup.view(shape)


def swiglu_backward_recompute(
    dout: torch.Tensor,
    gate: torch.Tensor,
    up: torch.Tensor,
    gate_multiplier: float = 1.0,
    down_multiplier: float = 1.0,
    preserve_inputs: bool = False,
):
    """Returns ``(h, dgate, dup)`` from one pass over ``(dout, gate, up)``: the backward of ``swiglu`` together with
    its forward output, for training steps that kept ``gate`` and ``up`` but not ``h`` (the reference's LoRA-MLP
    backward, kernels/lora_mlp/experiments/v3/lora_mlp_kernel_v3.py:324).  Unless ``preserve_inputs`` is set, ``h`` is
    written over ``dout``, ``dgate`` over ``gate`` and ``dup`` over ``up``.  No counterpart among the reference's
    ``kernels.swiglu`` names."""
    _check_same_shape_inputs(gate, up)
    _check_cuda_dtype(gate)
    _require_cuda(gate, "gate")
    gm = _as_float("gate_multiplier", gate_multiplier)
    dm = _as_float("down_multiplier", down_multiplier)
    if dout.dtype != gate.dtype or dout.device != gate.device:
        raise TypeError("dout must have the dtype and device of gate and up")
    if dout.shape != gate.shape:
        raise ValueError(f"dout of shape {tuple(dout.shape)} does not match gate of shape {tuple(gate.shape)}")
    if preserve_inputs:
        dout, gate, up = dout.contiguous(), gate.contiguous(), up.contiguous()
        h, dgate, dup = torch.empty_like(dout), torch.empty_like(gate), torch.empty_like(up)
    else:
        if not (dout.is_contiguous() and gate.is_contiguous() and up.is_contiguous()):
            raise ValueError("the in-place form needs contiguous dout, gate and up; pass preserve_inputs=True")
        h, dgate, dup = dout, gate, up
    _lib.check(
        "swiglu_backward_recompute",
        _lib.lib.swiglu_b200_bwd_recompute(
            h.data_ptr(), dgate.data_ptr(), dup.data_ptr(), dout.data_ptr(), gate.data_ptr(), up.data_ptr(),
            gate.numel(), _DTYPE_CODE[gate.dtype], gm, dm, gate.device.index, _stream(gate.device),
        ),
    )
    return h, dgate, dup


def swiglu_packed_forward(
    gate_up: torch.Tensor,
    gate_multiplier: float = 1.0,
    down_multiplier: float = 1.0,
):
    """``gate_up[..., :I]`` is gate and ``gate_up[..., I:]`` is up.  Returns ``(h, gate_up_2d)``."""
    _check_packed_input(gate_up)
    _check_cuda_dtype(gate_up)
    _require_cuda(gate_up, "gate_up")
    gm = _as_float("gate_multiplier", gate_multiplier)
    dm = _as_float("down_multiplier", down_multiplier)

    shape = gate_up.shape
    total_cols = shape[-1]
    n_cols = total_cols // 2
    gate_up_2d = _rows_2d(gate_up, total_cols)
    rows = gate_up_2d.shape[0]
    out = torch.empty((rows, n_cols), device=gate_up.device, dtype=gate_up.dtype)
    base = gate_up_2d.data_ptr()
    _lib.check(
        "swiglu_packed_forward",
        _lib.lib.swiglu_b200_fwd(
            out.data_ptr(), base, base + n_cols * gate_up.element_size(), rows, n_cols, total_cols, n_cols,
            _DTYPE_CODE[gate_up.dtype], gm, dm, gate_up.device.index, _stream(gate_up.device),
        ),
    )
    return out.view(*shape[:-1], n_cols), gate_up_2d


def swiglu_packed_backward(
    dout: torch.Tensor,
    gate_up: torch.Tensor,
    input_shape: torch.Size,
    gate_multiplier: float = 1.0,
    down_multiplier: float = 1.0,
    preserve_inputs: bool = False,
):
    """Returns ``dgate|dup`` in the packed layout, shaped ``input_shape``."""
    _check_packed_input(gate_up)
    _check_cuda_dtype(gate_up)
    _require_cuda(gate_up, "gate_up")
    gm = _as_float("gate_multiplier", gate_multiplier)
    dm = _as_float("down_multiplier", down_multiplier)
    if dout.dtype != gate_up.dtype or dout.device != gate_up.device:
        raise TypeError("dout must have the dtype and device of gate_up")

    n_cols = dout.shape[-1]
    total_cols = input_shape[-1]
    if total_cols != 2 * n_cols or gate_up.numel() != 2 * dout.numel():
        raise ValueError(f"dout of shape {tuple(dout.shape)} does not match packed input {tuple(input_shape)}")
    dout_2d = _rows_2d(dout, n_cols)
    if preserve_inputs:
        gate_up = gate_up.contiguous()
        dgate_up = torch.empty_like(gate_up)
    else:
        if not gate_up.is_contiguous():
            raise ValueError("the in-place backward needs a contiguous gate_up; pass preserve_inputs=True")
        dgate_up = gate_up
    rows = dout_2d.shape[0]
    half = n_cols * gate_up.element_size()
    _lib.check(
        "swiglu_packed_backward",
        _lib.lib.swiglu_b200_bwd(
            dgate_up.data_ptr(), dgate_up.data_ptr() + half, dout_2d.data_ptr(),
            gate_up.data_ptr(), gate_up.data_ptr() + half,
            rows, n_cols, total_cols, total_cols, n_cols, _DTYPE_CODE[gate_up.dtype], gm, dm,
            gate_up.device.index, _stream(gate_up.device),
        ),
    )
    return dgate_up.view(input_shape)


# ------------------------------------------------------------------------------------------
# autograd glue
# ------------------------------------------------------------------------------------------

class ForgeSwiGLUFunction(torch.autograd.Function):
    """``apply(gate, up, gate_multiplier=1.0, down_multiplier=1.0, preserve_inputs=False)``.

    Saves ``(gate_2d, up_2d)`` -- the contiguous 2-D views, gate first -- and recomputes the
    sigmoid in the backward; ``backward`` returns ``(dgate, dup, None, None, None)``.
    """

    @staticmethod
    def forward(ctx, gate, up, gate_multiplier=1.0, down_multiplier=1.0, preserve_inputs=False):
        h, gate_2d, up_2d = swiglu_forward(gate, up, gate_multiplier, down_multiplier)
        ctx.save_for_backward(gate_2d, up_2d)
        ctx.gate_multiplier = _as_float("gate_multiplier", gate_multiplier)
        ctx.down_multiplier = _as_float("down_multiplier", down_multiplier)
        ctx.preserve_inputs = bool(preserve_inputs)
        return h

    @staticmethod
    def backward(ctx, dout):
        gate_2d, up_2d = ctx.saved_tensors
        dgate, dup = swiglu_backward(
            dout, gate_2d, up_2d, ctx.gate_multiplier, ctx.down_multiplier, ctx.preserve_inputs
        )
        return dgate, dup, None, None, None


class ForgePackedSwiGLUFunction(torch.autograd.Function):
    """``apply(gate_up, gate_multiplier=1.0, down_multiplier=1.0, preserve_inputs=False)``.

    Saves ``(gate_up_2d,)`` and ``ctx.input_shape``; ``backward`` returns
    ``(dgate_up, None, None, None)``.
    """

    @staticmethod
    def forward(ctx, gate_up, gate_multiplier=1.0, down_multiplier=1.0, preserve_inputs=False):
        h, gate_up_2d = swiglu_packed_forward(gate_up, gate_multiplier, down_multiplier)
        ctx.save_for_backward(gate_up_2d)
        ctx.input_shape = gate_up.shape
        ctx.gate_multiplier = _as_float("gate_multiplier", gate_multiplier)
        ctx.down_multiplier = _as_float("down_multiplier", down_multiplier)
        ctx.preserve_inputs = bool(preserve_inputs)
        return h

    @staticmethod
    def backward(ctx, dout):
        (gate_up_2d,) = ctx.saved_tensors
        dgate_up = swiglu_packed_backward(
            dout, gate_up_2d, ctx.input_shape, ctx.gate_multiplier, ctx.down_multiplier, ctx.preserve_inputs
        )
        return dgate_up, None, None, None


# ------------------------------------------------------------------------------------------
# Public entry points
# ------------------------------------------------------------------------------------------

def swiglu(
    gate: torch.Tensor,
    up: torch.Tensor,
    gate_multiplier: float = 1.0,
    down_multiplier: float = 1.0,
    preserve_inputs: bool = False,
) -> torch.Tensor:
    """``silu(gate * gate_multiplier) * up * down_multiplier`` with an analytical backward."""
    _check_same_shape_inputs(gate, up)
    _as_float("gate_multiplier", gate_multiplier)
    _as_float("down_multiplier", down_multiplier)
    _require_cuda(gate, "gate")
    return ForgeSwiGLUFunction.apply(gate, up, gate_multiplier, down_multiplier, preserve_inputs)


def swiglu_packed(
    gate_up: torch.Tensor,
    gate_multiplier: float = 1.0,
    down_multiplier: float = 1.0,
    preserve_inputs: bool = False,
) -> torch.Tensor:
    _check_packed_input(gate_up)
    _as_float("gate_multiplier", gate_multiplier)
    _as_float("down_multiplier", down_multiplier)
    _require_cuda(gate_up, "gate_up")
    return ForgePackedSwiGLUFunction.apply(gate_up, gate_multiplier, down_multiplier, preserve_inputs)

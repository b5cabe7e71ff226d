"""SwiGLU forward + backward for activations held in host memory.

``swiglu_fwd_bwd_host`` streams row chunks of pinned host tensors through a device workspace
(``swiglu_b200_host_fwd_bwd`` in the C ABI): host-to-device copies, the two kernels and the
device-to-host copies of successive chunks overlap, so the step costs about one direction of
PCIe traffic instead of both plus the kernels.  The reference has no such call (its operator
takes device tensors only); this is the entry the end-to-end benchmark measures.
"""
from __future__ import annotations

import torch

from . import _lib
from .swiglu import _DTYPE_CODE, _as_float, _check_cuda_dtype, _check_same_shape_inputs


def workspace_bytes(rows: int, cols: int, dtype: torch.dtype) -> int:
    return int(_lib.lib.swiglu_b200_host_workspace_bytes(rows, cols, _DTYPE_CODE[dtype]))


def swiglu_fwd_bwd_host(
    gate: torch.Tensor,
    up: torch.Tensor,
    dout: torch.Tensor,
    gate_multiplier: float = 1.0,
    down_multiplier: float = 1.0,
    *,
    out: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
    workspace: torch.Tensor | None = None,
    device: torch.device | str | int | None = None,
):
    """``(h, dgate, dup)`` as host tensors for host tensors ``gate, up, dout`` of one shape.

    ``out`` supplies the three result tensors (pinned, contiguous, same shape and dtype);
    ``workspace`` a uint8 CUDA tensor used for staging (allocated when omitted).  The inputs are
    not modified.  Work is queued on the current stream of ``device``; the results are complete
    once that stream is synchronised (this function does not synchronise).
    """
    _check_same_shape_inputs(gate, up)
    _check_cuda_dtype(gate)
    gm = _as_float("gate_multiplier", gate_multiplier)
    dm = _as_float("down_multiplier", down_multiplier)
    if gate.is_cuda or dout.is_cuda:
        raise ValueError("swiglu_fwd_bwd_host takes host tensors; use swiglu() for device tensors")
    if dout.shape != gate.shape or dout.dtype != gate.dtype:
        raise ValueError("dout must have the shape and dtype of gate and up")
    if not (gate.is_contiguous() and up.is_contiguous() and dout.is_contiguous()):
        raise ValueError("host tensors must be contiguous")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.type != "cuda":
        raise ValueError("device must be a CUDA device")
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())

    if out is None:
        out = tuple(torch.empty(gate.shape, dtype=gate.dtype, pin_memory=True) for _ in range(3))
    h, dgate, dup = out
    for t in out:
        if t.is_cuda or t.shape != gate.shape or t.dtype != gate.dtype or not t.is_contiguous():
            raise ValueError("out tensors must be contiguous host tensors with the shape and dtype of gate")
    cols = gate.shape[-1] if gate.dim() else 1
    rows = gate.numel() // cols if cols else 0
    if workspace is None:
        workspace = torch.empty(max(workspace_bytes(rows, cols, gate.dtype), 256), dtype=torch.uint8, device=dev)
    if not workspace.is_cuda or workspace.dtype != torch.uint8 or not workspace.is_contiguous():
        raise ValueError("workspace must be a contiguous uint8 CUDA tensor")
    stream = torch.cuda.current_stream(workspace.device)
    _lib.check(
        "swiglu_fwd_bwd_host",
        _lib.lib.swiglu_b200_host_fwd_bwd(
            h.data_ptr(), dgate.data_ptr(), dup.data_ptr(), gate.data_ptr(), up.data_ptr(), dout.data_ptr(),
            rows, cols, _DTYPE_CODE[gate.dtype], gm, dm, workspace.data_ptr(), workspace.numel(),
            workspace.device.index, stream.cuda_stream,
        ),
    )
    # keep the staging buffer alive until the queued work has run
    workspace.record_stream(stream)
    return h, dgate, dup

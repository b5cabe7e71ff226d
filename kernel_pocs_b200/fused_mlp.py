"""Fused gate/up projection + SwiGLU: ``h = silu((x @ w_gate.T) * gm) * (x @ w_up.T) * dm`` in ONE
tcgen05 kernel (``swiglu_b200_gemm_fwd`` in the C ABI), bf16 in, fp32 accumulation, bf16 out.

This is the step in front of the activation path in the reference's patched MLP
(forge/forge/patching/kernels/basic.py:97-102 computes ``swiglu(gate_proj(x), up_proj(x))`` with two
cuBLAS GEMMs and one activation kernel); fusing it removes the write and re-read of both
pre-activation matrices.  The backward is this library's SwiGLU backward kernel on the saved
pre-activations (dgate/dup from dh, gate, up) followed by its tcgen05 backward GEMMs for dx, dw_gate and
dw_up (``SWIGLU_B200_GEMM_BWD=cublas`` selects PyTorch matmuls instead, for comparison).
"""
from __future__ import annotations

import threading

import torch

from . import _lib
from .swiglu import _as_float, swiglu_backward

class _StatusRing:
    """Status words of the tensor-core kernels of one device.

    Every launch gets its own word (launches that overlap on different streams never share one).  A kernel whose
    bounded waits gave up leaves a code there.  The words form a ring of two halves.  When the launches move on
    from one half to the other, the half just left is copied to pinned host memory, asynchronously, after the
    streams that launched into it (the stream current at that moment waits for the others first), and the half
    being entered is inspected: its copy, enqueued one turn ago, must have arrived before its words are handed
    out (and zeroed) again.  If that copy is still in flight the host waits for it, which bounds how far the host
    runs ahead of the device to one turn of the ring (``2 * HALF`` launches); otherwise nothing blocks.  A
    failure surfaces as a ``RuntimeError`` within one turn.  ``check_status`` synchronises and looks at once.

    Taking a word and launching the kernel that uses it happen under one lock (``launch()``), so the copy of a
    half is never enqueued between the two; the forward (caller's thread) and the backward (autograd's thread)
    both launch."""

    HALF = 16
    SLOTS = 2 * HALF

    def __init__(self, device: torch.device):
        self.device = device
        self.dev = torch.zeros(self.SLOTS, dtype=torch.int32, device=device)
        self.words = [self.dev[i:i + 1] for i in range(self.SLOTS)]
        self.host = [torch.zeros(self.HALF, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.pending = [None, None]  # per half: event of its copy in flight
        self.streams = [{}, {}]      # per half: streams that launched into it since its last copy
        self.next = 0
        self.lock = threading.RLock()

    @staticmethod
    def _raise(code: int):
        raise RuntimeError(f"a tensor-core kernel of swiglu_b200 reported a timed-out wait (code {code}); "
                           "its output is incomplete")

    def _inspect(self, half: int):
        """Waits for the copy of ``half`` if one is in flight and raises if it holds a code."""
        ev = self.pending[half]
        if ev is None:
            return
        ev.synchronize()  # returns at once unless the host is a whole turn ahead of the device
        self.pending[half] = None
        codes = [c for c in self.host[half].tolist() if c]
        if codes:
            # reported once: every launch into this half has finished (its copy came after them), so the
            # words can be cleared here; the launches that reuse them zero their own again anyway
            self.host[half].zero_()
            lo = half * self.HALF
            self.dev[lo:lo + self.HALF].zero_()
            self._raise(codes[0])

    def _send(self, half: int):
        """Enqueues the copy of ``half`` to the host behind every stream that launched into it."""
        current = torch.cuda.current_stream(self.device)
        for stream in self.streams[half].values():
            if stream != current:
                current.wait_stream(stream)
        self.streams[half] = {}
        lo = half * self.HALF
        self.host[half].copy_(self.dev[lo:lo + self.HALF], non_blocking=True)
        self.pending[half] = torch.cuda.Event()
        self.pending[half].record(current)

    def _acquire_locked(self) -> torch.Tensor:
        i = self.next
        half, first = divmod(i, self.HALF)
        if first == 0:
            other = 1 - half
            if self.streams[other]:
                self._send(other)
            self._inspect(half)  # may raise: the launch that asked is not made, the next one finds the ring clean
        stream = torch.cuda.current_stream(self.device)
        self.streams[half][stream.cuda_stream] = stream
        self.next = (i + 1) % self.SLOTS
        return self.words[i]

    def acquire(self) -> torch.Tensor:
        """The word for a launch that is about to be made (a one-element view; the C entry zeroes it).  Callers
        that launch should use ``launch()``; this is for tests that fill a word by hand."""
        with self.lock:
            return self._acquire_locked()

    def launch(self):
        """``with ring.launch() as word:`` hands out the next word and holds the ring's lock until the block,
        which enqueues the kernel, is left."""
        return _Launch(self)

    def check(self):
        with self.lock:
            torch.cuda.synchronize(self.device)
            codes = [c for c in self.dev.tolist() if c]
            for half in (0, 1):
                if self.pending[half] is not None:
                    codes += [c for c in self.host[half].tolist() if c]
                    self.host[half].zero_()
                    self.pending[half] = None
                self.streams[half] = {}
            self.dev.zero_()
        if codes:
            self._raise(codes[0])


class _Launch:
    __slots__ = ("ring",)

    def __init__(self, ring: _StatusRing):
        self.ring = ring

    def __enter__(self) -> torch.Tensor:
        self.ring.lock.acquire()
        try:
            return self.ring._acquire_locked()
        except BaseException:
            self.ring.lock.release()
            raise

    def __exit__(self, *exc):
        self.ring.lock.release()
        return False


_status_rings: dict[int, _StatusRing] = {}
_status_rings_lock = threading.Lock()


def _ring(device: torch.device) -> _StatusRing:
    index = device.index if device.index is not None else torch.cuda.current_device()
    ring = _status_rings.get(index)
    if ring is None:
        with _status_rings_lock:
            ring = _status_rings.get(index)
            if ring is None:
                ring = _status_rings[index] = _StatusRing(torch.device("cuda", index))
    return ring


def _status(device: torch.device) -> torch.Tensor:
    """The next status word of ``device`` without a launch (tests fill it by hand)."""
    return _ring(device).acquire()


def _launching(device: torch.device):
    """``with _launching(device) as word:`` around the C call that enqueues a tensor-core kernel."""
    return _ring(device).launch()


def check_status(device: torch.device | int | None = None) -> None:
    """Synchronises ``device`` and raises if a tensor-core launch on it since the last check gave up on an
    internal wait (the kernels bound every wait and report instead of hanging)."""
    if isinstance(device, torch.device):
        index = device.index if device.index is not None else torch.cuda.current_device()
    elif device is None:
        index = torch.cuda.current_device()
    else:
        index = torch.device(device).index or 0
    ring = _status_rings.get(index)
    if ring is not None:
        ring.check()


def selftest_wait_timeout(device: torch.device | int | None = None, mode: int = 0, limit_cycles: int = 2_000_000,
                          code: int = 901) -> torch.Tensor:
    """Test-only: launches the library's one-warp self-test kernel (``swiglu_b200_selftest_wait_timeout``), whose
    single wait is on a barrier that nothing ever arrives at and is limited to ``limit_cycles`` of the SM clock
    (about a millisecond by default).  The kernel gives up, leaves ``code`` in its status word, taken from the
    same ring as every tensor-core launch, and returns; so a later launch or ``check_status`` raises, exactly
    as it would for a real kernel whose wait ran out.  Returns the status word (a one-element view).
    ``mode`` selects the wait under test: 0 CTA-scope, 1 the pair kernels' CTA-scope wait, 2 the same with
    the 200 ns pause between polls, 3 their cluster-scope wait."""
    if device is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    else:
        dev = torch.device(device) if not isinstance(device, int) else torch.device("cuda", device)
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
    with _launching(dev) as status:
        rc = _lib.lib.swiglu_b200_selftest_wait_timeout(status.data_ptr(), int(mode), int(limit_cycles), int(code),
                                                        dev.index, torch.cuda.current_stream(dev).cuda_stream)
    _lib.check("selftest_wait_timeout", rc)
    return status


def _check_operands(x, w_gate, w_up):
    if not (x.is_cuda and w_gate.is_cuda and w_up.is_cuda):
        raise RuntimeError("fused gate/up SwiGLU has a CUDA (sm_100a) kernel only; there is no CPU fallback")
    if not (x.dtype == w_gate.dtype == w_up.dtype == torch.bfloat16):
        raise TypeError("fused gate/up SwiGLU supports bf16 operands only")
    if w_gate.shape != w_up.shape or w_gate.dim() != 2:
        raise ValueError(f"w_gate and w_up must be [n, k] matrices of one shape, got {w_gate.shape} and {w_up.shape}")
    if x.shape[-1] != w_gate.shape[1]:
        raise ValueError(f"x has {x.shape[-1]} features, the weights expect {w_gate.shape[1]}")
    if w_gate.shape[1] % 8 or w_gate.shape[0] % 16:
        raise ValueError("the fused kernel needs k % 8 == 0 and n % 16 == 0")


def gate_up_swiglu_forward(x, w_gate, w_up, gate_multiplier=1.0, down_multiplier=1.0, save_preactivations=False):
    """Returns ``h`` or, with ``save_preactivations``, ``(h, gate, up)`` (gate/up rounded to bf16)."""
    _check_operands(x, w_gate, w_up)
    gm = _as_float("gate_multiplier", gate_multiplier)
    dm = _as_float("down_multiplier", down_multiplier)
    n, k = w_gate.shape
    x2 = x.contiguous().view(-1, k)
    wg, wu = w_gate.contiguous(), w_up.contiguous()
    m = x2.shape[0]
    h = torch.empty((m, n), dtype=x.dtype, device=x.device)
    gate = torch.empty_like(h) if save_preactivations else None
    up = torch.empty_like(h) if save_preactivations else None
    with _launching(x.device) as status:
        rc = _lib.lib.swiglu_b200_gemm_fwd(
            h.data_ptr(), gate.data_ptr() if save_preactivations else None,
            up.data_ptr() if save_preactivations else None, x2.data_ptr(), wg.data_ptr(), wu.data_ptr(),
            m, n, k, gm, dm, status.data_ptr(), x.device.index,
            torch.cuda.current_stream(x.device).cuda_stream,
        )
    _lib.check("gate_up_swiglu_forward", rc)
    h = h.view(*x.shape[:-1], n)
    if save_preactivations:
        return h, gate, up
    return h


def lora_gate_up_swiglu_forward(x, w_gate, w_up, A_gate, B_gate, s_gate, A_up, B_up, s_up, save_eg=False,
                                activation: str = "silu"):
    """``h = act(e) * g`` (``activation``: ``"silu"``, ``"gelu_tanh"`` or ``"gelu_exact"``) with ``e = x W_g^T + s_g (x A_g^T) B_g^T`` and ``g`` likewise, in ONE tcgen05 launch
    (``swiglu_b200_lora_gemm_fwd``): the adapter terms ride along as extra steps of the projections' contraction.
    The counterpart of the reference's ``fused_gate_up_swiglu`` (kernels/lora_mlp/experiments/v2/
    lora_mlp_kernel_v2.py:141-209).  W ``[n, k]``, A ``[r, k]``, B ``[n, r]``, all bf16; r a multiple of 8 up to 64.
    Returns ``(h, e, g)`` with ``save_eg`` (e, g rounded to bf16, for a backward pass), else ``(h, None, None)``."""
    _check_operands(x, w_gate, w_up)
    n, k = w_gate.shape
    r = A_gate.shape[0]
    if A_gate.shape != (r, k) or A_up.shape != (r, k) or B_gate.shape != (n, r) or B_up.shape != (n, r):
        raise ValueError("expected A_gate, A_up of shape [r, k] and B_gate, B_up of shape [n, r]")
    if any(t.dtype != torch.bfloat16 for t in (A_gate, A_up, B_gate, B_up)):
        raise TypeError("fused gate/up SwiGLU supports bf16 operands only")
    if r % 8 or not 8 <= r <= 64:
        raise ValueError("the fused kernel needs a rank that is a multiple of 8 in [8, 64]")
    sg, su = _as_float("s_gate", s_gate), _as_float("s_up", s_up)
    x2 = x.contiguous().view(-1, k)
    m = x2.shape[0]
    # [s_g x A_g^T | s_u x A_u^T]: one skinny library GEMM against the stacked, pre-scaled A matrices (scaling
    # the small [2r, k] factor instead of the [m, 2r] product keeps this to two tiny launches and one GEMM)
    xa = x2 @ torch.cat((A_gate * sg, A_up * su), dim=0).t()
    wg, wu, bg, bu = w_gate.contiguous(), w_up.contiguous(), B_gate.contiguous(), B_up.contiguous()
    h = torch.empty((m, n), dtype=x.dtype, device=x.device)
    e = torch.empty_like(h) if save_eg else None
    g = torch.empty_like(h) if save_eg else None
    if activation not in ("silu", "gelu_tanh", "gelu_exact"):
        raise ValueError(f"activation must be 'silu', 'gelu_tanh' or 'gelu_exact', got {activation!r}")
    common = (h.data_ptr(), e.data_ptr() if save_eg else None, g.data_ptr() if save_eg else None, x2.data_ptr(),
              wg.data_ptr(), wu.data_ptr(), xa.data_ptr(), bg.data_ptr(), bu.data_ptr(), m, n, k, r)
    with _launching(x.device) as status:
        tail = (status.data_ptr(), x.device.index, torch.cuda.current_stream(x.device).cuda_stream)
        if activation == "silu":
            rc = _lib.lib.swiglu_b200_lora_gemm_fwd(*common, 1.0, 1.0, *tail)
        else:
            rc = _lib.lib.swiglu_b200_lora_geglu_gemm_fwd(*common, int(activation == "gelu_tanh"), *tail)
    _lib.check("lora_gate_up_swiglu_forward", rc)
    return h.view(*x.shape[:-1], n), e, g


def gate_up_swiglu_backward_gemms(dgate, dup, x, w_gate, w_up, need_dx=True, need_dw=True):
    """``(dx, dw_gate, dw_up)`` from the activation gradients, by this library's tcgen05 kernels
    (``swiglu_b200_gemm_bwd``); entries that are not needed are ``None``."""
    n, k = w_gate.shape
    x2 = x.contiguous().view(-1, k)
    m = x2.shape[0]
    dgate, dup = dgate.contiguous().view(m, n), dup.contiguous().view(m, n)
    wg, wu = w_gate.contiguous(), w_up.contiguous()
    dx = torch.empty_like(x2) if need_dx else None
    dwg = torch.empty_like(wg) if need_dw else None
    dwu = torch.empty_like(wu) if need_dw else None
    if not (need_dx or need_dw):
        return None, None, None
    with _launching(x.device) as status:
        rc = _lib.lib.swiglu_b200_gemm_bwd(
            dx.data_ptr() if need_dx else None, dwg.data_ptr() if need_dw else None,
            dwu.data_ptr() if need_dw else None, dgate.data_ptr(), dup.data_ptr(), x2.data_ptr(), wg.data_ptr(),
            wu.data_ptr(), m, n, k, status.data_ptr(), x.device.index,
            torch.cuda.current_stream(x.device).cuda_stream,
        )
    _lib.check("gate_up_swiglu_backward_gemms", rc)
    return (dx.view(x.shape) if need_dx else None), dwg, dwu


def _own_backward_gemms(n: int, k: int) -> bool:
    import os

    return os.environ.get("SWIGLU_B200_GEMM_BWD", "own") != "cublas" and k % 16 == 0 and n % 8 == 0


class FusedGateUpSwiGLUFunction(torch.autograd.Function):
    """``apply(x, w_gate, w_up, gate_multiplier=1.0, down_multiplier=1.0)``."""

    @staticmethod
    def forward(ctx, x, w_gate, w_up, gate_multiplier=1.0, down_multiplier=1.0):
        h, gate, up = gate_up_swiglu_forward(x, w_gate, w_up, gate_multiplier, down_multiplier, True)
        ctx.save_for_backward(x, w_gate, w_up, gate, up)
        ctx.gate_multiplier = _as_float("gate_multiplier", gate_multiplier)
        ctx.down_multiplier = _as_float("down_multiplier", down_multiplier)
        return h

    @staticmethod
    def backward(ctx, dh):
        x, w_gate, w_up, gate, up = ctx.saved_tensors
        n, k = w_gate.shape
        # gate/up are private to this node, so the in-place backward is safe
        dgate, dup = swiglu_backward(dh.reshape(-1, n), gate, up, ctx.gate_multiplier, ctx.down_multiplier, False)
        if _own_backward_gemms(n, k):
            need_dw = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
            dx, dw_gate, dw_up = gate_up_swiglu_backward_gemms(dgate, dup, x, w_gate, w_up,
                                                               ctx.needs_input_grad[0], need_dw)
            return dx, dw_gate, dw_up, None, None
        x2 = x.reshape(-1, k)
        dx = dw_gate = dw_up = None
        if ctx.needs_input_grad[0]:
            dx = torch.addmm(dgate @ w_gate, dup, w_up).view(x.shape)
        if ctx.needs_input_grad[1]:
            dw_gate = dgate.t() @ x2
        if ctx.needs_input_grad[2]:
            dw_up = dup.t() @ x2
        return dx, dw_gate, dw_up, None, None


def fused_gate_up_swiglu(x, w_gate, w_up, gate_multiplier=1.0, down_multiplier=1.0):
    """``silu((x @ w_gate.T) * gm) * (x @ w_up.T) * dm`` with autograd support."""
    _check_operands(x, w_gate, w_up)
    return FusedGateUpSwiGLUFunction.apply(x, w_gate, w_up, gate_multiplier, down_multiplier)

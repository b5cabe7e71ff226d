"""CPU ORACLE -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Python face of the oracle for the fused SwiGLU path of Forge-researchlab/kernel-POCs.  Only
tests/, __graft_entry__.smoke() and the cpu_baseline / ``--impl reference`` legs of bench.py
may import this module; the product package never does.

Two restatements live here:

* the plain-C one (oracle/swiglu_oracle.c, loaded through ctypes): explicit rounding chain of
  the reference, the round-once target, and a double-precision truth;
* ``aten_*``: the reference's CPU path as it actually executes -- ATen operators in the order
  of torch_swiglu_reference (kernels/swiglu/swiglu.py:179-188) with the backward derived by
  autograd, which is what the reference's ``swiglu()`` does for CPU tensors (:396-397).  This
  is the arm that bench.py times as the reference's CPU implementation.

Parity of both is pinned against vectors produced by the reference itself
(tests/golden/*.npz, written by tests/golden/make_golden.py); tests/test_oracle_golden.py
holds the comparison.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libswiglu_oracle.so"

F32, F16, BF16 = 0, 1, 2
DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


def build(force: bool = False) -> Path:
    """Compiles oracle/swiglu_oracle.c with the recipe in oracle/Makefile."""
    src = HERE / "swiglu_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        proc = subprocess.run(["make", "-C", str(HERE), "-B"], capture_output=True, text=True)
        if proc.returncode != 0 or not LIB_PATH.exists():
            raise RuntimeError(f"building the CPU oracle failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(LIB_PATH))
        p, i64, f, d, i = ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_double, ctypes.c_int
        for name in ("swiglu_oracle_fwd_chain", "swiglu_oracle_fwd_once"):
            getattr(L, name).restype = i
            getattr(L, name).argtypes = [i, i64, p, p, f, f, p]
        for name in ("swiglu_oracle_bwd_chain", "swiglu_oracle_bwd_once"):
            getattr(L, name).restype = i
            getattr(L, name).argtypes = [i, i64, p, p, p, f, f, p, p]
        L.swiglu_oracle_fwd_f64.restype = i
        L.swiglu_oracle_fwd_f64.argtypes = [i, i64, p, p, d, d, p]
        L.swiglu_oracle_bwd_f64.restype = i
        L.swiglu_oracle_bwd_f64.argtypes = [i, i64, p, p, p, d, d, p, p, p]
        L.geglu_oracle_fwd.restype = i
        L.geglu_oracle_fwd.argtypes = [i, i, i, i64, p, p, p]
        L.geglu_oracle_bwd.restype = i
        L.geglu_oracle_bwd.argtypes = [i, i, i, i64, p, p, p, p, p]
        L.geglu_oracle_f64.restype = i
        L.geglu_oracle_f64.argtypes = [i, i, i64, p, p, p, p, p, p, p]
        L.swiglu_oracle_to_f32.restype = None
        L.swiglu_oracle_to_f32.argtypes = [i, i64, p, p]
        L.swiglu_oracle_from_f32.restype = None
        L.swiglu_oracle_from_f32.argtypes = [i, i64, p, p]
        _lib = L
    return _lib


def _flat(x: torch.Tensor) -> torch.Tensor:
    if x.device.type != "cpu":
        raise ValueError("the oracle works on host tensors")
    return x.detach().contiguous().view(-1)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


# ------------------------------------------------------------------------------------------
# plain-C restatement
# ------------------------------------------------------------------------------------------

def fwd(gate: torch.Tensor, up: torch.Tensor, gm: float = 1.0, dm: float = 1.0, variant: str = "chain") -> torch.Tensor:
    """h in the dtype of ``gate``.  variant: "chain" = the reference's rounding points,
    "once" = fp32 throughout with one final rounding."""
    g, u = _flat(gate), _flat(up)
    out = torch.empty_like(g)
    fn = getattr(lib(), f"swiglu_oracle_fwd_{variant}")
    _check(fn(DTYPE_CODE[gate.dtype], g.numel(), g.data_ptr(), u.data_ptr(), gm, dm, out.data_ptr()), "oracle fwd")
    return out.view(gate.shape)


def bwd(dout: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, gm: float = 1.0, dm: float = 1.0,
        variant: str = "chain"):
    """(dgate, dup) in the dtype of ``gate``."""
    d, g, u = _flat(dout), _flat(gate), _flat(up)
    dgate, dup = torch.empty_like(g), torch.empty_like(u)
    fn = getattr(lib(), f"swiglu_oracle_bwd_{variant}")
    _check(
        fn(DTYPE_CODE[gate.dtype], g.numel(), d.data_ptr(), g.data_ptr(), u.data_ptr(), gm, dm,
           dgate.data_ptr(), dup.data_ptr()),
        "oracle bwd",
    )
    return dgate.view(gate.shape), dup.view(gate.shape)


def fwd_f64(gate: torch.Tensor, up: torch.Tensor, gm: float = 1.0, dm: float = 1.0) -> torch.Tensor:
    g, u = _flat(gate), _flat(up)
    out = torch.empty(g.numel(), dtype=torch.float64)
    _check(
        lib().swiglu_oracle_fwd_f64(DTYPE_CODE[gate.dtype], g.numel(), g.data_ptr(), u.data_ptr(), gm, dm,
                                    out.data_ptr()),
        "oracle fwd f64",
    )
    return out.view(gate.shape)


def bwd_f64(dout: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, gm: float = 1.0, dm: float = 1.0):
    """(dgate, dup, dgate_scale) as float64; dgate_scale = |dh*dm*up*gm|."""
    d, g, u = _flat(dout), _flat(gate), _flat(up)
    n = g.numel()
    dgate, dup, scale = (torch.empty(n, dtype=torch.float64) for _ in range(3))
    _check(
        lib().swiglu_oracle_bwd_f64(DTYPE_CODE[gate.dtype], n, d.data_ptr(), g.data_ptr(), u.data_ptr(), gm, dm,
                                    dgate.data_ptr(), dup.data_ptr(), scale.data_ptr()),
        "oracle bwd f64",
    )
    return dgate.view(gate.shape), dup.view(gate.shape), scale.view(gate.shape)


# GeGLU, the sibling operator (reference kernels/geglu/geglu.py)

def _tanh_flag(approximate: str) -> int:
    if approximate not in ("tanh", "none"):
        raise ValueError(approximate)
    return 1 if approximate == "tanh" else 0


def geglu_fwd(gate: torch.Tensor, up: torch.Tensor, approximate: str = "tanh", variant: str = "chain") -> torch.Tensor:
    g, u = _flat(gate), _flat(up)
    out = torch.empty_like(g)
    _check(lib().geglu_oracle_fwd(int(variant == "once"), DTYPE_CODE[gate.dtype], _tanh_flag(approximate), g.numel(),
                                  g.data_ptr(), u.data_ptr(), out.data_ptr()), "oracle geglu fwd")
    return out.view(gate.shape)


def geglu_bwd(dout: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, approximate: str = "tanh",
              variant: str = "chain"):
    d, g, u = _flat(dout), _flat(gate), _flat(up)
    dgate, dup = torch.empty_like(g), torch.empty_like(u)
    _check(lib().geglu_oracle_bwd(int(variant == "once"), DTYPE_CODE[gate.dtype], _tanh_flag(approximate), g.numel(),
                                  d.data_ptr(), g.data_ptr(), u.data_ptr(), dgate.data_ptr(), dup.data_ptr()),
           "oracle geglu bwd")
    return dgate.view(gate.shape), dup.view(gate.shape)


def geglu_f64(dout: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, approximate: str = "tanh"):
    """(h, dgate, dup, dgate_scale) as float64."""
    d, g, u = _flat(dout), _flat(gate), _flat(up)
    n = g.numel()
    h, dgate, dup, scale = (torch.empty(n, dtype=torch.float64) for _ in range(4))
    _check(lib().geglu_oracle_f64(DTYPE_CODE[gate.dtype], _tanh_flag(approximate), n, d.data_ptr(), g.data_ptr(),
                                  u.data_ptr(), h.data_ptr(), dgate.data_ptr(), dup.data_ptr(), scale.data_ptr()),
           "oracle geglu f64")
    return tuple(t.view(gate.shape) for t in (h, dgate, dup, scale))


def packed_split(gate_up: torch.Tensor):
    """gate = first half of the last axis, up = second half (swiglu.py:135-137, 195-197)."""
    half = gate_up.shape[-1] // 2
    return gate_up[..., :half].contiguous(), gate_up[..., half:].contiguous()


# ------------------------------------------------------------------------------------------
# ATen restatement: the reference's CPU path as executed
# ------------------------------------------------------------------------------------------

def aten_fwd(gate: torch.Tensor, up: torch.Tensor, gm: float = 1.0, dm: float = 1.0) -> torch.Tensor:
    act = torch.nn.functional.silu(gate.float() * float(gm)).to(gate.dtype)
    return (act * up) * float(dm)


def aten_fwd_bwd(gate: torch.Tensor, up: torch.Tensor, dout: torch.Tensor, gm: float = 1.0, dm: float = 1.0):
    """(h, dgate, dup): forward by the composite, backward by autograd, as the reference's
    swiglu() does for host tensors."""
    g = gate.detach().clone().requires_grad_(True)
    u = up.detach().clone().requires_grad_(True)
    h = aten_fwd(g, u, gm, dm)
    dgate, dup = torch.autograd.grad(h, (g, u), dout)
    return h.detach(), dgate, dup


# ------------------------------------------------------------------------------------------
# comparison helpers
# ------------------------------------------------------------------------------------------

def ordinal(x: torch.Tensor) -> torch.Tensor:
    """Maps floating-point bit patterns to integers that are monotone in the value, so that
    |ordinal(a) - ordinal(b)| counts representable values between a and b (ulp distance).
    +0 and -0 map to the same integer.  NaNs must be masked out by the caller."""
    if x.dtype == torch.float32:
        bits = x.contiguous().view(torch.int32).to(torch.int64)
        sign_bit = 1 << 31
    elif x.dtype in (torch.float16, torch.bfloat16):
        bits = x.contiguous().view(torch.int16).to(torch.int64)
        sign_bit = 1 << 15
    else:
        raise TypeError(x.dtype)
    bits = bits & ((sign_bit << 1) - 1)
    mag = bits & (sign_bit - 1)
    return torch.where((bits & sign_bit) != 0, -mag, mag)


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Elementwise ulp distance; positions where both are NaN count 0, where only one is NaN
    count a large number."""
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    dist = (ordinal(a) - ordinal(b)).abs()
    an, bn = torch.isnan(a), torch.isnan(b)
    dist = torch.where(an & bn, torch.zeros_like(dist), dist)
    dist = torch.where(an ^ bn, torch.full_like(dist, 1 << 40), dist)
    return dist


def to_numpy_bits(x: torch.Tensor) -> np.ndarray:
    """Raw storage as a numpy array (uint16 for the 16-bit types)."""
    x = x.detach().cpu().contiguous()
    if x.dtype == torch.float32:
        return x.numpy().copy()
    return x.view(torch.int16).numpy().view(np.uint16).copy()


def from_numpy_bits(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    if dtype == torch.float32:
        return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32).copy())
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(dtype)

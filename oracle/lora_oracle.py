"""CPU ORACLE -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Double-precision numpy restatement of the LoRA MLP that surrounds the SwiGLU path in the reference's LoRA
training step: every projection is ``x W^T + s (x A^T) B^T`` with W ``[out, in]``, A ``[r, in]``, B ``[out, r]``
(``matmul_lora``, kernels/lora_mlp/reference/lora_mlp_pytorch.py:22-58), the block is
``down(silu(gate(X)) * up(X))`` (``lora_swiglu_mlp``, :64-106), and the gradients are those of its hand-written
backward (``LoRAMLP.backward``, :145-236) for X and the six adapter matrices, base weights frozen.

Pinned against tests/golden/lora_mlp.npz, which holds outputs of those reference functions themselves
(written by tests/golden/make_golden.py); tests/test_oracle_golden.py holds the comparison.  Only tests/ may
import this module.
"""
from __future__ import annotations

import numpy as np


def _proj(x, W, A, B, s):
    y = x @ W.T
    if A is not None:
        y = y + s * ((x @ A.T) @ B.T)
    return y


def _sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def lora_mlp_fwd_bwd(X, p, dY):
    """``X`` [..., H], ``p`` a dict with W_/A_/B_/s_ entries for gate, up and down, ``dY`` like the output.
    Returns a dict: out, e, g, h, dX and dA_*/dB_* for the three projections (float64 arrays)."""
    f = lambda a: None if a is None else np.asarray(a, dtype=np.float64)
    x = f(X).reshape(-1, X.shape[-1])
    dy = f(dY).reshape(-1, dY.shape[-1])
    Wg, Ag, Bg, sg = f(p["W_gate"]), f(p["A_gate"]), f(p["B_gate"]), float(p["s_gate"])
    Wu, Au, Bu, su = f(p["W_up"]), f(p["A_up"]), f(p["B_up"]), float(p["s_up"])
    Wd, Ad, Bd, sd = f(p["W_down"]), f(p["A_down"]), f(p["B_down"]), float(p["s_down"])

    e = _proj(x, Wg, Ag, Bg, sg)
    g = _proj(x, Wu, Au, Bu, su)
    sig = _sigmoid(e)
    silu = e * sig
    h = silu * g
    out = _proj(h, Wd, Ad, Bd, sd)

    r = {"out": out.reshape(*X.shape[:-1], -1), "e": e, "g": g, "h": h}
    dh = dy @ Wd
    if Ad is not None:
        dh = dh + sd * ((dy @ Bd) @ Ad)
        r["dA_down"] = sd * ((dy @ Bd).T @ h)
        r["dB_down"] = sd * (dy.T @ (h @ Ad.T))
    dg = dh * silu
    de = dh * g * (sig * (1.0 + e * (1.0 - sig)))
    dX = de @ Wg + dg @ Wu
    if Ag is not None:
        r["dA_gate"] = sg * ((de @ Bg).T @ x)
        r["dB_gate"] = sg * (de.T @ (x @ Ag.T))
        r["dA_up"] = su * ((dg @ Bu).T @ x)
        r["dB_up"] = su * (dg.T @ (x @ Au.T))
        dX = dX + sg * ((de @ Bg) @ Ag) + su * ((dg @ Bu) @ Au)
    r["dX"] = dX.reshape(X.shape)
    r["de"], r["dg"] = de, dg
    return r

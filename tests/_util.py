"""Comparison helpers shared by the parity tests."""
from __future__ import annotations

import math

import torch

from oracle import oracle as O

DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
MANTISSA_BITS = {torch.float32: 23, torch.float16: 10, torch.bfloat16: 7}
MIN_NORMAL_EXP = {torch.float32: -126, torch.float16: -14, torch.bfloat16: -126}
MAX_FINITE = {torch.float32: 3.4028234663852886e38, torch.float16: 65504.0, torch.bfloat16: 3.3895313892515355e38}


def ulp_spacing(truth: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Distance between neighbouring values of ``dtype`` around each (float64) truth value."""
    t = truth.abs().double()
    exp = torch.floor(torch.log2(t.clamp_min(1e-300)))
    exp = exp.clamp_min(MIN_NORMAL_EXP[dtype])
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), exp - MANTISSA_BITS[dtype])


def assert_rounded_once(got: torch.Tensor, truth: torch.Tensor, what: str, slack: float = 0.51,
                        extra: torch.Tensor | None = None) -> None:
    """``got`` (fp16/bf16) must be a correct rounding of the float64 truth, up to ``slack``
    ulps (0.5 = perfect rounding; the small excess covers the fp32 evaluation error) plus an
    optional absolute allowance ``extra`` per element (dgate: the fp32 evaluation error scales
    with |dh*up|, not with the result, where the derivative factor crosses zero)."""
    dtype = got.dtype
    g = got.detach().cpu().double().reshape(-1)
    t = truth.detach().cpu().double().reshape(-1)
    finite = torch.isfinite(t) & (t.abs() < MAX_FINITE[dtype])
    assert torch.equal(torch.isnan(g), torch.isnan(t)), f"{what}: NaN pattern differs"
    err = (g - t).abs()[finite]
    # 1e-30: where exp(-z) overflows fp32 (z < -88.7) the fp32 closed form returns 0 for a
    # truth of magnitude < 1e-36
    bound = slack * ulp_spacing(t[finite], dtype) + 1e-30
    if extra is not None:
        bound = bound + extra.detach().cpu().double().reshape(-1)[finite]
    bad = err > bound
    assert not bad.any(), (
        f"{what}: {int(bad.sum())} of {bad.numel()} elements are not within {slack} ulp of the exact value; "
        f"worst {float((err / ulp_spacing(t[finite], dtype)).max()):.3f} ulp"
    )


def assert_ulp(got: torch.Tensor, want: torch.Tensor, max_ulp: int, what: str, min_exact: float | None = None) -> None:
    d = O.ulp_distance(got.detach().cpu(), want.detach().cpu())
    worst = int(d.max()) if d.numel() else 0
    assert worst <= max_ulp, f"{what}: worst ulp distance {worst} > {max_ulp} ({int((d > max_ulp).sum())} elements)"
    if min_exact is not None and d.numel():
        exact = float((d == 0).double().mean())
        assert exact >= min_exact, f"{what}: only {exact:.5f} of elements bit-identical (need {min_exact})"


def assert_rel_scaled(got: torch.Tensor, truth: torch.Tensor, rel: float, what: str, scale: torch.Tensor | None = None,
                      floor: float = 1e-25) -> None:
    """|got - truth| <= rel * max(|truth|, scale, floor), NaN/inf patterns equal."""
    g = got.detach().cpu().double().reshape(-1)
    t = truth.detach().cpu().double().reshape(-1)
    assert torch.equal(torch.isnan(g), torch.isnan(t)), f"{what}: NaN pattern differs"
    inf = torch.isinf(t)
    assert torch.equal(g[inf], t[inf]), f"{what}: infinities differ"
    ok = torch.isfinite(t) & (t.abs() < 3.0e38)
    denom = t.abs()
    if scale is not None:
        denom = torch.maximum(denom, scale.detach().cpu().double().reshape(-1))
    denom = denom.clamp_min(floor)
    ratio = ((g - t).abs() / denom)[ok]
    worst = float(ratio.max()) if ratio.numel() else 0.0
    assert worst <= rel, f"{what}: worst scaled error {worst:.3e} > {rel:.1e}"


def guarded(shape, dtype, device, pad: int = 64, fill: float = 1234.0):
    """A tensor of ``shape`` carved out of a larger sentinel-filled buffer; returns
    (view, check) where check() asserts that the guard bands are untouched."""
    n = math.prod(shape)
    buf = torch.full((n + 2 * pad,), fill, dtype=dtype, device=device)
    view = buf[pad:pad + n].view(shape)

    def check(what: str = "output") -> None:
        lo, hi = buf[:pad], buf[pad + n:]
        assert bool((lo == fill).all()) and bool((hi == fill).all()), f"{what}: wrote outside its extent"

    return view, check

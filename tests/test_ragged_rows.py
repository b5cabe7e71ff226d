"""Ragged rows: pitched and mutually skewed tensors through the C ABI.

The packed gate|up layout with a half-width that is not a multiple of 16 bytes (and, generally, any
row pitch, width or base address that is not) is served by kernels that work out the alignment row
by row: aligned 32-byte accesses for the primary output, window loads for the inputs, and a second
output (dup) whose vectors are realigned across lanes before they are stored.  These tests drive
``swiglu_b200_fwd`` / ``swiglu_b200_bwd`` directly with arbitrary pitches and base offsets and hold
the results to the flat kernels on contiguous copies of the same data, bit for bit (the flat kernels
are the ones the oracle tests pin).  Every buffer is filled with a sentinel first: the gaps between
rows and the bands around the tensors must come back untouched.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from kernel_pocs_b200 import _lib
from kernels.swiglu import swiglu_backward, swiglu_forward, swiglu_packed_backward, swiglu_packed_forward

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
CODE = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
SENTINEL = 1234.0
PAD = 64


class Pitched:
    """rows x cols elements inside a sentinel-filled buffer, with a row pitch and a base offset."""

    def __init__(self, rows, cols, pitch, offset, dtype, values=None):
        self.rows, self.cols, self.pitch, self.offset = rows, cols, pitch, offset
        n = PAD + offset + rows * pitch + PAD
        self.buf = torch.full((n,), SENTINEL, dtype=dtype, device=DEVICE)
        self.start = PAD + offset
        self.view = torch.as_strided(self.buf, (rows, cols), (pitch, 1), self.start)
        if values is not None:
            self.view.copy_(values)
        self.mask = torch.ones(n, dtype=torch.bool, device=DEVICE)
        torch.as_strided(self.mask, (rows, cols), (pitch, 1), self.start).fill_(False)

    @property
    def ptr(self):
        return self.view.data_ptr()

    def untouched(self) -> bool:
        return bool((self.buf[self.mask] == SENTINEL).all())


def flat_reference(gate, up, dout, gm, dm):
    h = swiglu_forward(gate.contiguous(), up.contiguous(), gm, dm)[0]
    dgate, dup = swiglu_backward(dout.contiguous(), gate.contiguous(), up.contiguous(), gm, dm, preserve_inputs=True)
    return h, dgate, dup


def test_random_pitches_offsets_and_modes():
    rng = np.random.default_rng(20250)
    stream = torch.cuda.current_stream().cuda_stream
    widths = [1, 2, 3, 5, 7, 8, 9, 15, 16, 17, 31, 33, 63, 65, 127, 129, 255, 257, 1001, 2049, 5503]
    ragged_seen = 0
    for case in range(240):
        dtype = [torch.bfloat16, torch.float16, torch.float32][case % 3]
        rows = int(rng.choice([1, 2, 3, 7, 33, 70]))
        cols = int(rng.choice(widths)) if rng.random() < 0.8 else int(rng.integers(1, 3000))
        gm, dm = (1.0, 1.0) if rng.random() < 0.5 else (float(rng.uniform(0.5, 1.5)), float(rng.uniform(0.5, 1.5)))
        extra = lambda: int(rng.choice([0, 0, 1, 3, 8, 13, 17, 29]))
        off = lambda: int(rng.integers(0, 34))  # up to 33 elements: every skew against a 32-byte frame occurs
        g = torch.Generator(device=DEVICE).manual_seed(case)
        gate0, up0, dout0 = (1.5 * torch.randn(rows, cols, generator=g, device=DEVICE).to(dtype) for _ in range(3))
        want_h, want_dg, want_du = flat_reference(gate0, up0, dout0, gm, dm)
        pitch_in, pitch_out = cols + extra(), cols + extra()
        packed = rng.random() < 0.4  # gate|up halves of one buffer, as swiglu_packed lays them out
        if packed:
            pitch_in = 2 * cols + extra()
            both = Pitched(rows, 2 * cols, pitch_in, off(), dtype, torch.cat([gate0, up0], dim=1))
            gate_ptr, up_ptr = both.ptr, both.ptr + cols * gate0.element_size()
            inputs = [both]
        else:
            gate, up = Pitched(rows, cols, pitch_in, off(), dtype, gate0), Pitched(rows, cols, pitch_in, off(), dtype, up0)
            gate_ptr, up_ptr = gate.ptr, up.ptr
            inputs = [gate, up]
        dout = Pitched(rows, cols, pitch_out, off(), dtype, dout0)
        what = f"case {case}: {dtype} rows={rows} cols={cols} pitch_in={pitch_in} pitch_out={pitch_out} packed={packed}"

        # forward
        out = Pitched(rows, cols, pitch_out, off(), dtype)
        code = _lib.lib.swiglu_b200_plan_fwd(out.ptr, gate_ptr, up_ptr, rows, cols, pitch_in, pitch_out, CODE[dtype])
        ragged_seen += bool(code & 0x800)
        _lib.check(what, _lib.lib.swiglu_b200_fwd(out.ptr, gate_ptr, up_ptr, rows, cols, pitch_in, pitch_out,
                                                  CODE[dtype], gm, dm, 0, stream))
        assert torch.equal(out.view, want_h), what + " h"
        assert out.untouched(), what + " h wrote outside its rows"

        # backward, out of place: dgate/dup halves of one buffer (packed) or two buffers with their own offsets
        if packed:
            pitch_grad = 2 * cols + extra()
            grads = Pitched(rows, 2 * cols, pitch_grad, off(), dtype)
            dg_ptr, du_ptr = grads.ptr, grads.ptr + cols * gate0.element_size()
            outs = [grads]
            read = lambda: (grads.view[:, :cols], grads.view[:, cols:])
        else:
            pitch_grad = cols + extra()
            dg, du = Pitched(rows, cols, pitch_grad, off(), dtype), Pitched(rows, cols, pitch_grad, off(), dtype)
            dg_ptr, du_ptr = dg.ptr, du.ptr
            outs = [dg, du]
            read = lambda: (dg.view, du.view)
        code = _lib.lib.swiglu_b200_plan_bwd(dg_ptr, du_ptr, dout.ptr, gate_ptr, up_ptr, rows, cols, pitch_in,
                                             pitch_grad, pitch_out, CODE[dtype])
        ragged_seen += bool(code & 0x800)
        _lib.check(what, _lib.lib.swiglu_b200_bwd(dg_ptr, du_ptr, dout.ptr, gate_ptr, up_ptr, rows, cols, pitch_in,
                                                  pitch_grad, pitch_out, CODE[dtype], gm, dm, 0, stream))
        got_dg, got_du = read()
        assert torch.equal(got_dg, want_dg), what + " dgate"
        assert torch.equal(got_du, want_du), what + " dup"
        assert all(t.untouched() for t in outs), what + " gradients wrote outside their rows"

        # backward, in place over gate/up
        _lib.check(what, _lib.lib.swiglu_b200_bwd(gate_ptr, up_ptr, dout.ptr, gate_ptr, up_ptr, rows, cols, pitch_in,
                                                  pitch_in, pitch_out, CODE[dtype], gm, dm, 0, stream))
        if packed:
            got_dg, got_du = both.view[:, :cols], both.view[:, cols:]
        else:
            got_dg, got_du = gate.view, up.view
        assert torch.equal(got_dg, want_dg), what + " dgate in place"
        assert torch.equal(got_du, want_du), what + " dup in place"
        assert all(t.untouched() for t in inputs) and dout.untouched(), what + " in place wrote outside its rows"
        assert torch.equal(dout.view, dout0), what + " dout changed"
    assert ragged_seen > 150, "the ragged-row kernels should serve most of these cases"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("half_width", [3, 257, 1001, 5503])
@pytest.mark.parametrize("offset", [0, 1, 5])
def test_packed_operator_with_odd_half_widths_and_misaligned_bases(dtype, half_width, offset):
    """``swiglu_packed_forward/backward`` (the operator's own wrappers) on a gate|up buffer whose half-width is odd
    and whose first element sits ``offset`` elements past a 16-byte boundary: bit-equal to the separate layout."""
    rows = 37
    g = torch.Generator(device=DEVICE).manual_seed(half_width + offset)
    gate0, up0, dout = (2.0 * torch.randn(rows, half_width, generator=g, device=DEVICE).to(dtype) for _ in range(3))
    want_h, want_dg, want_du = flat_reference(gate0, up0, dout, 1.5, 0.5)
    for preserve in (True, False):
        src = Pitched(rows, 2 * half_width, 2 * half_width, offset, dtype, torch.cat([gate0, up0], dim=1))
        gate_up = src.view
        assert gate_up.is_contiguous() and (gate_up.data_ptr() % 16) == (offset * gate_up.element_size()) % 16
        h, saved = swiglu_packed_forward(gate_up, 1.5, 0.5)
        assert torch.equal(h, want_h)
        grad = swiglu_packed_backward(dout, saved, gate_up.shape, 1.5, 0.5, preserve_inputs=preserve)
        assert torch.equal(grad[:, :half_width], want_dg) and torch.equal(grad[:, half_width:], want_du)
        assert src.untouched()
        if preserve:
            assert torch.equal(gate_up, torch.cat([gate0, up0], dim=1))
        else:
            assert grad.data_ptr() == gate_up.data_ptr()


def test_large_packed_odd_half_width_in_place():
    """The benchmark's ragged variant at size: 4096 token rows, half-width 11009, first row sliced off so that the
    base is misaligned too; forward and in-place backward against the separate layout."""
    rows, half = 4096, 11009
    g = torch.Generator(device=DEVICE).manual_seed(5)
    full = (2.0 * torch.randn(rows + 1, 2 * half, generator=g, device=DEVICE)).bfloat16()
    dout = torch.randn(rows, half, generator=g, device=DEVICE).bfloat16()
    gate_up = full[1:]
    gate0, up0 = gate_up[:, :half].contiguous(), gate_up[:, half:].contiguous()
    want_h, want_dg, want_du = flat_reference(gate0, up0, dout, 1.0, 1.0)
    first_row = full[0].clone()
    h, saved = swiglu_packed_forward(gate_up)
    assert torch.equal(h, want_h)
    grad = swiglu_packed_backward(dout, saved, gate_up.shape)
    assert grad.data_ptr() == gate_up.data_ptr()
    assert torch.equal(grad[:, :half], want_dg) and torch.equal(grad[:, half:], want_du)
    assert torch.equal(full[0], first_row)


def test_long_flat_streams_as_one_ragged_row():
    """Contiguous tensors that cannot share an alignment are one long ragged row: the forward with inputs skewed
    against its output, the backward with its two outputs skewed against each other.  2^28 + 5 elements (over two
    million warp tasks in a single row), against the aligned result of the same data."""
    n = (1 << 28) + 5
    g = torch.Generator(device=DEVICE).manual_seed(8)
    base = [torch.randn(n + 16, generator=g, device=DEVICE).bfloat16() for _ in range(3)]
    aligned = [b[:n].clone() for b in base]
    want_h = swiglu_forward(aligned[0], aligned[1], 0.9, 1.1)[0]
    want_dg, want_du = swiglu_backward(aligned[2], aligned[0], aligned[1], 0.9, 1.1, preserve_inputs=True)
    stream = torch.cuda.current_stream().cuda_stream
    code = CODE[torch.bfloat16]
    # forward: gate 1 element off, up 3 elements off, output aligned
    gate, up, dout = base[0][1:1 + n], base[1][3:3 + n], base[2][5:5 + n]
    gate.copy_(aligned[0]), up.copy_(aligned[1]), dout.copy_(aligned[2])
    out = torch.empty(n, dtype=torch.bfloat16, device=DEVICE)
    assert _lib.lib.swiglu_b200_plan_fwd(out.data_ptr(), gate.data_ptr(), up.data_ptr(), 1, n, n, n, code) & 0x800
    _lib.check("fwd", _lib.lib.swiglu_b200_fwd(out.data_ptr(), gate.data_ptr(), up.data_ptr(), 1, n, n, n, code, 0.9, 1.1,
                                               0, stream))
    assert torch.equal(out, want_h)
    del out, want_h
    # backward: dgate aligned, dup 2 elements off, every input at its own offset
    grads = torch.full((2 * n + 64,), SENTINEL, dtype=torch.bfloat16, device=DEVICE)
    dg, du = grads[8:8 + n], grads[n + 26:2 * n + 26]
    assert (dg.data_ptr() - du.data_ptr()) % 16 != 0
    assert _lib.lib.swiglu_b200_plan_bwd(dg.data_ptr(), du.data_ptr(), dout.data_ptr(), gate.data_ptr(), up.data_ptr(),
                                         1, n, n, n, n, code) & 0x800
    _lib.check("bwd", _lib.lib.swiglu_b200_bwd(dg.data_ptr(), du.data_ptr(), dout.data_ptr(), gate.data_ptr(),
                                               up.data_ptr(), 1, n, n, n, n, code, 0.9, 1.1, 0, stream))
    assert torch.equal(dg, want_dg) and torch.equal(du, want_du)
    assert bool((grads[:8] == SENTINEL).all()) and bool((grads[8 + n:n + 26] == SENTINEL).all())
    assert bool((grads[2 * n + 26:] == SENTINEL).all())


@pytest.mark.parametrize("approximate", ["tanh", "none"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_geglu_sibling_on_ragged_rows(approximate, dtype):
    """The GeGLU operator shares the ragged-row kernels (the activation is a template argument): packed layout,
    odd half-width, misaligned base, in place and out of place, against its own separate-layout result."""
    from kernels.geglu import geglu_backward, geglu_forward, geglu_packed_backward, geglu_packed_forward

    rows, half, offset = 41, 1001, 3
    g = torch.Generator(device=DEVICE).manual_seed(17)
    gate0, up0, dout = (1.5 * torch.randn(rows, half, generator=g, device=DEVICE).to(dtype) for _ in range(3))
    want_h = geglu_forward(gate0.clone(), up0.clone(), approximate)[0]
    want_dg, want_du = geglu_backward(dout, gate0.clone(), up0.clone(), approximate, preserve_inputs=True)
    for preserve in (True, False):
        src = Pitched(rows, 2 * half, 2 * half, offset, dtype, torch.cat([gate0, up0], dim=1))
        h, saved = geglu_packed_forward(src.view, approximate)
        assert torch.equal(h, want_h)
        grad = geglu_packed_backward(dout, saved, src.view.shape, approximate, preserve_inputs=preserve)
        assert torch.equal(grad[:, :half], want_dg) and torch.equal(grad[:, half:], want_du)
        assert src.untouched()

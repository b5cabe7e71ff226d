"""The C-ABI library loads without a GPU and exports every symbol include/swiglu_b200.h
declares; argument checks that need no device return the documented codes."""
import ctypes
import re
from pathlib import Path

import pytest

from kernel_pocs_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "swiglu_b200.h"


def _declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(swiglu_b200_\w+)\s*\(", text)))


def _codes():
    text = HEADER.read_text()
    return {name: int(val) for name, val in re.findall(r"#define\s+SWIGLU_B200_(\w+)\s+(\d+)", text)}


def test_every_declared_symbol_is_exported():
    names = _declared_symbols()
    assert {"swiglu_b200_fwd", "swiglu_b200_bwd", "swiglu_b200_version", "swiglu_b200_strerror"} <= set(names)
    raw = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in names:
        assert hasattr(raw, name), f"{name} declared in the header but not exported"
    # and the Python binding covers the whole header
    assert set(_lib.SIGNATURES) == set(names)


def test_version_and_error_strings():
    assert _lib.lib.swiglu_b200_version() // 1000 == 1
    codes = _codes()
    assert codes["OK"] == 0 and codes["F32"] == _lib.F32 and codes["F16"] == _lib.F16 and codes["BF16"] == _lib.BF16
    seen = set()
    for name, val in codes.items():
        if name.startswith("ERR_") or name == "OK":
            text = _lib.lib.swiglu_b200_strerror(val).decode()
            assert text and "unknown" not in text
            seen.add(text)
    assert len(seen) == sum(1 for n in codes if n.startswith("ERR_")) + 1
    assert "unknown" in _lib.lib.swiglu_b200_strerror(999).decode()


def test_argument_errors_need_no_device():
    c = _codes()
    f, b = _lib.lib.swiglu_b200_fwd, _lib.lib.swiglu_b200_bwd
    p = 0x1000  # never dereferenced: every call below returns before any CUDA call
    assert f(p, p + 0x10000, p + 0x20000, 4, 8, 8, 8, 7, 1.0, 1.0, -1, None) == c["ERR_DTYPE"]
    assert f(p, p + 0x10000, p + 0x20000, -1, 8, 8, 8, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_SHAPE"]
    assert f(p, p + 0x10000, p + 0x20000, 4, 8, 4, 8, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_SHAPE"]
    assert f(None, p, p + 0x10000, 4, 8, 8, 8, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_NULL"]
    assert f(p + 2, p + 0x10000, p + 0x20000, 4, 8, 8, 8, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_ALIGN"]
    assert f(p + 1, p + 0x10000, p + 0x20000, 4, 8, 8, 8, _lib.BF16, 1.0, 1.0, -1, None) == c["ERR_ALIGN"]
    assert f(p, p, p + 0x20000, 4, 8, 8, 8, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_ALIAS"]  # out over gate
    # empty problems succeed without touching the device, whatever the pointers
    assert f(None, None, None, 0, 8, 8, 8, _lib.F32, 1.0, 1.0, -1, None) == 0
    assert f(None, None, None, 5, 0, 0, 0, _lib.BF16, 1.0, 1.0, -1, None) == 0
    assert b(None, None, None, None, None, 0, 8, 8, 8, 8, _lib.F16, 1.0, 1.0, -1, None) == 0

    g, u, d, dg, du = p, p + 0x10000, p + 0x20000, p + 0x30000, p + 0x40000
    assert b(dg, du, d, g, u, 4, 8, 8, 8, 8, 9, 1.0, 1.0, -1, None) == c["ERR_DTYPE"]
    assert b(dg, du, d, g, u, 4, 8, 8, 8, 7, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_SHAPE"]
    assert b(dg, du, None, g, u, 4, 8, 8, 8, 8, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_NULL"]
    assert b(g, du, d, g, u, 4, 8, 8, 8, 8, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_ALIAS"]  # only one aliased
    assert b(g, u, d, g, u, 4, 8, 8, 16, 8, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_ALIAS"]  # aliased, other pitch
    assert b(g + 16, du, d, g, u, 4, 8, 8, 8, 8, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_ALIAS"]  # partial overlap
    assert b(dg, du, dg, g, u, 4, 8, 8, 8, 8, _lib.F32, 1.0, 1.0, -1, None) == c["ERR_ALIAS"]  # dgate over dout


def test_recompute_and_tensor_core_entries_argument_errors_need_no_device():
    """swiglu_b200_bwd_recompute and the GEMM / LoRA entries reject bad arguments before any CUDA call."""
    c = _codes()
    r = _lib.lib.swiglu_b200_bwd_recompute
    p = 0x1000
    h, dg, du, d, g, u = (p + i * 0x10000 for i in range(6))
    assert r(h, dg, du, d, g, u, 64, 5, 1.0, 1.0, -1, None) == c["ERR_DTYPE"]
    assert r(h, dg, du, d, g, u, -1, _lib.BF16, 1.0, 1.0, -1, None) == c["ERR_SHAPE"]
    assert r(None, None, None, None, None, None, 0, _lib.BF16, 1.0, 1.0, -1, None) == 0
    assert r(h, dg, None, d, g, u, 64, _lib.BF16, 1.0, 1.0, -1, None) == c["ERR_NULL"]
    assert r(h + 1, dg, du, d, g, u, 64, _lib.BF16, 1.0, 1.0, -1, None) == c["ERR_ALIGN"]
    assert r(h, h, du, d, g, u, 64, _lib.BF16, 1.0, 1.0, -1, None) == c["ERR_ALIAS"]       # two outputs, one buffer
    assert r(d + 32, dg, du, d, g, u, 64, _lib.BF16, 1.0, 1.0, -1, None) == c["ERR_ALIAS"]  # partial overlap

    gf, gb, lo = _lib.lib.swiglu_b200_gemm_fwd, _lib.lib.swiglu_b200_gemm_bwd, _lib.lib.swiglu_b200_lora_swiglu_fwd
    st = p + 0x70000
    assert gf(h, None, None, d, g, u, -1, 128, 64, 1.0, 1.0, st, -1, None) == c["ERR_SHAPE"]
    assert gf(h, None, None, d, g, u, 128, 120, 64, 1.0, 1.0, st, -1, None) == c["ERR_SHAPE"]   # n % 16
    assert gf(h, None, None, d, g, u, 128, 128, 60, 1.0, 1.0, st, -1, None) == c["ERR_SHAPE"]   # k % 8
    assert gf(None, None, None, d, g, u, 128, 128, 64, 1.0, 1.0, st, -1, None) == c["ERR_NULL"]
    assert gf(h, dg, None, d, g, u, 128, 128, 64, 1.0, 1.0, st, -1, None) == c["ERR_NULL"]      # gate_out without up_out
    assert gf(h + 8, None, None, d, g, u, 128, 128, 64, 1.0, 1.0, st, -1, None) == c["ERR_ALIGN"]
    assert gf(None, None, None, None, None, None, 0, 128, 64, 1.0, 1.0, None, -1, None) == 0
    assert gb(h, dg, du, d, g, u, p + 0x80000, p + 0x90000, 128, 128, 72, st, -1, None) == c["ERR_SHAPE"]  # k % 16
    assert gb(h, dg, None, d, g, u, p + 0x80000, p + 0x90000, 128, 128, 64, st, -1, None) == c["ERR_NULL"]
    assert gb(h, None, None, d, g, None, None, None, 128, 128, 64, st, -1, None) == c["ERR_NULL"]  # dx needs weights
    assert lo(h, None, None, d, g, u, u, dg, du, 128, 64, 12, 1.0, 1.0, st, -1, None) == c["ERR_SHAPE"]   # rank % 8
    assert lo(h, None, None, d, g, u, u, dg, du, 128, 64, 72, 1.0, 1.0, st, -1, None) == c["ERR_SHAPE"]   # rank > 64
    assert lo(h, dg, None, d, g, u, u, dg, du, 128, 64, 16, 1.0, 1.0, st, -1, None) == c["ERR_NULL"]
    assert lo(h, None, None, d, g, u, u, dg, du, 128, 64, 16, 1.0, 1.0, None, -1, None) == c["ERR_NULL"]
    assert lo(None, None, None, None, None, None, None, None, None, 0, 64, 16, 1.0, 1.0, None, -1, None) == 0


def test_host_entry_argument_errors_need_no_device():
    c = _codes()
    f = _lib.lib.swiglu_b200_host_fwd_bwd
    p = 0x1000
    args = (p, p, p, p, p, p)
    assert f(*args, 4, 8, 5, 1.0, 1.0, 0x100000, 1 << 20, -1, None) == c["ERR_DTYPE"]
    assert f(*args, -4, 8, _lib.F32, 1.0, 1.0, 0x100000, 1 << 20, -1, None) == c["ERR_SHAPE"]
    assert f(*args, 0, 8, _lib.F32, 1.0, 1.0, None, 0, -1, None) == 0
    assert f(None, p, p, p, p, p, 4, 8, _lib.F32, 1.0, 1.0, 0x100000, 1 << 20, -1, None) == c["ERR_NULL"]
    assert f(*args, 4, 8, _lib.F32, 1.0, 1.0, None, 1 << 20, -1, None) == c["ERR_NULL"]
    assert f(*args, 4, 8, _lib.F32, 1.0, 1.0, 0x100010, 1 << 20, -1, None) == c["ERR_ALIGN"]
    assert f(*args, 4, 1 << 20, _lib.F32, 1.0, 1.0, 0x100000, 1 << 20, -1, None) == c["ERR_WORKSPACE"]
    w = _lib.lib.swiglu_b200_host_workspace_bytes
    assert w(0, 8, _lib.BF16) == 0
    assert w(32768, 14336, _lib.BF16) == 12 * ((32 << 20) // (14336 * 2)) * 14336 * 2  # 12 buffers of <= 32 MiB
    assert w(3, 8, _lib.F32) == 12 * 256  # never more than the problem, rounded to the buffer alignment


def test_launch_counter_is_exported_and_idle():
    before = _lib.launch_count()
    _lib.lib.swiglu_b200_fwd(None, None, None, 0, 8, 8, 8, _lib.F32, 1.0, 1.0, -1, None)
    assert _lib.launch_count() == before


def test_check_raises_with_code():
    with pytest.raises(_lib.SwigluB200Error, match="unsupported dtype") as info:
        _lib.check("here", 1)
    assert info.value.code == 1


def _plan(v):
    return {"bytes": v & 0xff, "rows": bool(v & 0x100), "shift": bool(v & 0x200), "head": (v >> 16) & 0xff,
            "edge": (v >> 24) & 0xff}


RAGGED = 0x800  # bit 11: 16-byte accesses with per-row alignment (skewed loads, realigned second store)


def test_access_planning_without_a_device():
    """Which access width, addressing and edge handling a call would get, from its addresses alone."""
    f, b = _lib.lib.swiglu_b200_plan_fwd, _lib.lib.swiglu_b200_plan_bwd
    A = 0x7f0000000000  # a 16-byte aligned "allocation"; nothing is dereferenced
    G, U, O, D = A, A + (1 << 32), A + (2 << 32), A + (3 << 32)
    BF, F32 = _lib.BF16, _lib.F32
    # the benchmark shape: flat, 16-byte vectors, no edges
    assert _plan(f(O, G, U, 32768, 14336, 14336, 14336, BF)) == dict(bytes=16, rows=False, shift=False, head=0, edge=0)
    # odd width, aligned bases: still flat 16-byte vectors; 3 * 11009 = 33027 = 8 * 4128 + 3 tail elements
    assert _plan(f(O, G, U, 3, 11009, 11009, 11009, BF)) == dict(bytes=16, rows=False, shift=False, head=0, edge=3)
    # every tensor 2 bytes past a boundary: 7 head elements, then vectors
    p = _plan(f(O + 2, G + 2, U + 2, 1, 1000, 1000, 1000, BF))
    assert (p["bytes"], p["shift"], p["head"]) == (16, False, 7) and p["edge"] == 7 + (1000 - 7) % 8
    # forward, inputs skewed against an aligned output: one long ragged row (window loads)
    for code in (f(O, G + 2, U + 6, 4, 4096, 4096, 4096, BF), f(O, G + 4, U, 4, 4096, 4096, 4096, F32),
                 f(O, G + 2, U + 2, 4, 4096, 4096, 4096, BF)):
        assert code & RAGGED and _plan(code) == dict(bytes=16, rows=False, shift=False, head=0, edge=0)
    assert not f(O, G, U, 4, 4096, 4096, 4096, BF) & (RAGGED | 0x600)     # aligned: plain vectors
    # backward: the shuffled-load kernel; its one-word variant (bit 10) when no input is more than 4 bytes off
    assert b(G, U, D + 2, G, U, 16, 512, 512, 512, 512, BF) & 0x400 and not b(G, U, D + 10, G, U, 16, 512, 512, 512, 512, BF) & 0x400
    # packed gate|up: pitched rows; a half-width that is a multiple of 16 bytes keeps plain 16-byte vectors ...
    code = f(O, G, G + 2 * 5504, 8, 5504, 11008, 5504, BF)
    assert _plan(code) == dict(bytes=16, rows=True, shift=False, head=0, edge=0) and not code & RAGGED
    # ... any other takes the ragged-row kernel: still 16-byte accesses, alignment worked out row by row
    for code in (f(O, G, G + 2 * 257, 3, 257, 514, 257, BF), f(O, G, G + 4 * 257, 3, 257, 514, 257, F32),
                 f(O, G, G + 2 * 260, 3, 260, 520, 260, BF), f(O + 6, G + 2, G + 2 + 2 * 5503, 9, 5503, 11006, 5503, BF),
                 b(G, G + 2 * 5503, D, G, G + 2 * 5503, 9, 5503, 11006, 11006, 5503, BF),
                 b(O, O + 2 * 1001, D + 4, G, G + 2 * 1001, 9, 1001, 2002, 2002, 1001, BF)):
        assert code & RAGGED and _plan(code) == dict(bytes=16, rows=True, shift=False, head=0, edge=0)
    # a single row is flat whatever its stride says
    assert not _plan(f(O, G, U, 1, 100, 4000, 100, BF))["rows"]
    # backward in place: outputs are gate/up; dh skewed against them -> skewed loads for dh only
    assert _plan(b(G, U, D + 10, G, U, 16, 512, 512, 512, 512, BF)) == dict(bytes=16, rows=False, shift=True, head=0, edge=0)
    # backward out of place with everything congruent
    assert _plan(b(O, O + (1 << 30), D, G, U, 16, 512, 512, 512, 512, BF)) == dict(bytes=16, rows=False, shift=False, head=0, edge=0)
    # outputs skewed against each other: one long ragged row, the second output realigned on the way out
    code = b(O, O + (1 << 30) + 4, D, G, U, 16, 512, 512, 512, 512, BF)
    assert code & RAGGED and _plan(code) == dict(bytes=16, rows=False, shift=False, head=0, edge=0)
    assert not b(O, O + (1 << 30), D, G, U, 16, 512, 512, 512, 512, BF) & RAGGED
    # argument errors come back negated
    c = _codes()
    assert f(O, G, U, 4, 8, 4, 8, BF) == -c["ERR_SHAPE"]
    assert f(O + 1, G, U, 4, 8, 8, 8, BF) == -c["ERR_ALIGN"]
    assert b(G, U, D, G, U, 4, 8, 8, 8, 8, 11) == -c["ERR_DTYPE"]

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

"""Host-side mirror of the reference operator interface: names, argument checks and their
messages (reference tests/test_swiglu.py:134-145), and the absence of a CPU path."""
import importlib
import inspect

import numpy as np
import pytest
import torch

import kernels.swiglu as dropin
from oracle import oracle as O
from tests._util import DTYPES, assert_ulp

host = importlib.import_module("kernel_pocs_b200.swiglu")  # the module, not the function of that name

PUBLIC = [
    "ForgeSwiGLUFunction", "ForgePackedSwiGLUFunction", "swiglu", "swiglu_backward", "swiglu_forward",
    "swiglu_packed", "swiglu_packed_backward", "swiglu_packed_forward", "torch_swiglu_packed_reference",
    "torch_swiglu_reference",
]


def test_drop_in_import_path_exports_the_reference_names():
    assert sorted(dropin.__all__) == sorted(PUBLIC)
    for name in PUBLIC:
        assert getattr(dropin, name) is getattr(host, name)


def test_call_signatures_match_the_reference():
    def params(fn):
        return [(p.name, p.default) for p in inspect.signature(fn).parameters.values()]

    E = inspect.Parameter.empty
    assert params(host.swiglu) == [
        ("gate", E), ("up", E), ("gate_multiplier", 1.0), ("down_multiplier", 1.0), ("preserve_inputs", False)]
    assert params(host.swiglu_packed) == [
        ("gate_up", E), ("gate_multiplier", 1.0), ("down_multiplier", 1.0), ("preserve_inputs", False)]
    assert params(host.swiglu_forward) == [("gate", E), ("up", E), ("gate_multiplier", 1.0), ("down_multiplier", 1.0)]
    assert params(host.swiglu_backward) == [
        ("dout", E), ("gate", E), ("up", E), ("gate_multiplier", 1.0), ("down_multiplier", 1.0),
        ("preserve_inputs", False)]
    assert params(host.swiglu_packed_forward) == [("gate_up", E), ("gate_multiplier", 1.0), ("down_multiplier", 1.0)]
    assert params(host.swiglu_packed_backward) == [
        ("dout", E), ("gate_up", E), ("input_shape", E), ("gate_multiplier", 1.0), ("down_multiplier", 1.0),
        ("preserve_inputs", False)]
    assert params(host.ForgeSwiGLUFunction.forward)[1:] == [
        ("gate", E), ("up", E), ("gate_multiplier", 1.0), ("down_multiplier", 1.0), ("preserve_inputs", False)]
    assert params(host.ForgePackedSwiGLUFunction.forward)[1:] == [
        ("gate_up", E), ("gate_multiplier", 1.0), ("down_multiplier", 1.0), ("preserve_inputs", False)]


def test_swiglu_rejects_invalid_inputs():
    gate = torch.randn(2, 3)
    up = torch.randn(2, 4)
    with pytest.raises(ValueError, match="same shape"):
        dropin.swiglu(gate, up)

    gate_up = torch.randn(2, 5)
    with pytest.raises(ValueError, match="even"):
        dropin.swiglu_packed(gate_up)

    with pytest.raises(TypeError, match="Python scalar"):
        dropin.swiglu(torch.randn(2, 3), torch.randn(2, 3), gate_multiplier=torch.tensor(1.0))
    with pytest.raises(TypeError, match="real Python scalar"):
        dropin.swiglu(torch.randn(2, 3), torch.randn(2, 3), down_multiplier="2")
    with pytest.raises(TypeError, match="same dtype"):
        dropin.swiglu(torch.randn(2, 3), torch.randn(2, 3).half())
    with pytest.raises(TypeError, match="floating point"):
        dropin.swiglu(torch.ones(2, 3, dtype=torch.int32), torch.ones(2, 3, dtype=torch.int32))
    with pytest.raises(TypeError, match="floating point"):
        dropin.swiglu_packed(torch.ones(2, 4, dtype=torch.int64))
    with pytest.raises(TypeError, match="fp16, bf16, and fp32"):
        dropin.swiglu_forward(torch.randn(2, 3, dtype=torch.float64), torch.randn(2, 3, dtype=torch.float64))


def test_no_cpu_fallback():
    """The reference evaluates its PyTorch composite for host tensors (swiglu.py:396-397); this
    implementation has CUDA kernels only and says so instead of computing on the CPU."""
    gate, up = torch.randn(2, 3, 17), torch.randn(2, 3, 17)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        dropin.swiglu(gate, up)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        dropin.swiglu_packed(torch.randn(2, 3, 18))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        dropin.swiglu_forward(gate, up)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        dropin.swiglu_backward(torch.randn(2, 3, 17), gate, up)


def test_public_torch_reference_agrees_with_the_reference_vectors(golden_dir):
    """torch_swiglu_reference is part of the public surface (the reference's tests compare the
    kernels with it); it must reproduce the reference's own outputs."""
    z = np.load(golden_dir / "separate.npz")
    for key in sorted({k.rsplit("|", 1)[0] for k in z.files}):
        dname, _, gm, dm = key.split("|")
        dtype = DTYPES[dname]
        gate, up, want = (O.from_numpy_bits(z[f"{key}|{n}"], dtype) for n in ("gate", "up", "h"))
        got = host.torch_swiglu_reference(gate, up, float(gm), float(dm))
        assert got.dtype == dtype and got.shape == gate.shape
        assert_ulp(got, want, 0, f"torch_swiglu_reference {key}")
    z = np.load(golden_dir / "packed.npz")
    for key in sorted({k.rsplit("|", 1)[0] for k in z.files}):
        dname, _, gm, dm = key.split("|")
        dtype = DTYPES[dname]
        gate_up, want = (O.from_numpy_bits(z[f"{key}|{n}"], dtype) for n in ("gate_up", "h"))
        got = host.torch_swiglu_packed_reference(gate_up, float(gm), float(dm))
        assert_ulp(got, want, 0, f"torch_swiglu_packed_reference {key}")

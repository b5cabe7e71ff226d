"""Writes tests/golden/*.npz by running the REFERENCE ITSELF on the host.

    python tests/golden/make_golden.py --reference /path/to/kernel-POCs

Imports ``kernels.swiglu`` from a checkout of Forge-researchlab/kernel-POCs and calls its own
``swiglu`` / ``swiglu_packed`` on CPU tensors (for which it evaluates torch_swiglu_reference,
kernels/swiglu/swiglu.py:396-397, with the backward by autograd).  Shapes, seeds, draw order
and multipliers follow the reference's tests/test_swiglu.py:28-113; the extra cases are the
benchmark configuration "fp32 [2,128,1024], seed 0" and wide-tailed N(0, 2^2) inputs.

lora_mlp.npz comes from the reference's own ground truth for its LoRA-MLP kernels,
kernels/lora_mlp/reference/lora_mlp_pytorch.py (``matmul_lora``, ``lora_swiglu_mlp`` and the autograd Function
``LoRAMLP``, the comparators of kernels/lora_mlp/tests/test_lora_mlp.py), run on CPU in fp32 and bf16.

The reference checkout is needed only to regenerate the vectors; the tests read the .npz
files.  Arrays hold raw storage: float32, or uint16 bit patterns for fp16/bf16.
"""
from __future__ import annotations

import argparse
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def bits(x: torch.Tensor) -> np.ndarray:
    x = x.detach().contiguous()
    if x.dtype == torch.float32:
        return x.numpy().copy()
    return x.view(torch.int16).numpy().view(np.uint16).copy()


def run_separate(ref, gate, up, dout, gm, dm):
    g = gate.detach().clone().requires_grad_(True)
    u = up.detach().clone().requires_grad_(True)
    h = ref.swiglu(g, u, gm, dm)
    h.backward(dout)
    return h.detach(), g.grad, u.grad


def run_packed(ref, gate_up, dout, gm, dm):
    gu = gate_up.detach().clone().requires_grad_(True)
    h = ref.swiglu_packed(gu, gm, dm)
    h.backward(dout)
    return h.detach(), gu.grad


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of Forge-researchlab/kernel-POCs")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import kernels.swiglu as ref  # the reference package, not this repository's drop-in

    assert Path(ref.__file__).resolve().is_relative_to(Path(args.reference).resolve()), ref.__file__
    torch.set_num_threads(1)

    # --- separate layout: reference tests/test_swiglu.py:28-65 (smaller last shape) ----------
    out = {}
    for dname, dtype in DTYPES.items():
        for shape in [(2, 8, 128), (1, 3, 257), (3, 5, 200)]:
            for gm, dm in [(1.0, 1.0), (0.7, 1.3)]:
                torch.manual_seed(0)
                gate = torch.randn(*shape, dtype=dtype)
                up = torch.randn(*shape, dtype=dtype)
                dout = torch.randn(*shape, dtype=dtype)  # randn_like(out_ref) in the reference test
                h, dgate, dup = run_separate(ref, gate, up, dout, gm, dm)
                key = f"{dname}|{'x'.join(map(str, shape))}|{gm}|{dm}"
                for name, t in dict(gate=gate, up=up, dout=dout, h=h, dgate=dgate, dup=dup).items():
                    out[f"{key}|{name}"] = bits(t)
    np.savez_compressed(HERE / "separate.npz", **out)

    # --- packed layout: reference tests/test_swiglu.py:68-99 ----------------------------------
    out = {}
    for dname, dtype in DTYPES.items():
        for shape in [(2, 8, 256), (1, 3, 514)]:
            for gm, dm in [(1.0, 1.0), (1.5, 0.5)]:
                torch.manual_seed(1)
                gate_up = torch.randn(*shape, dtype=dtype)
                dout = torch.randn(*shape[:-1], shape[-1] // 2, dtype=dtype)
                h, dgate_up = run_packed(ref, gate_up, dout, gm, dm)
                key = f"{dname}|{'x'.join(map(str, shape))}|{gm}|{dm}"
                for name, t in dict(gate_up=gate_up, dout=dout, h=h, dgate_up=dgate_up).items():
                    out[f"{key}|{name}"] = bits(t)
    np.savez_compressed(HERE / "packed.npz", **out)

    # --- special values: reference tests/test_swiglu.py:102-113, in all three dtypes ---------
    out = {}
    inf, nan = float("inf"), float("nan")
    for dname, dtype in DTYPES.items():
        gate = torch.tensor([[[0.0, inf, -inf, nan, 20.0, -20.0, 88.0, -88.0, 1e-30, -0.0]]], dtype=dtype)
        up = torch.tensor([[[1.0, 2.0, 3.0, 4.0, -1.0, -2.0, 0.5, 0.5, 1.0, 1.0]]], dtype=dtype)
        h = ref.swiglu(gate, up)
        out[f"{dname}|gate"], out[f"{dname}|up"], out[f"{dname}|h"] = bits(gate), bits(up), bits(h)
    np.savez_compressed(HERE / "special.npz", **out)

    # --- wide tails: N(0, 2^2) inputs, odd width, as in the var-len benchmark configuration --
    out = {}
    for dname, dtype in DTYPES.items():
        g = torch.Generator().manual_seed(2)
        shape = (7, 1101)
        gate = (2.0 * torch.randn(*shape, generator=g)).to(dtype)
        up = (2.0 * torch.randn(*shape, generator=g)).to(dtype)
        dout = (2.0 * torch.randn(*shape, generator=g)).to(dtype)
        h, dgate, dup = run_separate(ref, gate, up, dout, 1.0, 1.0)
        for name, t in dict(gate=gate, up=up, dout=dout, h=h, dgate=dgate, dup=dup).items():
            out[f"{dname}|{name}"] = bits(t)
    np.savez_compressed(HERE / "tails.npz", **out)

    # --- benchmark configuration 1: fp32 [2,128,1024], seed 0, draw order gate, up, dh --------
    torch.manual_seed(0)
    gate = torch.randn(2, 128, 1024)
    up = torch.randn(2, 128, 1024)
    dout = torch.randn(2, 128, 1024)
    h, dgate, dup = run_separate(ref, gate, up, dout, 1.0, 1.0)
    rows = np.array([0, 37, 255])
    out = {
        "rows": rows,
        "inputs_sha256": np.frombuffer(
            hashlib.sha256(bits(gate).tobytes() + bits(up).tobytes() + bits(dout).tobytes()).digest(), dtype=np.uint8
        ),
    }
    for name, t in dict(gate=gate, up=up, dout=dout, h=h, dgate=dgate, dup=dup).items():
        flat = t.reshape(256, 1024)
        out[f"{name}_rows"] = bits(flat[rows])
        out[f"{name}_sum"] = np.array(flat.double().sum().item())
        out[f"{name}_meanabs"] = np.array(flat.double().abs().mean().item())
    np.savez_compressed(HERE / "config1.npz", **out)

    # --- GeGLU sibling: reference tests/test_geglu.py:32-103 (shapes reduced), both GELU forms -----------
    import kernels.geglu as ref_geglu

    assert Path(ref_geglu.__file__).resolve().is_relative_to(Path(args.reference).resolve())
    out = {}
    for dname, dtype in DTYPES.items():
        for approximate in ("tanh", "none"):
            for shape in [(2, 8, 128), (1, 3, 257)]:
                torch.manual_seed(0)
                gate = (1.5 * torch.randn(*shape)).to(dtype)
                up = torch.randn(*shape, dtype=dtype)
                dout = torch.randn(*shape, dtype=dtype)
                g = gate.detach().clone().requires_grad_(True)
                u = up.detach().clone().requires_grad_(True)
                h = ref_geglu.geglu(g, u, approximate)
                h.backward(dout)
                key = f"{dname}|{'x'.join(map(str, shape))}|{approximate}"
                for name, t in dict(gate=gate, up=up, dout=dout, h=h.detach(), dgate=g.grad, dup=u.grad).items():
                    out[f"{key}|{name}"] = bits(t)
            torch.manual_seed(1)
            gate_up = torch.randn(1, 3, 514, dtype=dtype)
            dout = torch.randn(1, 3, 257, dtype=dtype)
            gu = gate_up.detach().clone().requires_grad_(True)
            h = ref_geglu.geglu_packed(gu, approximate)
            h.backward(dout)
            key = f"{dname}|packed|{approximate}"
            for name, t in dict(gate_up=gate_up, dout=dout, h=h.detach(), dgate_up=gu.grad).items():
                out[f"{key}|{name}"] = bits(t)
    np.savez_compressed(HERE / "geglu.npz", **out)

    # --- LoRA MLP: the reference's PyTorch ground truth (kernels/lora_mlp/reference/lora_mlp_pytorch.py) ------
    sys.path.insert(0, str(Path(args.reference) / "kernels" / "lora_mlp"))
    from reference import lora_mlp_pytorch as ref_lora  # as kernels/lora_mlp/tests/test_lora_mlp.py:21 imports it

    assert Path(ref_lora.__file__).resolve().is_relative_to(Path(args.reference).resolve())
    out = {}
    for dname, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        for b, s_, hidden, inter, rank in [(2, 32, 128, 256, 8), (1, 50, 64, 144, 16)]:
            g = torch.Generator().manual_seed(42)
            mk = lambda *shape, std: (std * torch.randn(*shape, generator=g)).to(dtype)
            p = {}
            for name, (o, i) in dict(gate=(inter, hidden), up=(inter, hidden), down=(hidden, inter)).items():
                p[f"W_{name}"] = mk(o, i, std=i ** -0.5)
                p[f"A_{name}"] = mk(rank, i, std=i ** -0.5).requires_grad_(True)
                p[f"B_{name}"] = mk(o, rank, std=0.3).requires_grad_(True)
                p[f"s_{name}"] = 2.0
            X = mk(b, s_, hidden, std=1.0).requires_grad_(True)
            dY = mk(b, s_, hidden, std=1.0)
            y = ref_lora.LoRAMLP.apply(
                X, p["W_gate"], p["A_gate"], p["B_gate"], p["s_gate"], p["W_up"], p["A_up"], p["B_up"], p["s_up"],
                p["W_down"], p["A_down"], p["B_down"], p["s_down"])
            y.backward(dY)
            with torch.no_grad():
                e = ref_lora.matmul_lora(X, p["W_gate"], p["A_gate"], p["B_gate"], p["s_gate"])
                gg = ref_lora.matmul_lora(X, p["W_up"], p["A_up"], p["B_up"], p["s_up"])
                h = torch.nn.functional.silu(e) * gg
                y_fn = ref_lora.lora_swiglu_mlp(X, **p)
                e0 = ref_lora.matmul_lora(X, p["W_gate"], None, None, 1.0)
                g0 = ref_lora.matmul_lora(X, p["W_up"], None, None, 1.0)
                h0 = torch.nn.functional.silu(e0) * g0
                y0 = ref_lora.lora_swiglu_mlp(X, p["W_gate"], None, None, 1.0, p["W_up"], None, None, 1.0,
                                              p["W_down"], None, None, 1.0)
            key = f"{dname}|{b}x{s_}x{hidden}x{inter}x{rank}"
            tensors = dict(X=X, dY=dY, out=y, out_functional=y_fn, e=e, g=gg, h=h, dX=X.grad,
                           e_noadapter=e0, g_noadapter=g0, h_noadapter=h0, out_noadapter=y0)
            for name in ("gate", "up", "down"):
                tensors[f"W_{name}"] = p[f"W_{name}"]
                tensors[f"A_{name}"], tensors[f"dA_{name}"] = p[f"A_{name}"], p[f"A_{name}"].grad
                tensors[f"B_{name}"], tensors[f"dB_{name}"] = p[f"B_{name}"], p[f"B_{name}"].grad
            for name, t in tensors.items():
                out[f"{key}|{name}"] = bits(t)
    np.savez_compressed(HERE / "lora_mlp.npz", **out)

    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()

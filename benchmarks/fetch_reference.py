"""Places the reference's own SwiGLU and GeGLU modules where the benchmark and the comparison tests look for them.

    python benchmarks/fetch_reference.py --reference /path/to/kernel-POCs

Copies ``kernels/swiglu/{__init__,swiglu}.py``, ``kernels/geglu/{__init__,geglu}.py`` and
``kernels/lora_mlp/experiments/{v2/lora_mlp_kernel_v2,v3/lora_mlp_kernel_v3}.py`` of a checkout of Forge-researchlab/kernel-POCs,
unmodified, to ``baseline/_ref/kernels/`` under this repository.  That directory is
git-ignored: the copies are comparators that are timed beside this library (benchmarks/bench_all.py providers
``ref-triton-fast``, ``ref-triton-safe``, ``ref-triton-packed``, ``ref-triton-geglu-tanh``, ``ref-triton-geglu-erf``,
``ref-triton-lora-epilogue`` of the ``lora`` section and ``ref-triton-dual-gemm`` of the ``c4`` section;
bench.py --impl reference; tests/test_reference_triton.py), never product source, and nothing under
kernel_pocs_b200/ imports them.  Without the copies those providers report ``unavailable`` and the tests skip.

``load()`` imports a copied module under a private name, so that it can live in one process with this
repository's drop-in package of the same import path (``kernels.swiglu``, ``kernels.geglu``).
"""
from __future__ import annotations

import argparse
import importlib.util
import shutil
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
DEST_ROOT = ROOT / "baseline" / "_ref" / "kernels"
DEST = DEST_ROOT / "swiglu"
# name -> (directory under kernels/, files copied, the file that load() imports)
OPERATORS = {
    "swiglu": ("swiglu", ("__init__.py", "swiglu.py"), "swiglu.py"),
    "geglu": ("geglu", ("__init__.py", "geglu.py"), "geglu.py"),
    "lora_v3": ("lora_mlp/experiments/v3", ("lora_mlp_kernel_v3.py",), "lora_mlp_kernel_v3.py"),
    "lora_v2": ("lora_mlp/experiments/v2", ("lora_mlp_kernel_v2.py",), "lora_mlp_kernel_v2.py"),
}
# The two lora_mlp experiment files import names of a vendored third-party baseline at module level, for their
# full-MLP classes; fused_lora_swiglu (v3) and fused_gate_up_swiglu (v2), the functions compared here, use none of
# them.  The baseline is not copied: load() puts an empty stand-in module under that import path instead.
_BASELINE_NAMES = {"reference": (), "reference.unsloth_baseline": ("swiglu_DWf_DW_dfg_kernel", "matmul_lora")}
_STAND_INS = {"lora_v3": _BASELINE_NAMES, "lora_v2": _BASELINE_NAMES}


def fetch(reference: Path) -> Path:
    """Copies the operators' modules; the SwiGLU one must be there, the others are taken when they are."""
    for op, (rel, files, _) in OPERATORS.items():
        src = Path(reference) / "kernels" / rel
        missing = [f for f in files if not (src / f).is_file()]
        if missing:
            if op == "swiglu":
                raise FileNotFoundError(f"{src} lacks {missing}: not a kernel-POCs checkout")
            continue
        (DEST_ROOT / rel).mkdir(parents=True, exist_ok=True)
        for f in files:
            shutil.copyfile(src / f, DEST_ROOT / rel / f)
    return DEST


def _module_path(op: str) -> Path:
    rel, _, module_file = OPERATORS[op]
    return DEST_ROOT / rel / module_file


def available(op: str = "swiglu") -> bool:
    return _module_path(op).is_file()


def load(op: str = "swiglu"):
    """One of the reference's modules (they import triton at module level) under a private name.
    Raises FileNotFoundError when the copy is absent."""
    name = f"_kernel_pocs_reference_{op}"
    if name in sys.modules:
        return sys.modules[name]
    path = _module_path(op)
    if not path.is_file():
        raise FileNotFoundError(f"{path} is absent; run benchmarks/fetch_reference.py --reference <checkout>")
    added = []
    for mod_name, names in _STAND_INS.get(op, {}).items():
        if mod_name not in sys.modules:
            import types

            stand_in = types.ModuleType(mod_name)
            for n in names:
                setattr(stand_in, n, None)
            sys.modules[mod_name] = stand_in
            added.append(mod_name)
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    try:
        spec.loader.exec_module(module)
    except BaseException:
        sys.modules.pop(name, None)
        raise
    finally:
        for mod_name in added:
            sys.modules.pop(mod_name, None)
    return module


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--reference", required=True, help="checkout of Forge-researchlab/kernel-POCs")
    args = ap.parse_args()
    print(fetch(Path(args.reference)))


if __name__ == "__main__":
    main()

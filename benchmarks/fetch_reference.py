"""Places the reference's own SwiGLU and GeGLU modules where the benchmark and the comparison tests look for them.

    python benchmarks/fetch_reference.py --reference /path/to/kernel-POCs

Copies ``kernels/swiglu/{__init__,swiglu}.py`` and ``kernels/geglu/{__init__,geglu}.py`` of a checkout of
Forge-researchlab/kernel-POCs, unmodified, to ``baseline/_ref/kernels/`` under this repository.  That directory is
git-ignored: the copies are comparators that are timed beside this library (benchmarks/bench_all.py providers
``ref-triton-fast``, ``ref-triton-safe``, ``ref-triton-packed``, ``ref-triton-geglu-tanh``, ``ref-triton-geglu-erf``;
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
OPERATORS = {"swiglu": ("__init__.py", "swiglu.py"), "geglu": ("__init__.py", "geglu.py")}


def fetch(reference: Path) -> Path:
    """Copies both operators' modules; the SwiGLU one must be there, the GeGLU one is taken when it is."""
    for op, files in OPERATORS.items():
        src = Path(reference) / "kernels" / op
        missing = [f for f in files if not (src / f).is_file()]
        if missing:
            if op == "swiglu":
                raise FileNotFoundError(f"{src} lacks {missing}: not a kernel-POCs checkout")
            continue
        (DEST_ROOT / op).mkdir(parents=True, exist_ok=True)
        for f in files:
            shutil.copyfile(src / f, DEST_ROOT / op / f)
    return DEST


def available(op: str = "swiglu") -> bool:
    return (DEST_ROOT / op / f"{op}.py").is_file()


def load(op: str = "swiglu"):
    """The reference's ``kernels/<op>/<op>.py`` as a module (it imports triton at module level).
    Raises FileNotFoundError when the copy is absent."""
    name = f"_kernel_pocs_reference_{op}"
    if name in sys.modules:
        return sys.modules[name]
    path = DEST_ROOT / op / f"{op}.py"
    if not path.is_file():
        raise FileNotFoundError(f"{path} is absent; run benchmarks/fetch_reference.py --reference <checkout>")
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    try:
        spec.loader.exec_module(module)
    except BaseException:
        sys.modules.pop(name, None)
        raise
    return module


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--reference", required=True, help="checkout of Forge-researchlab/kernel-POCs")
    args = ap.parse_args()
    print(fetch(Path(args.reference)))


if __name__ == "__main__":
    main()

"""Places the reference's own SwiGLU module where the benchmark and the comparison test look for it.

    python benchmarks/fetch_reference.py --reference /path/to/kernel-POCs

Copies ``kernels/swiglu/__init__.py`` and ``kernels/swiglu/swiglu.py`` of a checkout of
Forge-researchlab/kernel-POCs, unmodified, to ``baseline/_ref/kernels/swiglu/`` under this
repository.  That directory is git-ignored: the copy is a comparator that is timed beside this
library (benchmarks/bench_all.py providers ``ref-triton-fast``, ``ref-triton-safe``,
``ref-triton-packed``; bench.py --impl reference; tests/test_reference_triton.py), never product
source, and nothing under kernel_pocs_b200/ imports it.  Without the copy those providers report
``unavailable`` and the test skips.

``load()`` imports the copied module under a private name, so that it can live in one process
with this repository's drop-in package of the same import path (``kernels.swiglu``).
"""
from __future__ import annotations

import argparse
import importlib.util
import shutil
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
DEST = ROOT / "baseline" / "_ref" / "kernels" / "swiglu"
FILES = ("__init__.py", "swiglu.py")
_MODULE_NAME = "_kernel_pocs_reference_swiglu"


def fetch(reference: Path) -> Path:
    src = Path(reference) / "kernels" / "swiglu"
    missing = [f for f in FILES if not (src / f).is_file()]
    if missing:
        raise FileNotFoundError(f"{src} lacks {missing}: not a kernel-POCs checkout")
    DEST.mkdir(parents=True, exist_ok=True)
    for f in FILES:
        shutil.copyfile(src / f, DEST / f)
    return DEST


def available() -> bool:
    return (DEST / "swiglu.py").is_file()


def load():
    """The reference's ``kernels/swiglu/swiglu.py`` as a module (it imports triton at module level).
    Raises FileNotFoundError when the copy is absent."""
    if _MODULE_NAME in sys.modules:
        return sys.modules[_MODULE_NAME]
    path = DEST / "swiglu.py"
    if not path.is_file():
        raise FileNotFoundError(f"{path} is absent; run benchmarks/fetch_reference.py --reference <checkout>")
    spec = importlib.util.spec_from_file_location(_MODULE_NAME, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[_MODULE_NAME] = module
    try:
        spec.loader.exec_module(module)
    except BaseException:
        sys.modules.pop(_MODULE_NAME, None)
        raise
    return module


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--reference", required=True, help="checkout of Forge-researchlab/kernel-POCs")
    args = ap.parse_args()
    print(fetch(Path(args.reference)))


if __name__ == "__main__":
    main()

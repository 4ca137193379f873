"""Stage the reference itself for use as a checker and as the timed CPU baseline.

    python oracle/make_ref.py [/path/to/llm-quant]

(default: $LLM_QUANT_REFERENCE, else a checkout named `reference` beside this repository)

The reference is pure Python, so "building" it means placing its package where the tests and
the benchmark's reference arm can import it: `oracle/_ref/llmquant`, plus its `examples/`
scripts under `oracle/_ref/examples`. `oracle/_ref/` is listed in .gitignore -- nothing of the
reference enters this repository's history -- but it travels with the working tree to the GPU
machine, where the reference checkout itself does not exist. TEST INFRASTRUCTURE ONLY: no
module of llmquant_b200 imports it.
"""

import pathlib
import shutil
import sys

import os

HERE = pathlib.Path(__file__).resolve().parent
DEST = HERE / "_ref"


def default_checkout() -> pathlib.Path:
    """Where the reference is looked for when no path is given."""
    return pathlib.Path(os.environ.get("LLM_QUANT_REFERENCE") or HERE.parent.parent / "reference")


def stage(ref_root=None) -> pathlib.Path:
    src = pathlib.Path(ref_root) if ref_root else default_checkout()
    if not (src / "llmquant" / "__init__.py").exists():
        raise FileNotFoundError(f"{src} does not hold an llm-quant checkout")
    DEST.mkdir(exist_ok=True)
    for name in ("llmquant", "examples"):
        target = DEST / name
        if target.exists():
            shutil.rmtree(target)
        shutil.copytree(src / name, target, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return DEST


def available() -> bool:
    return (DEST / "llmquant" / "__init__.py").exists()


def import_reference():
    """Import the staged reference package as `llmquant` (raises if it was never staged)."""
    if not available():
        raise ImportError("the reference is not staged: run `python oracle/make_ref.py <llm-quant checkout>`")
    if str(DEST) not in sys.path:
        sys.path.insert(0, str(DEST))
    import llmquant

    return llmquant


if __name__ == "__main__":
    print(stage(sys.argv[1] if len(sys.argv) > 1 else None))

"""Offline build of libllmquant_b200.so: nvcc straight to sm_100a, no JIT, no torch headers.

    python -m llmquant_b200.build            # rebuild what changed
    python -m llmquant_b200.build --force
    LQ_NVCC_EXTRA=-DLQ_DIAGNOSTICS python -m llmquant_b200.build --out /tmp/libdiag.so

The library carries only `extern "C"` entry points (include/llmquant_b200.h), so it needs
nothing but the CUDA runtime, which is linked statically.
"""

import concurrent.futures
import os
import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG.parent / "build" / "obj"
LIB = PKG / "libllmquant_b200.so"

# no --use_fast_math: division and rounding must stay IEEE for bit-exact codes and scales
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the kernels are built offline with the CUDA toolkit")
    return found


def sources():
    return sorted(CSRC.glob("*.cu"))


def _stale(target: pathlib.Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _extra_flags():
    """Extra nvcc flags from LQ_NVCC_EXTRA (e.g. -DLQ_DIAGNOSTICS for a build with the per-CTA
    timeline stamps and the tuning overrides compiled in)."""
    return os.environ.get("LQ_NVCC_EXTRA", "").split()


def _compile(src: pathlib.Path, force: bool, verbose: bool, obj_dir: pathlib.Path = OBJ):
    obj = obj_dir / (src.stem + ".o")
    headers = list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "llmquant_b200.h"]
    if not force and not _stale(obj, [src, *headers]):
        return obj, ""
    cmd = [nvcc(), *NVCC_FLAGS, *_extra_flags(), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{done.stdout}\n{done.stderr}")
    return obj, done.stderr


def build(force: bool = False, verbose: bool = False, out: pathlib.Path = LIB) -> pathlib.Path:
    """Build the library at `out` (default: beside the package, where it is loaded from). A
    build somewhere else -- e.g. a diagnostic one, loaded through LLMQUANT_B200_LIBRARY --
    keeps its objects in a directory of its own."""
    out = pathlib.Path(out)
    obj_dir = OBJ if out == LIB else OBJ.parent / ("obj_" + out.stem)
    obj_dir.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        results = list(pool.map(lambda s: _compile(s, force, verbose, obj_dir), srcs))
    objs = [r[0] for r in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if force or _stale(out, objs):
        cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(out), *map(str, objs)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode:
            raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return out


if __name__ == "__main__":
    target = LIB
    if "--out" in sys.argv:
        target = pathlib.Path(sys.argv[sys.argv.index("--out") + 1]).resolve()
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, out=target))

"""Offline build of libllmquant_b200.so: nvcc straight to sm_100a, no JIT, no torch headers.

    python -m llmquant_b200.build            # rebuild what changed
    python -m llmquant_b200.build --force

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


def _compile(src: pathlib.Path, force: bool, verbose: bool):
    obj = OBJ / (src.stem + ".o")
    headers = list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "llmquant_b200.h"]
    if not force and not _stale(obj, [src, *headers]):
        return obj, ""
    cmd = [nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{done.stdout}\n{done.stderr}")
    return obj, done.stderr


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        results = list(pool.map(lambda s: _compile(s, force, verbose), srcs))
    objs = [r[0] for r in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if force or _stale(LIB, objs):
        cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(LIB), *map(str, objs)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode:
            raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

"""In-tree build of the native libraries.

``build_all()`` compiles every ``csrc/*.cu`` for ``sm_100a`` with ``nvcc``, twice: with bf16 elements into
``lib/libfbam_kernels.so`` and with ``-DFBAM_ELEM_FP16`` (IEEE half elements) into ``lib/libfbam_kernels_fp16.so``; ``csrc/runtime/*.cpp`` (host-only runtime: tokenizer trie, SplitMix64,
safetensors, durable cursor writer, TCP rendezvous, membership master) goes into
``lib/libfbam_runtime.so`` with ``g++``.  Objects are rebuilt only when their source (or a header)
is newer.  Run as ``python -m fbamtrain_b200.build``.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(LIB, "obj")
KERNELS_SO = os.path.join(LIB, "libfbam_kernels.so")
KERNELS_FP16_SO = os.path.join(LIB, "libfbam_kernels_fp16.so")
RUNTIME_SO = os.path.join(LIB, "libfbam_runtime.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _feature_flags() -> list:
    """Optional code paths that are compiled in on request (use with --force, then rebuild without to go back):
    ``FBAMTRAIN_RS_ROW_STORES=1`` — the row-store variant of the GEMM -> reduce-scatter epilogue."""
    flags = []
    if os.environ.get("FBAMTRAIN_RS_ROW_STORES", "0") == "1":
        flags.append("-DFBAM_RS_ROW_STORES=1")
    return flags


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newest(paths: List[str]) -> float:
    return max((os.path.getmtime(p) for p in paths), default=0.0)


def _compile(cmd: List[str], log_path: str) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(log_path, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    hdr_time = _newest(headers)
    nvcc = _nvcc()
    jobs, relinked = [], False
    variants = ((KERNELS_SO, "", []), (KERNELS_FP16_SO, "_fp16", ["-DFBAM_ELEM_FP16"]))
    objs_of = {}
    for so, suffix, defs in variants:
        objs_of[so] = []
        for src in sources:
            obj = os.path.join(OBJ, os.path.basename(src)[:-3] + suffix + ".o")
            objs_of[so].append(obj)
            if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time):
                jobs.append(([nvcc] + NVCC_FLAGS + _feature_flags() + defs + ["-I", CSRC, "-c", src, "-o", obj],
                             obj + ".log"))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(os.cpu_count() or 8, len(jobs))) as ex:
            list(ex.map(lambda j: _compile(*j), jobs))
    for so, suffix, _ in variants:
        objs = objs_of[so]
        if jobs or not os.path.exists(so) or os.path.getmtime(so) < _newest(objs):
            _compile([nvcc, "-shared", "-o", so] + objs + ["-lcudart"], os.path.join(OBJ, f"link_kernels{suffix}.log"))
    if verbose:
        for _, log in jobs:
            sys.stdout.write(open(log).read())
    return KERNELS_SO


SANITIZE_FLAGS = ["-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer"]


def sanitizer_preload() -> str:
    """``LD_PRELOAD`` value for running Python with the sanitised runtime library (the sanitizer runtime must come
    first, and libstdc++ has to be loaded with it for its C++ exception interceptor)."""
    cxx = shutil.which("g++") or "g++"
    libs = [subprocess.run([cxx, f"-print-file-name={n}"], capture_output=True, text=True).stdout.strip()
            for n in ("libasan.so", "libstdc++.so")]
    return " ".join(libs)


def build_runtime(force: bool = False, sanitize: bool = False) -> str:
    """``sanitize``: AddressSanitizer + UndefinedBehaviorSanitizer build of the host runtime (``--sanitize`` on the
    command line; forces a rebuild — rebuild without it afterwards).  Run the CPU tests of the native runtime with
    ``LD_PRELOAD="$(python -c 'from fbamtrain_b200.build import sanitizer_preload as p; print(p())')"
    ASAN_OPTIONS=detect_leaks=0 python -m pytest tests/test_native_runtime.py tests/test_properties.py``."""
    if sanitize:
        os.makedirs(OBJ, exist_ok=True)
        sources = sorted(glob.glob(os.path.join(CSRC, "runtime", "*.cpp")))
        cxx = shutil.which("g++") or "g++"
        flags = [f for f in CXX_FLAGS if f != "-O2"] + SANITIZE_FLAGS
        _compile([cxx] + flags + ["-shared", "-o", RUNTIME_SO] + sources, os.path.join(OBJ, "link_runtime.log"))
        return RUNTIME_SO
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "runtime", "*.cpp")))
    if not sources:
        return ""
    headers = glob.glob(os.path.join(CSRC, "runtime", "*.h"))
    if force or not os.path.exists(RUNTIME_SO) or os.path.getmtime(RUNTIME_SO) < _newest(sources + headers):
        cxx = shutil.which("g++") or "g++"
        _compile([cxx] + CXX_FLAGS + ["-shared", "-o", RUNTIME_SO] + sources, os.path.join(OBJ, "link_runtime.log"))
    return RUNTIME_SO


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force, verbose)
    build_runtime(force)


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        print("built (sanitised host runtime):", build_runtime(sanitize=True))
        print("LD_PRELOAD=" + sanitizer_preload())
        sys.exit(0)
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", KERNELS_SO, KERNELS_FP16_SO, RUNTIME_SO if os.path.exists(RUNTIME_SO) else "")

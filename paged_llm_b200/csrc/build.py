"""Builds the CUDA modules of this package for sm_100a with nvcc, in-tree.

A module is a shared library made of a few .cu files; it is compiled the first
time it is asked for and found again by the hash of its sources and flags.
Libraries land in `csrc/_build/` (or, if the package folder cannot be written,
in `$PAGED_LLM_B200_BUILD_DIR` or a per-user folder under the temporary
directory).  No torch headers are involved: the kernels have a C interface and
are called through ctypes, so a fresh checkout compiles in well under a minute.
While it compiles it prints a line now and then to standard error.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]

# extra nvcc flags for experiments (e.g. -DNAME): part of the hash, so such a build never replaces the regular one
NVCC_FLAGS += os.environ.get("PAGED_LLM_B200_NVCC_FLAGS", "").split()

HEAD_DIM_BUILDS = (16, 32, 64, 128, 256)

MODULES: dict[str, list[str]] = {
    "core": ["common.cu", "elementwise.cu", "gemm_f32.cu", "gemm_skinny.cu", "gemm_tc.cu", "attention_f32.cu",
             "sampling.cu"],
    **{f"attn_bf16_d{d}": ["common.cu", f"attention_bf16_d{d}.cu"] for d in HEAD_DIM_BUILDS},
    # decode attention whose scratch is a static array of the library (see attention_decode_static.h)
    "attn_static": ["common.cu", "attention_decode_static.cu"],
}


def say(msg: str) -> None:
    print(f"[paged_llm_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("PAGED_LLM_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError("nvcc not found: the CUDA kernels of paged_llm_b200 have to be compiled (set CUDA_HOME)")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        with tempfile.NamedTemporaryFile(dir=path):
            pass
        return True
    except OSError:
        return False


def build_dir() -> str:
    cands = [os.environ.get("PAGED_LLM_B200_BUILD_DIR"), os.path.join(HERE, "_build"),
             os.path.join(tempfile.gettempdir(), f"paged_llm_b200_build_{os.getuid()}")]
    for c in cands:
        if c and _writable_dir(c):
            return c
    raise RuntimeError(f"no writable folder for compiled kernels among {cands}")


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def module_hash(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in MODULES[name] + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def library_path(name: str, folder: str | None = None) -> str:
    return os.path.join(folder or build_dir(), f"libpl_{name}-{module_hash(name)}.so")


def find_built(name: str) -> str | None:
    """An up-to-date library of this module, in any of the known folders."""
    fname = f"libpl_{name}-{module_hash(name)}.so"
    for folder in (os.environ.get("PAGED_LLM_B200_BUILD_DIR"), os.path.join(HERE, "_build"),
                   os.path.join(tempfile.gettempdir(), f"paged_llm_b200_build_{os.getuid()}")):
        if folder and os.path.isfile(os.path.join(folder, fname)):
            return os.path.join(folder, fname)
    return None


def module_available(name: str) -> bool:
    """Whether all sources of an optional module are there."""
    return name in MODULES and all(os.path.exists(os.path.join(HERE, src)) for src in MODULES[name])


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def build_module(name: str, verbose: bool = True) -> str:
    """Compiles module `name` if no up-to-date library exists; returns its path."""
    if name not in MODULES:
        raise KeyError(f"unknown kernel module {name!r}; known: {sorted(MODULES)}")
    built = find_built(name)
    if built:
        return built
    nvcc = find_nvcc()
    folder = build_dir()
    out = library_path(name, folder)
    t0 = time.time()
    if verbose:
        say(f"compiling module '{name}' ({len(MODULES[name])} files) for sm_100a ...")
    stop = threading.Event()

    def heartbeat():
        while not stop.wait(10.0):
            say(f"  still compiling '{name}' ({time.time() - t0:.0f}s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        hb.start()
    work = tempfile.mkdtemp(prefix=f"pl_{name}_", dir=folder)
    try:
        def compile_one(src: str) -> str:
            obj = os.path.join(work, os.path.splitext(src)[0] + ".o")
            _run([nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj])
            if verbose:
                say(f"  {src} done ({time.time() - t0:.0f}s)")
            return obj

        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(MODULES[name]))) as pool:
            objs = list(pool.map(compile_one, MODULES[name]))
        tmp_out = os.path.join(work, "lib.so")
        _run([nvcc, "--shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp_out, *objs])
        os.replace(tmp_out, out)
        # libraries of this module from older sources are of no use any more
        prefix = f"libpl_{name}-"
        for old in os.listdir(folder):
            if old.startswith(prefix) and old.endswith(".so") and os.path.join(folder, old) != out:
                try:
                    os.remove(os.path.join(folder, old))
                except OSError:
                    pass
    finally:
        stop.set()
        shutil.rmtree(work, ignore_errors=True)
    if verbose:
        say(f"module '{name}' ready in {time.time() - t0:.0f}s: {out}")
    return out


def build_all(verbose: bool = True) -> dict[str, str]:
    return {name: build_module(name, verbose) for name in MODULES if module_available(name)}


if __name__ == "__main__":
    for n, path in build_all().items():
        print(n, path)

"""Compile the CUDA sources beside this file into one shared library for sm_100a.

The library is built in-tree (``csrc/_build/``) by calling ``nvcc`` directly: one object
per ``.cu`` file, compiled in parallel, then linked.  A stamp holds a hash of the sources
and flags, so a checkout whose library is current loads it at once and a fresh checkout
compiles at its first call, printing a line as each file finishes.  If the source tree is
not writable the build goes to a per-user folder under the system's temporary directory.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

CSRC = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libnhv_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]


def _say(msg: str) -> None:
    print(f"[nanohybrid_vlm_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NHV_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError("nvcc not found: set CUDA_HOME or put nvcc on PATH; the engine's kernels must be compiled "
                       "for sm_100a and there is no fallback without them")


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def source_hash() -> str:
    h = hashlib.sha256()
    for name in sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h"))):
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("NHV_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    in_tree = os.path.join(CSRC, "_build")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"nhv_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise RuntimeError(f"no writable folder for the compiled kernels (tried {in_tree} and {fallback})")


def _current(bdir: str, digest: str) -> bool:
    stamp = os.path.join(bdir, LIB_NAME + ".hash")
    lib = os.path.join(bdir, LIB_NAME)
    if not (os.path.isfile(stamp) and os.path.isfile(lib)):
        return False
    with open(stamp) as f:
        return f.read().strip() == digest


def _compile_one(nvcc: str, src: str, obj: str) -> tuple[str, float]:
    t0 = time.time()
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return src, time.time() - t0


def ensure_built(verbose: bool = True) -> str:
    """Return the path of a current library, compiling it first if needed."""
    digest = source_hash()
    # A library that travelled with the tree is used even if the tree is read-only.
    in_tree = os.path.join(CSRC, "_build")
    if _current(in_tree, digest):
        return os.path.join(in_tree, LIB_NAME)
    bdir = build_dir()
    if _current(bdir, digest):
        return os.path.join(bdir, LIB_NAME)
    with open(os.path.join(bdir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if _current(bdir, digest):  # another process built it while we waited
            return os.path.join(bdir, LIB_NAME)
        nvcc = find_nvcc()
        srcs = sources()
        if verbose:
            _say(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} (first call only)")
        t0 = time.time()
        objs = [os.path.join(bdir, s[:-3] + ".o") for s in srcs]
        workers = max(1, min(len(srcs), os.cpu_count() or 1))
        with concurrent.futures.ThreadPoolExecutor(workers) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o) for s, o in zip(srcs, objs)]
            pending = set(futs)
            while pending:
                done, pending = concurrent.futures.wait(pending, timeout=10)
                for f in done:
                    src, dt = f.result()
                    if verbose:
                        _say(f"  compiled {src} in {dt:.0f} s")
                if pending and not done and verbose:
                    _say(f"  still compiling, {len(pending)} files to go ({time.time() - t0:.0f} s)")
        tmp_lib = os.path.join(bdir, f".{LIB_NAME}.{os.getpid()}")
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_lib, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking the kernels failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        os.replace(tmp_lib, os.path.join(bdir, LIB_NAME))
        with open(os.path.join(bdir, LIB_NAME + ".hash"), "w") as f:
            f.write(digest)
        if verbose:
            _say(f"kernels ready after {time.time() - t0:.0f} s")
    return os.path.join(bdir, LIB_NAME)


def ensure_variant(source: str, defines: dict, verbose: bool = True, folder: str = "variants") -> str:
    """Compile one file of ``csrc/variants/`` with the given -D values into a library of its own
    (for kernels whose sizes are compile-time constants: a model compiles only what it needs).
    ``folder=""`` takes a file of ``csrc/`` itself (tests build a kernel with other constants that way)."""
    src = os.path.join(CSRC, folder, source)
    tag = "_".join(f"{k.lower()}{v}" for k, v in sorted(defines.items()))
    name = f"libnhv_{os.path.splitext(source)[0]}_{tag}.so"
    h = hashlib.sha256()
    headers = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    for path in (src, *headers):
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode() + repr(sorted(defines.items())).encode())
    digest = h.hexdigest()

    def current(bdir):
        stamp, lib = os.path.join(bdir, name + ".hash"), os.path.join(bdir, name)
        if not (os.path.isfile(stamp) and os.path.isfile(lib)):
            return False
        with open(stamp) as f:
            return f.read().strip() == digest

    in_tree = os.path.join(CSRC, "_build")
    if current(in_tree):
        return os.path.join(in_tree, name)
    bdir = build_dir()
    if current(bdir):
        return os.path.join(bdir, name)
    with open(os.path.join(bdir, f".lock_{name}"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if current(bdir):
            return os.path.join(bdir, name)
        nvcc = find_nvcc()
        if verbose:
            _say(f"compiling {source} for {defines} (first call only)")
        t0 = time.time()
        tmp = os.path.join(bdir, f".{name}.{os.getpid()}")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, *[f"-D{k}={v}" for k, v in sorted(defines.items())],
               "-shared", "-o", tmp, src]
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        while True:
            try:
                out, _ = proc.communicate(timeout=10)
                break
            except subprocess.TimeoutExpired:
                if verbose:
                    _say(f"  still compiling {source} ({time.time() - t0:.0f} s)")
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {source}:\n{' '.join(cmd)}\n{out}")
        os.replace(tmp, os.path.join(bdir, name))
        with open(os.path.join(bdir, name + ".hash"), "w") as f:
            f.write(digest)
        if verbose:
            _say(f"  compiled {source} {defines} in {time.time() - t0:.0f} s")
    return os.path.join(bdir, name)


if __name__ == "__main__":
    print(ensure_built())

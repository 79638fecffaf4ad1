"""In-tree build of the native libraries.

Two shared objects are produced next to the sources and loaded through ``ctypes``:

* ``areno_b200/lib/libareno_kernels.so`` -- every CUDA kernel, compiled by ``nvcc`` for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a``).  nvcc cross-compiles, so
  this works on a machine without a GPU.
* ``areno_b200/lib/libareno_runtime.so`` -- the host-side C++ runtime (paged-KV block
  allocator, continuous-batching scheduler, batch packer).

A content hash of the sources is stored beside each library; ``ensure_built`` is a no-op
when the hash matches, so a prebuilt tree never recompiles at import time.

Run ``python -m areno_b200.build`` to build explicitly (``--force`` to rebuild,
``--verbose`` to print ptxas register/shared-memory usage).
"""

from __future__ import annotations

import contextlib
import fcntl
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = LIB / "obj"

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=default",
]


def _sources(suffixes: tuple[str, ...], subdir: str = "") -> list[Path]:
    base = CSRC / subdir if subdir else CSRC
    if not base.is_dir():
        return []
    return sorted(p for p in base.iterdir() if p.suffix in suffixes and p.is_file())


def _hash(files: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def _run(cmd: list[str], verbose: bool) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build command failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout + proc.stderr)


@contextlib.contextmanager
def _build_lock():
    """Serialise builds across processes (several ranks may import the package at once): the first
    one in builds, the others wait and then find the stamp up to date."""
    LIB.mkdir(parents=True, exist_ok=True)
    with open(LIB / ".build.lock", "w") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def _link(cmd_prefix: list[str], out: Path, verbose: bool) -> None:
    """Link into a temporary name and rename: a concurrent loader never sees a half-written library."""
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    _run([*cmd_prefix[:1], *cmd_prefix[1:], "-o", str(tmp)], verbose)
    os.replace(tmp, out)


def kernels_lib_path() -> Path:
    return LIB / "libareno_kernels.so"


def runtime_lib_path() -> Path:
    return LIB / "libareno_runtime.so"


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libareno_kernels.so``."""
    out = kernels_lib_path()
    cu = _sources((".cu",))
    headers = _sources((".cuh", ".h"))
    digest = _hash(cu + headers, " ".join(NVCC_FLAGS))
    stamp = LIB / "libareno_kernels.stamp"
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    if not os.path.exists(NVCC):
        raise RuntimeError(
            f"nvcc not found at {NVCC}: cannot build {out.name}.  Install the CUDA toolkit (12.8 or newer: the kernels "
            "are compiled for sm_100a) or point CUDA_HOME at it; no GPU is needed to compile.  `areno check` lists what "
            "else the machine is missing.")
    with _build_lock():
        if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
            return out   # another process built it while we waited
        return _build_kernels_locked(out, cu, headers, digest, stamp, force, verbose)


def _build_kernels_locked(out, cu, headers, digest, stamp, force, verbose) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    header_digest = _hash(headers, " ".join(NVCC_FLAGS))

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        ostamp = OBJ / (src.stem + ".stamp")
        d = hashlib.sha256((header_digest + src.read_text()).encode()).hexdigest()
        if not force and obj.exists() and ostamp.exists() and ostamp.read_text() == d:
            return obj
        flags = list(NVCC_FLAGS)
        if verbose:
            flags += ["-Xptxas", "-v"]
        _run([NVCC, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], verbose)
        ostamp.write_text(d)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as pool:
        objs = list(pool.map(compile_one, cu))
    _link([NVCC, "-shared", *map(str, objs), "-lcudart"], out, verbose)
    stamp.write_text(digest)
    return out


def build_runtime(force: bool = False, verbose: bool = False) -> Path:
    """Compile the host-side C++ runtime (``csrc/runtime/*.cpp``)."""
    out = runtime_lib_path()
    srcs = _sources((".cpp",), "runtime")
    headers = _sources((".h", ".hpp"), "runtime")
    if not srcs:
        return out
    digest = _hash(srcs + headers, "runtime-v1")
    stamp = LIB / "libareno_runtime.stamp"
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    with _build_lock():
        if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
            return out
        cxx = os.environ.get("CXX", "g++")
        _link([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", *map(str, srcs)], out, verbose)
        stamp.write_text(digest)
    return out


def ensure_built(verbose: bool = False) -> None:
    build_kernels(verbose=verbose)
    build_runtime(verbose=verbose)


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    force = "--force" in argv
    verbose = "--verbose" in argv
    k = build_kernels(force=force, verbose=verbose)
    r = build_runtime(force=force, verbose=verbose)
    print(f"built {k}")
    print(f"built {r}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

"""Offline install of the unmodified reference package into ``baseline/_ref``.

``bench.py --impl reference`` imports the reference from that directory and from nowhere else.  The
directory is not tracked (it holds a compiled extension), so it has to be produced on the machine
that builds this tree: ``__graft_entry__.build()`` calls ``ensure_installed()``, and the reference arm
calls it once more as a fallback when the directory is missing at run time.

The install is ``pip install --no-index --no-build-isolation --no-deps --target baseline/_ref`` from a
scratch copy of the reference source (the build writes into its source tree, which may be read-only).
``--no-deps`` because dependency resolution is the only step that fails without an index: the
reference's requirements (torch, flash-attn, ...) are already importable in the image.  The
extension is built for compute capability 10.0 (``TORCH_CUDA_ARCH_LIST``), which works without a GPU.

Nothing of ``areno_b200`` is imported here or by the installed package.
"""

from __future__ import annotations

import fcntl
import os
import shutil
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
_LOG = os.path.join(ROOT, "baseline", "_ref_install.log")


def source_dir() -> str:
    """Where the reference source tree lives: ``ARENO_REFERENCE_SRC`` or a ``reference`` folder beside the repo."""
    return os.environ.get("ARENO_REFERENCE_SRC") or os.path.join(os.path.dirname(ROOT), "reference")


def is_installed() -> bool:
    pkg = os.path.join(REF, "areno")
    accel = os.path.join(pkg, "accel")
    if not os.path.isfile(os.path.join(pkg, "__init__.py")) or not os.path.isdir(accel):
        return False
    return any(f.startswith("_areno_accel") and f.endswith(".so") for f in os.listdir(accel))


def ensure_installed(verbose: bool = False) -> tuple[bool, str]:
    """Install the reference if it is not there yet.  Returns ``(ok, one-line reason)``; never raises."""
    if is_installed():
        return True, "already installed"
    src = source_dir()
    if not os.path.isdir(src):
        return False, f"reference source tree not found at {src} (set ARENO_REFERENCE_SRC)"
    os.makedirs(os.path.dirname(REF), exist_ok=True)
    try:
        with open(os.path.join(ROOT, "baseline", ".install.lock"), "w") as lock:
            fcntl.flock(lock, fcntl.LOCK_EX)      # several ranks may get here at once: one installs, the rest wait
            try:
                if is_installed():
                    return True, "already installed"
                return _install(src, verbose)
            finally:
                fcntl.flock(lock, fcntl.LOCK_UN)
    except Exception as exc:  # a missing reference must never break the build or the bench
        return False, f"install raised {type(exc).__name__}: {str(exc)[:200]}"


def _install(src: str, verbose: bool) -> tuple[bool, str]:
    scratch = tempfile.mkdtemp(prefix="areno_ref_src_")
    try:
        copy = os.path.join(scratch, "src")
        shutil.copytree(src, copy, symlinks=True, ignore=shutil.ignore_patterns(".git", "__pycache__", "*.pyc"))
        env = dict(os.environ)
        env.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
        env.setdefault("MAX_JOBS", str(min(16, os.cpu_count() or 4)))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--target", REF, "--upgrade"]
        wheelhouse = os.environ.get("ARENO_WHEELHOUSE", "/opt/wheelhouse")
        if os.path.isdir(wheelhouse):
            cmd += ["--find-links", wheelhouse]
        cmd.append(copy)
        proc = subprocess.run(cmd, env=env, capture_output=True, text=True,
                              timeout=float(os.environ.get("ARENO_REF_INSTALL_TIMEOUT_S", 1500)))
        with open(_LOG, "w") as f:
            f.write(" ".join(cmd) + "\n" + proc.stdout[-20000:] + "\n" + proc.stderr[-20000:])
        if verbose:
            print(proc.stdout[-2000:], proc.stderr[-2000:], file=sys.stderr)
        if proc.returncode != 0 or not is_installed():
            tail = (proc.stderr.strip().splitlines() or proc.stdout.strip().splitlines() or ["no output"])[-1]
            return False, f"pip install exited {proc.returncode}: {tail[:200]}"
        return True, "installed"
    except subprocess.TimeoutExpired:
        return False, "pip install of the reference did not finish in time"
    finally:
        shutil.rmtree(scratch, ignore_errors=True)


if __name__ == "__main__":
    ok, why = ensure_installed(verbose=True)
    print(("ok: " if ok else "failed: ") + why)
    raise SystemExit(0 if ok else 1)

"""``areno env`` / ``areno check``: a support report and a readiness check list.

Neither command starts the engine.  ``collect_env`` gathers versions, GPUs, toolchain and the state
of the in-tree native libraries; ``run_checks`` turns the report into PASS / WARN / FAIL rows with a
next step for each problem; ``check`` exits 1 when any row is FAIL.  Counterpart of
``areno/cli/diagnostics.py:36-250`` in the reference, with the checks that matter for this package:
an sm_100 GPU, nvcc >= 12.8 for ``sm_100a``, and the two shared libraries built from ``csrc/``.
"""

from __future__ import annotations

import json
import os
import platform
import shutil
import subprocess
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import click

from ..api.defaults import DEFAULT_METRICS_LOG_DIR

ENV_VARS = ("CUDA_HOME", "CUDA_PATH", "CUDA_VISIBLE_DEVICES", "NCCL_DEBUG", "NCCL_NVLS_ENABLE", "ARENO_LOG_LEVEL",
            "ARENO_CKPT_RESERVE_GB", "HF_HOME", "HF_HUB_CACHE")
MIN_NVCC = (12, 8)


@dataclass(frozen=True)
class CheckResult:
    status: str  # PASS | WARN | FAIL
    name: str
    detail: str = ""
    next_step: str = ""


def _package_version(name: str) -> str | None:
    from importlib import metadata

    try:
        return metadata.version(name)
    except metadata.PackageNotFoundError:
        return None


def _torch_info() -> dict[str, Any]:
    try:
        import torch
    except Exception as exc:  # pragma: no cover - torch is a hard dependency
        return {"imported": False, "error": f"{type(exc).__name__}: {exc}", "gpus": []}
    info: dict[str, Any] = {"imported": True, "version": torch.__version__, "cuda_build": torch.version.cuda,
                            "cuda_available": bool(torch.cuda.is_available()), "gpus": []}
    try:
        info["nccl"] = ".".join(str(v) for v in torch.cuda.nccl.version()) if torch.version.cuda else None
    except Exception:
        info["nccl"] = None
    if info["cuda_available"]:
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            info["gpus"].append({"index": i, "name": p.name, "capability": f"{p.major}.{p.minor}",
                                 "memory_gb": round(p.total_memory / 2**30, 1), "sm_count": p.multi_processor_count})
    return info


def _run(cmd: list[str]) -> str | None:
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=20, check=False)
    except (OSError, subprocess.SubprocessError):
        return None
    return out.stdout if out.returncode == 0 else None


def _nvcc_info(path: str | None) -> dict[str, str | None]:
    if not path:
        return {"path": None, "version": None}
    text = _run([path, "--version"]) or ""
    version = None
    for token in text.replace(",", " ").split():
        if token.startswith("V") and token[1:2].isdigit():
            version = token[1:]
    return {"path": path, "version": version}


def _driver_info() -> dict[str, str | None]:
    exe = shutil.which("nvidia-smi")
    if not exe:
        return {"nvidia_smi": None, "driver_version": None}
    text = _run([exe, "--query-gpu=driver_version", "--format=csv,noheader"])
    first = text.strip().splitlines()[0].strip() if text and text.strip() else None
    return {"nvidia_smi": exe, "driver_version": first}


def _native_libs() -> dict[str, Any]:
    from .. import build

    out = {}
    for label, fn in (("kernels", build.kernels_lib_path), ("runtime", build.runtime_lib_path)):
        path = Path(fn())
        out[label] = {"path": str(path), "built": path.exists(),
                      "size_bytes": path.stat().st_size if path.exists() else None}
    return out


def _version_tuple(text: str | None) -> tuple[int, ...]:
    if not text:
        return ()
    parts = []
    for piece in text.split("."):
        digits = ""
        for ch in piece:            # leading digits only: "8rc1" is 8, not 81
            if not ch.isdigit():
                break
            digits += ch
        if not digits:
            break
        parts.append(int(digits))
        if len(digits) != len(piece):
            break
    return tuple(parts)


def collect_env() -> dict[str, Any]:
    torch_info = _torch_info()
    return {
        "areno_b200": {"version": _package_version("areno_b200") or "source tree"},
        "python": {"version": platform.python_version(), "executable": sys.executable},
        "platform": {"system": platform.system(), "release": platform.release(), "machine": platform.machine()},
        "torch": torch_info,
        "cuda": {"cuda_home": os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH"),
                 "nvcc": _nvcc_info(shutil.which("nvcc")), "driver": _driver_info()},
        "gpus": torch_info.get("gpus", []),
        "native": _native_libs(),
        "dependencies": {name: _package_version(name) for name in
                         ("transformers", "safetensors", "datasets", "fastapi", "uvicorn", "tensorboard", "click")},
        "env": {name: os.environ.get(name) for name in ENV_VARS},
        "paths": {"metrics_log_dir": DEFAULT_METRICS_LOG_DIR,
                  "hf_cache": os.environ.get("HF_HUB_CACHE") or str(Path.home() / ".cache" / "huggingface" / "hub")},
    }


def _row(ok: bool, name: str, detail: str, next_step: str, *, warn: bool = False) -> CheckResult:
    if ok:
        return CheckResult("PASS", name, detail)
    return CheckResult("WARN" if warn else "FAIL", name, detail, next_step)


def _nearest_existing(path: Path) -> Path:
    cur = path
    while not cur.exists() and cur != cur.parent:
        cur = cur.parent
    return cur


def _writable(label: str, path_text: str) -> CheckResult:
    target = Path(path_text).expanduser()
    base = _nearest_existing(target)
    ok = os.access(base, os.W_OK)
    return _row(ok, f"{label} writable", f"{target} (checked {base})",
                f"Choose a writable directory for {label} or fix permissions on {base}.", warn=True)


def run_checks(report: dict[str, Any]) -> list[CheckResult]:
    rows = [_row(sys.version_info >= (3, 10), "Python >= 3.10", report["python"]["version"],
                 "Use a Python 3.10+ interpreter.")]
    t = report["torch"]
    rows.append(_row(bool(t.get("imported")), "PyTorch importable", t.get("version") or t.get("error", ""),
                     "Install a CUDA build of PyTorch."))
    rows.append(_row(bool(t.get("cuda_build")), "PyTorch built with CUDA", str(t.get("cuda_build")),
                     "Install a CUDA build of PyTorch (CPU-only wheels cannot run the kernels)."))
    rows.append(_row(bool(t.get("cuda_available")), "CUDA device visible", f"{len(report['gpus'])} GPU(s)",
                     "Check the driver, CUDA_VISIBLE_DEVICES and container GPU access."))
    gpus = report["gpus"]
    if gpus:
        bad = [g for g in gpus if not g["capability"].startswith("10.")]
        rows.append(_row(not bad, "GPUs are sm_100 (B200 class)", ", ".join(f"{g['name']} sm_{g['capability']}" for g in gpus),
                         "The kernels are compiled for sm_100a only; run on B200 GPUs."))
    rows.append(_row(bool(t.get("nccl")), "NCCL available", str(t.get("nccl")),
                     "Multi-GPU runs need torch built with NCCL.", warn=True))
    nvcc = report["cuda"]["nvcc"]
    native = report["native"]
    all_built = all(v["built"] for v in native.values())
    nvcc_ok = _version_tuple(nvcc["version"])[:2] >= MIN_NVCC if nvcc["version"] else False
    rows.append(_row(nvcc_ok, "nvcc >= 12.8 (sm_100a)", f"{nvcc['path']} {nvcc['version']}",
                     "Install CUDA 12.8+ so the kernels can be rebuilt; prebuilt libraries keep working without it.",
                     warn=all_built))
    for label, v in native.items():
        rows.append(_row(v["built"], f"native {label} library built", v["path"],
                         "Run `python -m areno_b200.build`."))
    drv = report["cuda"]["driver"]
    rows.append(_row(bool(drv["driver_version"]), "NVIDIA driver reported", str(drv["driver_version"]),
                     "nvidia-smi not found or failed; install the NVIDIA driver.", warn=True))
    deps = report["dependencies"]
    for name, hard in (("transformers", True), ("safetensors", True), ("datasets", False), ("fastapi", False),
                       ("uvicorn", False), ("tensorboard", False)):
        rows.append(_row(bool(deps.get(name)), f"{name} installed", str(deps.get(name)),
                         f"pip install {name}", warn=not hard))
    rows.append(_writable("metrics_log_dir", report["paths"]["metrics_log_dir"]))
    rows.append(_writable("hf_cache", report["paths"]["hf_cache"]))
    return rows


def format_env_report(report: dict[str, Any]) -> str:
    lines = ["AReno-B200 environment", ""]
    lines.append(f"package   {report['areno_b200']['version']}")
    lines.append(f"python    {report['python']['version']}  ({report['python']['executable']})")
    lines.append(f"platform  {report['platform']['system']} {report['platform']['release']} {report['platform']['machine']}")
    t = report["torch"]
    lines.append(f"torch     {t.get('version')}  cuda={t.get('cuda_build')}  nccl={t.get('nccl')}  available={t.get('cuda_available')}")
    c = report["cuda"]
    lines.append(f"nvcc      {c['nvcc']['path']}  {c['nvcc']['version']}")
    lines.append(f"driver    {c['driver']['driver_version']}")
    lines.append("")
    lines.append("GPUs")
    for g in report["gpus"]:
        lines.append(f"  [{g['index']}] {g['name']}  sm_{g['capability']}  {g['memory_gb']} GiB  {g['sm_count']} SMs")
    if not report["gpus"]:
        lines.append("  none visible")
    lines.append("")
    lines.append("Native libraries")
    for label, v in report["native"].items():
        lines.append(f"  {label:<8} {'built' if v['built'] else 'MISSING'}  {v['path']}")
    lines.append("")
    lines.append("Dependencies")
    for name, ver in report["dependencies"].items():
        lines.append(f"  {name:<13} {ver or 'not installed'}")
    lines.append("")
    lines.append("Environment")
    for name, value in report["env"].items():
        lines.append(f"  {name}={value if value is not None else ''}")
    return "\n".join(lines)


@click.command(name="env", context_settings={"help_option_names": ["-h", "--help"]})
@click.option("--json", "as_json", is_flag=True, help="Emit a machine-readable JSON report.")
def env_command(as_json: bool) -> None:
    """Print an environment / support report."""
    report = collect_env()
    click.echo(json.dumps(report, indent=2, sort_keys=True) if as_json else format_env_report(report))


@click.command(name="check", context_settings={"help_option_names": ["-h", "--help"]})
def check_command() -> None:
    """Check whether this machine is ready to run the framework."""
    rows = run_checks(collect_env())
    failed = any(r.status == "FAIL" for r in rows)
    click.echo(f"AReno-B200 check: {'not ready' if failed else 'ready'}")
    click.echo()
    for r in rows:
        click.echo(f"{r.status:<4} {r.name}")
        if r.detail:
            click.echo(f"     {r.detail}")
    steps = [r.next_step for r in rows if r.status != "PASS" and r.next_step]
    if steps:
        click.echo()
        click.echo("Next:")
        for s in steps:
            click.echo(f"  {s}")
    if failed:
        raise click.exceptions.Exit(1)

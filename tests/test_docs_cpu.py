"""The written material agrees with the code: every environment switch the package reads is documented, every
profile summary is indexed, flags and files that the guides name exist."""

from __future__ import annotations

import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
GUIDES = sorted((ROOT / "docs").glob("*.md")) + [ROOT / "README.md"]


def _text(paths) -> str:
    return "\n".join(p.read_text(errors="ignore") for p in paths)


def test_every_environment_switch_is_documented():
    sources = [p for p in (ROOT / "areno_b200").rglob("*") if p.suffix in {".py", ".cu", ".cuh", ".h", ".cpp"}]
    sources += [ROOT / "bench.py", ROOT / "bench_extra.py"]
    read = set(re.findall(r"ARENO_[A-Z0-9_]+", _text(sources)))
    documented = set(re.findall(r"ARENO_[A-Z0-9_]+", _text(GUIDES)))
    # constants of the no-allocation entry point's header, not switches
    constants = {n for n in read if n.startswith(("ARENO_NOALLOC_", "ARENO_RMSNORM_BWD_STATIC_"))}
    assert not sorted(read - documented - constants)


def test_every_profile_summary_is_indexed():
    index = (ROOT / "profiles" / "README.md").read_text()
    missing = [p.name for p in (ROOT / "profiles").glob("*.md") if p.name != "README.md" and p.name not in index]
    assert not missing


def test_flags_named_in_the_guides_exist():
    from areno_b200.cli import serve, train

    known = set()
    for flag, _kw, _group in train.OPTIONS:
        known.update(part.strip() for part in flag.split("/"))
    for param in serve.serve_command.params:
        known.update(param.opts)
        known.update(param.secondary_opts)
    # flags of other programs that the guides quote (pytest, torchrun, pip, ncu, the tools and examples of this tree)
    foreign = {"--help", "--json", "--steps", "--warmup", "--gpus", "--impl", "--config", "--no-e2e", "--nnodes", "--nproc-per-node",
               "--master-addr", "--master-port", "--standalone", "--local-addr", "--case", "--iters", "--graph", "--profile-last",
               "--pattern", "--top-k", "--set", "--clock-control", "--metrics", "--csv", "--log-file", "--profile-from-start",
               "--device", "--agentic", "--keep", "--small", "--pid", "--section"}
    named = set(re.findall(r"(?<![\w-])--[a-z][a-z0-9-]+", _text(sorted((ROOT / "docs").glob("*.md")) + [ROOT / "README.md"])))
    assert not sorted(named - known - foreign)


def test_python_files_named_in_the_guides_exist():
    missing = []
    for guide in GUIDES + [ROOT / "CONTRIBUTING.md"]:
        for name in re.findall(r"`((?:areno_b200|tests|examples|ci|baseline|profiles|docs)/[A-Za-z0-9_./-]+\.(?:py|md|cu|cuh|h|cpp))`",
                               guide.read_text()):
            if not (ROOT / name).exists():
                missing.append((guide.name, name))
    assert not missing

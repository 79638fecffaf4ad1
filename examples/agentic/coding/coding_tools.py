"""Workspace tools of the coding agent: every path is resolved inside the task's temporary directory,
commands run there with a short timeout and truncated output, and destructive ``rm`` commands are refused."""

from __future__ import annotations

import os
import re
import shlex
import subprocess
import tempfile

MAX_OUTPUT = 4000


class Workspace:
    def __init__(self, files: dict[str, str]):
        self._tmp = tempfile.TemporaryDirectory(prefix="areno_coding_")
        self.root = self._tmp.name
        for rel, text in files.items():
            path = self._resolve(rel)
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "w") as f:
                f.write(text)

    def close(self) -> None:
        self._tmp.cleanup()

    def _resolve(self, rel: str) -> str:
        path = os.path.realpath(os.path.join(self.root, rel))
        if not (path == os.path.realpath(self.root) or path.startswith(os.path.realpath(self.root) + os.sep)):
            raise ValueError("path escapes the workspace")
        return path

    # ------------------------------------------------------------------ tools
    def list_files(self) -> dict:
        out = []
        for base, _dirs, names in os.walk(self.root):
            for n in sorted(names):
                out.append(os.path.relpath(os.path.join(base, n), self.root))
        return {"files": sorted(out)}

    def read_file(self, path: str, start: int = 1, end: int = 200) -> dict:
        with open(self._resolve(path)) as f:
            lines = f.read().splitlines()
        start, end = max(1, int(start)), min(len(lines), int(end))
        return {"path": path, "lines": [f"{i}: {lines[i - 1]}" for i in range(start, end + 1)]}

    def rg(self, pattern: str) -> dict:
        rx, hits = re.compile(pattern), []
        for rel in self.list_files()["files"]:
            with open(self._resolve(rel), errors="replace") as f:
                for i, line in enumerate(f, 1):
                    if rx.search(line):
                        hits.append(f"{rel}:{i}: {line.rstrip()}")
        return {"matches": hits[:50]}

    def replace_text(self, path: str, old: str, new: str) -> dict:
        full = self._resolve(path)
        with open(full) as f:
            text = f.read()
        if text.count(old) != 1:
            return {"error": f"expected exactly one occurrence, found {text.count(old)}"}
        with open(full, "w") as f:
            f.write(text.replace(old, new))
        return {"ok": True}

    def write_file(self, path: str, content: str) -> dict:
        full = self._resolve(path)
        os.makedirs(os.path.dirname(full), exist_ok=True)
        with open(full, "w") as f:
            f.write(content)
        return {"ok": True, "bytes": len(content)}

    def run_command(self, command: str, timeout_s: float = 20.0) -> dict:
        argv = shlex.split(command)
        if not argv or argv[0] in ("rm", "sudo") or " rm " in f" {command} ":
            return {"error": "command refused"}
        try:
            proc = subprocess.run(argv, cwd=self.root, capture_output=True, text=True, timeout=timeout_s,
                                  env={**os.environ, "PYTHONDONTWRITEBYTECODE": "1"})
        except subprocess.TimeoutExpired:
            return {"error": "timeout"}
        except OSError as exc:
            return {"error": str(exc)}
        return {"returncode": proc.returncode, "output": (proc.stdout + proc.stderr)[-MAX_OUTPUT:]}

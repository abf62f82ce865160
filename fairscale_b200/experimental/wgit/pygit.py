"""Minimal git wrapper for the metadata repository inside ``.wgit`` (parity: .../wgit/pygit.py:14-153).

Drives the ``git`` executable instead of ``pygit2``: the metadata tree is tiny, so process-spawn cost is irrelevant
and no binary dependency is needed.
"""

from __future__ import annotations

from pathlib import Path
import subprocess
from typing import Dict, List, Optional


class PyGit:
    def __init__(self, parent_path: Path, gitignore: Optional[List[str]] = None, name: str = "user", email: str = "user@email.com") -> None:
        self._parent_path = Path(parent_path)
        self.name, self.email = name, email
        if not (self._parent_path / ".git").exists():
            self._git("init", "-q")
            (self._parent_path / ".gitignore").write_text("".join(f"{g}\n" for g in (gitignore or [])))
        self._git("config", "user.name", name)
        self._git("config", "user.email", email)

    def _git(self, *args: str, check: bool = True) -> str:
        r = subprocess.run(["git", *args], cwd=self._parent_path, capture_output=True, text=True)
        if check and r.returncode != 0:
            raise RuntimeError(f"git {' '.join(args)} failed: {r.stderr.strip()}")
        return r.stdout

    @property
    def path(self) -> str:
        return str(self._parent_path / ".git")

    def add(self) -> None:
        self._git("add", "-A")

    def commit(self, message: str) -> None:
        self._git("commit", "-q", "--allow-empty", "-m", message)

    def status(self) -> Dict[str, str]:
        out = self._git("status", "--porcelain")
        return {line[3:]: line[:2] for line in out.splitlines() if line}

    def log(self, file: Optional[str] = None) -> str:
        args = ["log", "--oneline"] + (["--", file] if file else [])
        return self._git(*args, check=False)

    def checkout(self, sha1: str) -> None:
        self._git("checkout", "-q", sha1)

"""The weigit repository: tracks checkpoints in the working directory through small metadata files.

Capability parity with fairscale/experimental/wgit/repo.py:31-472: ``Repo(parent_dir, init=True)`` creates
``.wgit/`` with a SHA1 store and a git repository of metadata; ``add(path, per_tensor=..., sparsify ...)`` stores
a checkpoint (optionally tensor by tensor, optionally as SST / DST of :class:`SignalSparsity`) and writes its
metadata file, ``commit``, ``status``, ``log``, ``checkout``, ``size_info``.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
import json
from pathlib import Path
import sys
from typing import Any, Dict, List, Optional, Union

import torch

from .pygit import PyGit
from .sha1_store import SHA1_Store
from .signal_sparsity import SignalSparsity
from .utils import ExitCode

SHA1_KEY, LAST_MODIFIED_TS_KEY, REL_PATH_KEY = "SHA1", "last_modified_time_stamp", "file_path"


class RepoStatus(Enum):
    CLEAN = 1
    CHANGES_NOT_ADDED = 2
    CHANGES_ADDED_NOT_COMMITED = 3


@dataclass
class SizeInfo:
    """Bytes before de-duplication, after it, and after compression (plus sparsification)."""

    original: int
    deduped: int
    gzipped: int


class Repo:
    def __init__(self, parent_dir: Union[Path, str] = "", init: bool = False) -> None:
        self._wgit_parent = Path(parent_dir if parent_dir != "" else Path.cwd())
        self._dot_wgit = self._wgit_parent / ".wgit"
        exists = (self._dot_wgit / "sha1_store").exists() and (self._dot_wgit / ".git").exists()
        if init and not exists:
            if self._dot_wgit.exists():
                sys.stderr.write("An exception occured while wgit initialization: .wgit exists but is incomplete\n")
                sys.exit(ExitCode.FILE_EXISTS_ERROR.value)
            self._dot_wgit.mkdir(parents=True)
            self._sha1_store = SHA1_Store(self._dot_wgit / "sha1_store", init=True)
            self._pygit = PyGit(self._dot_wgit, gitignore=["sha1_store"])
        elif exists:
            self._sha1_store = SHA1_Store(self._dot_wgit / "sha1_store")
            self._pygit = PyGit(self._dot_wgit)
        else:
            sys.stderr.write("fatal: not a wgit repository!\n")
            sys.exit(ExitCode.FILE_DOES_NOT_EXIST_ERROR.value)

    # ------------------------------------------------------------------ paths
    def _rel_file_path(self, filepath: Path) -> Path:
        return Path(filepath).resolve().relative_to(self._wgit_parent.resolve())

    def _metadata_path(self, file_path: Path) -> Path:
        return self._dot_wgit / self._rel_file_path(file_path)

    # ------------------------------------------------------------------ commands
    def add(self, in_file_path: str, per_tensor: bool = True, gzip: bool = True, sparsify: bool = False,
            sparsify_policy: Any = None) -> Optional[Dict[Any, Any]]:
        """Store the checkpoint at ``in_file_path`` and write its metadata.  With ``per_tensor`` a state dict is
        stored tensor by tensor (shared layers are stored once).  With ``sparsify`` every floating tensor is kept
        as its SST and DST under ``sparsify_policy`` (a :class:`SignalSparsity`, or a callable name -> config)."""
        file_path = Path(in_file_path)
        if not file_path.exists():
            sys.stderr.write(f"fatal: {file_path} does not exist\n")
            sys.exit(ExitCode.FILE_DOES_NOT_EXIST_ERROR.value)
        if sparsify and not per_tensor:
            raise ValueError("Sparsification requires per_tensor storage")
        ret: Optional[Dict[Any, Any]] = None
        if per_tensor:
            state = torch.load(file_path, weights_only=False)
            if not isinstance(state, dict):
                state = {"": state}

            def store(obj: Any, name: str) -> Any:
                if isinstance(obj, dict):
                    return {k: store(v, f"{name}.{k}" if name else str(k)) for k, v in obj.items()}
                if isinstance(obj, torch.Tensor):
                    if sparsify and obj.is_floating_point() and obj.dim() >= 1:
                        policy = sparsify_policy(name) if callable(sparsify_policy) else (sparsify_policy or SignalSparsity(sst_top_k_percent=10, dst_top_k_percent=10))
                        _, sst, dst = policy.lossy_compress(obj)
                        return {"sst": None if sst is None else self._sha1_store.add(sst, gzip, name + ".sst"),
                                "dst": None if dst is None else self._sha1_store.add(dst.to_sparse() if dst is not obj else dst, gzip, name + ".dst")}
                    return self._sha1_store.add(obj, gzip, name)
                return {"_value": obj if isinstance(obj, (int, float, str, bool, type(None))) else repr(obj)}

            sha1: Any = store(state, "")
            ret = sha1
        else:
            sha1 = self._sha1_store.add(file_path, gzip, str(self._rel_file_path(file_path)))
        meta = self._metadata_path(file_path)
        meta.parent.mkdir(parents=True, exist_ok=True)
        meta.write_text(json.dumps({SHA1_KEY: sha1, LAST_MODIFIED_TS_KEY: file_path.stat().st_mtime,
                                    REL_PATH_KEY: str(self._rel_file_path(file_path))}, indent=1))
        self._pygit.add()
        return ret

    def commit(self, message: str) -> None:
        self._pygit.commit(message)

    def size_info(self, path: Optional[str] = None) -> SizeInfo:
        if path is None:
            return SizeInfo(*self._sha1_store.size_info())
        meta = json.loads(self._metadata_path(Path(path)).read_text())
        tot = [0, 0, 0]

        def walk(x: Any) -> None:
            if isinstance(x, str):
                for i, v in enumerate(self._sha1_store.size_info(x)):
                    tot[i] += v
            elif isinstance(x, dict) and "_value" not in x:
                for v in x.values():
                    walk(v)

        walk(meta[SHA1_KEY])
        return SizeInfo(*tot)

    def _metadata_files(self) -> List[Path]:
        return [p for p in self._dot_wgit.rglob("*") if p.is_file() and ".git" not in p.relative_to(self._dot_wgit).parts
                and "sha1_store" not in p.relative_to(self._dot_wgit).parts and p.name != ".gitignore"]

    def status(self) -> Dict[str, RepoStatus]:
        """Status of every tracked file."""
        staged = self._pygit.status()
        out: Dict[str, RepoStatus] = {}
        for meta_file in self._metadata_files():
            meta = json.loads(meta_file.read_text())
            rel = meta[REL_PATH_KEY]
            real = self._wgit_parent / rel
            if real.exists() and real.stat().st_mtime != meta[LAST_MODIFIED_TS_KEY]:
                out[rel] = RepoStatus.CHANGES_NOT_ADDED
            elif str(meta_file.relative_to(self._dot_wgit)) in staged:
                out[rel] = RepoStatus.CHANGES_ADDED_NOT_COMMITED
            else:
                out[rel] = RepoStatus.CLEAN
        return out

    def log(self, file: str) -> None:
        if file:
            print(f"wgit log of the file: {file}")
            print(self._pygit.log(str(self._rel_file_path(Path(file)))))
        else:
            print("wgit log")
            print(self._pygit.log())

    def checkout(self, sha1: str) -> None:
        """Move the metadata tree to git revision ``sha1`` (checkpoint contents are fetched with :meth:`get`)."""
        self._pygit.checkout(sha1)

    def checkout_by_steps(self) -> None:
        raise NotImplementedError

    def get(self, path: str) -> Any:
        """Rebuild the object stored for ``path`` at the current metadata revision."""
        meta = json.loads(self._metadata_path(Path(path)).read_text())

        def load(x: Any) -> Any:
            if isinstance(x, str):
                return self._sha1_store.get(x)
            if isinstance(x, dict) and set(x.keys()) == {"sst", "dst"}:
                sst = None if x["sst"] is None else self._sha1_store.get(x["sst"])
                dst = None if x["dst"] is None else self._sha1_store.get(x["dst"])
                dst = dst.to_dense() if dst is not None and dst.is_sparse else dst
                return SignalSparsity(sst_top_k_percent=100).sst_dst_to_dense(sst, dst)
            if isinstance(x, dict) and set(x.keys()) == {"_value"}:
                return x["_value"]
            if isinstance(x, dict):
                return {k: load(v) for k, v in x.items()}
            return x

        out = load(meta[SHA1_KEY])
        return out[""] if isinstance(out, dict) and set(out.keys()) == {""} else out

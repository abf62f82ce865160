"""Content-addressed store for tensors, state dicts and files, with reference counts and optional compression.

Capability parity with fairscale/experimental/wgit/sha1_store.py:122-509: ``add`` returns the SHA1 of the content
and stores it once however often it is added (a state dict is stored tensor by tensor, so unchanged layers of
successive checkpoints are shared), ``get`` / ``delete`` / ``size_info`` / ``names``; bookkeeping lives in one JSON
file guarded by a lock file.  Compression uses the standard library's gzip (the reference needs ``pgzip``).
"""

from __future__ import annotations

from collections import OrderedDict
import fcntl
import gzip
import hashlib
import io
import json
import os
from pathlib import Path
import shutil
import sys
import tempfile
import time
from typing import Any, Dict, Optional, Tuple, Union

import torch
from torch import Tensor

from .utils import ExitCode

ENTRY_RF_KEY, ENTRY_COMP_KEY, ENTRY_OS_KEY, ENTRY_DS_KEY, ENTRY_CS_KEY, ENTRY_NAMES_KEY = (
    "ref_count", "compressed", "original_size", "deduped_size", "compressed_size", "names")
STORE_CREATE_DATE_KEY, STORE_OS_KEY, STORE_DS_KEY, STORE_CS_KEY = "created_on", "original_size", "deduped_size", "compressed_size"
_STORE_KEYS = (STORE_CREATE_DATE_KEY, STORE_OS_KEY, STORE_DS_KEY, STORE_CS_KEY)


class _Locked:
    """Hold the store's lock file and the parsed JSON state; write it back on exit unless read-only."""

    def __init__(self, store: "SHA1_Store", readonly: bool):
        self.s, self.readonly = store, readonly

    def __enter__(self) -> None:
        self.fd = open(self.s._lock_path, "w")
        fcntl.flock(self.fd, fcntl.LOCK_EX)
        self.s._json = json.loads(self.s._meta_path.read_text()) if self.s._meta_path.exists() else {}

    def __exit__(self, *exc: Any) -> None:
        if not self.readonly and exc[0] is None:
            tmp = self.s._meta_path.with_suffix(".tmp")
            tmp.write_text(json.dumps(self.s._json, indent=1))
            os.replace(tmp, self.s._meta_path)
        self.s._json = None
        fcntl.flock(self.fd, fcntl.LOCK_UN)
        self.fd.close()


class SHA1_Store:
    """Args: ``path`` of the store directory; ``init``: create it (must not exist) instead of opening it;
    ``sha1_buf_size``: read block size when hashing; ``tmp_dir``: where serialisations are staged."""

    def __init__(self, path: Path, init: bool = False, sha1_buf_size: int = 100 * 1024 * 1024, tmp_dir: str = "",
                 pgzip_threads: Optional[int] = None, pgzip_block_size: int = 10 * 1024 * 1024) -> None:
        self._path = Path(path)
        self._meta_path = self._path / "sha1_store.json"
        self._lock_path = self._path / ".lock"
        self._sha1_buf_size = sha1_buf_size
        self._json: Optional[Dict[str, Any]] = None
        if init:
            if self._path.exists():
                sys.stderr.write(f"An exception occured while creating Sha1_store: {self._path} exists\n")
                sys.exit(ExitCode.FILE_EXISTS_ERROR.value)
            self._path.mkdir(parents=True)
            with _Locked(self, readonly=False):
                self._json = {STORE_CREATE_DATE_KEY: time.ctime(), STORE_OS_KEY: 0, STORE_DS_KEY: 0, STORE_CS_KEY: 0}
        if not self._meta_path.exists():
            raise RuntimeError(f"Metadata file {self._meta_path} is expected")
        self._tmp_dir = Path(tmp_dir) if tmp_dir else self._path / "tmp"
        self._tmp_dir.mkdir(exist_ok=True)

    # ------------------------------------------------------------------ helpers
    def _sha1_to_dir(self, sha1: str) -> Path:
        assert len(sha1) > 4, "sha1 too short"
        return self._path / sha1[:2] / sha1[2:4]

    def _get_sha1_hash(self, file_path: Union[str, Path]) -> str:
        h = hashlib.sha1()
        with open(file_path, "rb") as f:
            while True:
                data = f.read(self._sha1_buf_size)
                if not data:
                    break
                h.update(data)
        return h.hexdigest()

    def _stage(self, obj: Any) -> Path:
        fd, name = tempfile.mkstemp(dir=self._tmp_dir)
        buf = io.BytesIO()  # serialising to memory keeps the archive's internal names, hence the hash, stable
        torch.save(obj, buf)
        with os.fdopen(fd, "wb") as f:
            f.write(buf.getvalue())
        return Path(name)

    # ------------------------------------------------------------------ API
    def add(self, file_or_obj: Union[Path, str, Tensor, Dict], compress: bool = True, name: Optional[str] = None) -> Union[str, Dict]:
        """Store a file, a tensor, or (recursively) a state dict.  Returns the SHA1, or for a dict the same
        structure with every tensor replaced by its SHA1 string."""
        if isinstance(file_or_obj, (dict, OrderedDict)):
            return {k: self.add(v, compress, f"{name}.{k}" if name else str(k)) for k, v in file_or_obj.items()}
        staged = None
        if isinstance(file_or_obj, (Path, str)) and Path(file_or_obj).exists():
            src = Path(file_or_obj)
            try:  # a serialised tensor / state dict stays loadable by get(); any other file is kept as bytes
                torch.load(src, weights_only=True)
            except Exception:
                pass
        elif isinstance(file_or_obj, Tensor):
            staged = src = self._stage(file_or_obj.detach().cpu())
        else:
            raise ValueError(f"unsupported type for add: {type(file_or_obj)}")
        try:
            sha1 = self._get_sha1_hash(src)
            orig = src.stat().st_size
            with _Locked(self, readonly=False):
                assert self._json is not None
                entry = self._json.get(sha1)
                if entry is None:
                    d = self._sha1_to_dir(sha1)
                    d.mkdir(parents=True, exist_ok=True)
                    dest = d / sha1
                    if compress:
                        with open(src, "rb") as fi, gzip.open(dest, "wb", compresslevel=5) as fo:
                            shutil.copyfileobj(fi, fo, 16 * 1024 * 1024)
                    else:
                        shutil.copyfile(src, dest)
                    csize = dest.stat().st_size
                    # the original size of an entry counts every reference, the other two count the stored copy once
                    entry = {ENTRY_RF_KEY: 0, ENTRY_COMP_KEY: compress, ENTRY_OS_KEY: 0, ENTRY_DS_KEY: orig,
                             ENTRY_CS_KEY: csize, ENTRY_NAMES_KEY: {}}
                    self._json[sha1] = entry
                    self._json[STORE_DS_KEY] += orig
                    self._json[STORE_CS_KEY] += csize
                elif entry[ENTRY_COMP_KEY] != compress:
                    raise ValueError(f"{sha1} was stored with compress={entry[ENTRY_COMP_KEY]}; cannot add it with compress={compress}")
                entry[ENTRY_RF_KEY] += 1
                entry[ENTRY_OS_KEY] += orig
                if name:
                    entry[ENTRY_NAMES_KEY][name] = entry[ENTRY_NAMES_KEY].get(name, 0) + 1
                self._json[STORE_OS_KEY] += orig
            return sha1
        finally:
            if staged is not None:
                staged.unlink(missing_ok=True)

    def get(self, sha1: str) -> Any:
        """Load the object stored under ``sha1`` (raises ValueError when unknown)."""
        with _Locked(self, readonly=True):
            assert self._json is not None
            entry = self._json.get(sha1)
        path = self._sha1_to_dir(sha1) / sha1
        if entry is None or not path.exists():
            raise ValueError(f"Try to get SHA1 {sha1} but it is not found")
        if entry[ENTRY_COMP_KEY]:
            with gzip.open(path, "rb") as f:
                return torch.load(io.BytesIO(f.read()), weights_only=False)
        return torch.load(path, weights_only=False)

    def delete(self, sha1: str) -> None:
        """Drop one reference; the content goes away with the last one."""
        with _Locked(self, readonly=False):
            assert self._json is not None
            entry = self._json.get(sha1)
            if entry is None:
                raise ValueError(f"Try to delete SHA1 {sha1} but it is not found")
            one = entry[ENTRY_OS_KEY] // max(1, entry[ENTRY_RF_KEY])
            entry[ENTRY_RF_KEY] -= 1
            entry[ENTRY_OS_KEY] -= one
            self._json[STORE_OS_KEY] -= one
            if entry[ENTRY_RF_KEY] <= 0:
                (self._sha1_to_dir(sha1) / sha1).unlink(missing_ok=True)
                self._json[STORE_DS_KEY] -= entry[ENTRY_DS_KEY]
                self._json[STORE_CS_KEY] -= entry[ENTRY_CS_KEY]
                del self._json[sha1]

    def size_info(self, sha1: Optional[str] = None) -> Tuple[int, int, int]:
        """(original, de-duplicated, compressed) bytes of the whole store or of one entry."""
        with _Locked(self, readonly=True):
            assert self._json is not None
            d = self._json if sha1 is None else self._json[sha1]
            return d[STORE_OS_KEY], d[STORE_DS_KEY], d[STORE_CS_KEY]

    def names(self, sha1: Optional[str] = None) -> Dict[str, int]:
        """Names (with counts) under which ``sha1`` was added; ``None`` lists all SHA1s with their ref counts."""
        with _Locked(self, readonly=True):
            assert self._json is not None
            if sha1 is None:
                return {k: v[ENTRY_RF_KEY] for k, v in self._json.items() if k not in _STORE_KEYS}
            if sha1 not in self._json:
                return {}
            return dict(self._json[sha1][ENTRY_NAMES_KEY])

"""Where checkpoint folders live: a local directory tree or any fsspec URI (`gs://`, `s3://`, `memory://`, ...)
(reference: llmtuner/components/checkpointer/storage/filesystem.py:1-93 and storage/storage.py:19-78 keep the same split
between path operations and the checkpoint logic that calls them).

The checkpoint manager never touches `os` or `shutil` itself; it asks a `CheckpointStorage` to join, list, rename and
delete, and to hand out the torch-DCP reader and writer for a folder. Paths stay strings from end to end so that a URI
scheme survives every join. Publication is a rename of `step-N.tmp-<id>` to `step-N`: atomic on a POSIX filesystem; on an
object store it is a copy followed by a delete, which is why a folder only counts as a checkpoint once its `.metadata`
object (written last by the coordinator) exists under the final name.
"""
from __future__ import annotations

import os
import posixpath
import re
import shutil

from ...errors import EnvironmentUnsupportedError

_SCHEME = re.compile(r"^[A-Za-z][A-Za-z0-9+.\-]*://")


def is_remote(path) -> bool:
    """True for `scheme://...`; a Windows drive letter or a bare path is local. `file://` counts as remote here (it goes
    through fsspec's local filesystem), which gives tests a second backend without any network."""
    return bool(_SCHEME.match(os.fspath(path)))


class LocalStorage:
    remote = False

    def join(self, base: str, *names: str) -> str:
        out = os.fspath(base)
        for n in names:
            out = n if is_remote(n) else os.path.join(out, n)
        return out

    def isdir(self, path: str) -> bool:
        return os.path.isdir(path)

    def exists(self, path: str) -> bool:
        return os.path.exists(path)

    def listdir(self, path: str) -> list[str]:
        return os.listdir(path)

    def makedirs(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)

    def rmtree(self, path: str) -> None:
        """Missing paths are fine (a concurrent purge, a retry); every other failure propagates."""
        try:
            shutil.rmtree(path)
        except FileNotFoundError:
            pass

    def rename(self, src: str, dst: str) -> None:
        os.replace(src, dst)

    def reader(self, path: str):
        import torch.distributed.checkpoint as dcp
        return dcp.FileSystemReader(path)

    def writer(self, path: str):
        import torch.distributed.checkpoint as dcp
        return dcp.FileSystemWriter(path)


class FsspecStorage:
    """Every operation resolves its own (filesystem, path) pair from the URI, so one manager can read an initial
    checkpoint from one store and write its own steps to another."""
    remote = True

    def __init__(self):
        try:
            from fsspec.core import url_to_fs
        except ImportError as e:                                                    # pragma: no cover - fsspec ships here
            raise EnvironmentUnsupportedError("checkpoint paths with a URI scheme need the fsspec package") from e
        self._url_to_fs = url_to_fs

    def _fs(self, path: str):
        return self._url_to_fs(os.fspath(path))

    def join(self, base: str, *names: str) -> str:
        out = os.fspath(base)
        for n in names:
            if is_remote(n):
                out = n
            elif is_remote(out):
                out = posixpath.join(out, n)              # URIs are '/'-separated on every platform
            else:
                out = os.path.join(out, n)
        return out

    def isdir(self, path: str) -> bool:
        fs, p = self._fs(path)
        return fs.isdir(p)

    def exists(self, path: str) -> bool:
        fs, p = self._fs(path)
        return fs.exists(p)

    def listdir(self, path: str) -> list[str]:
        """Basenames, like `os.listdir`. Object stores may list a zero-byte marker for the folder itself; it is dropped
        by comparing whole paths, so a child that shares its parent's basename stays."""
        fs, p = self._fs(path)
        me = p.rstrip("/")
        return [posixpath.basename(e.rstrip("/")) for e in fs.ls(p, detail=False) if e.rstrip("/") != me]

    def makedirs(self, path: str) -> None:
        fs, p = self._fs(path)
        fs.makedirs(p, exist_ok=True)

    def rmtree(self, path: str) -> None:
        fs, p = self._fs(path)
        try:
            fs.rm(p, recursive=True)
        except FileNotFoundError:
            pass

    def rename(self, src: str, dst: str) -> None:
        fs, s = self._fs(src)
        fs2, d = self._fs(dst)
        if type(fs) is not type(fs2):
            raise ValueError(f"cannot rename across stores: {src} -> {dst}")
        fs.mv(s, d, recursive=True)

    def reader(self, path: str):
        from torch.distributed.checkpoint._fsspec_filesystem import FsspecReader
        return FsspecReader(path)

    def writer(self, path: str):
        from torch.distributed.checkpoint._fsspec_filesystem import FsspecWriter
        return FsspecWriter(path)


def storage_for(path) -> "LocalStorage | FsspecStorage":
    return FsspecStorage() if is_remote(path) else LocalStorage()

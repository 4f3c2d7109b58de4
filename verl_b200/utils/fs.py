"""Local / remote (``hdfs://``) path handling with a local cache: checkpoints and datasets are addressed by one string and
materialised on local disk (or ``/dev/shm``) before use.

Parity target: ``verl/utils/fs.py`` (``is_non_local`` :34, ``md5_encode`` :46, ``get_local_temp_path`` :61, ``verify_copy``
:82, ``copy_to_shm`` :141, ``copy_to_local`` :195, ``copy_local_path_from_hdfs`` :232, ``local_mkdir_safe`` :277).
"""

from __future__ import annotations

import hashlib
import os
import shutil
import tempfile
from typing import Optional

from . import hdfs_io

__all__ = ["is_non_local", "md5_encode", "get_local_temp_path", "verify_copy", "copy_to_shm", "copy_to_local",
           "copy_local_path_from_hdfs", "local_mkdir_safe"]

_HDFS_PREFIX = "hdfs://"


def is_non_local(path: Optional[str]) -> bool:
    return bool(path) and str(path).startswith(_HDFS_PREFIX)


def md5_encode(path: str) -> str:
    return hashlib.md5(path.encode()).hexdigest()


def get_local_temp_path(hdfs_path: str, cache_dir: str) -> str:
    """``cache_dir/<md5 of the remote path>/<basename>``: distinct remote files never collide, the name stays readable."""
    d = os.path.join(cache_dir, md5_encode(hdfs_path))
    os.makedirs(d, exist_ok=True)
    return os.path.join(d, os.path.basename(hdfs_path.rstrip("/")))


def _tree(path: str) -> list[tuple[str, int]]:
    if os.path.isfile(path):
        return [("", os.path.getsize(path))]
    out = []
    for root, _, files in os.walk(path):
        for f in sorted(files):
            full = os.path.join(root, f)
            out.append((os.path.relpath(full, path), os.path.getsize(full)))
    return sorted(out)


def verify_copy(src: str, dest: str) -> bool:
    """Same file (or same tree of relative names) with the same sizes."""
    if not os.path.exists(src) or not os.path.exists(dest):
        return False
    if os.path.isfile(src) != os.path.isfile(dest):
        return False
    return _tree(src) == _tree(dest)


def copy_to_shm(src: str) -> str:
    """Stage a local file or directory in shared memory (fast repeated loads by several processes of a node)."""
    base = "/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir()
    dest = os.path.join(base, "verl-cache", md5_encode(os.path.abspath(src)), os.path.basename(src.rstrip("/")))
    if os.path.exists(dest) and verify_copy(src, dest):
        return dest
    os.makedirs(os.path.dirname(dest), exist_ok=True)
    if os.path.isdir(src):
        shutil.copytree(src, dest, symlinks=False, dirs_exist_ok=True)
    else:
        shutil.copy2(src, dest)
    return dest


def copy_local_path_from_hdfs(src: str, cache_dir: Optional[str] = None, filelock: str = ".file.lock", verbose: bool = False,
                              always_recopy: bool = False) -> str:
    """Remote paths are fetched into the cache (once, under a file lock so that the ranks of a node do not race); local
    paths are returned unchanged."""
    if not is_non_local(src):
        return src
    cache_dir = cache_dir or os.path.join(tempfile.gettempdir(), "verl-cache")
    os.makedirs(cache_dir, exist_ok=True)
    local = get_local_temp_path(src, cache_dir)
    from filelock import FileLock

    with FileLock(os.path.join(cache_dir, md5_encode(src) + filelock)):
        if always_recopy and os.path.exists(local):
            shutil.rmtree(local, ignore_errors=True) if os.path.isdir(local) else os.remove(local)
        if not os.path.exists(local):
            if verbose:
                print(f"copy {src} -> {local}")
            if not hdfs_io.copy(src, local):
                raise IOError(f"could not fetch {src}")
    return local


def copy_to_local(src: str, cache_dir: Optional[str] = None, filelock: str = ".file.lock", verbose: bool = False,
                  always_recopy: bool = False, use_shm: bool = False) -> str:
    local = copy_local_path_from_hdfs(src, cache_dir, filelock, verbose, always_recopy)
    return copy_to_shm(local) if use_shm and os.path.exists(local) else local


def local_mkdir_safe(path: str) -> str:
    """``makedirs`` that several processes may call for the same path at once."""
    if not os.path.isabs(path):
        path = os.path.join(os.getcwd(), path)
    from filelock import FileLock

    lock = os.path.join(tempfile.gettempdir(), f"ckpt_{hash(path) & 0xFFFFFFFF:08x}.lock")
    try:
        with FileLock(lock, timeout=60):
            os.makedirs(path, exist_ok=True)
    except Exception:
        os.makedirs(path, exist_ok=True)
    return path

"""``exists`` / ``makedirs`` / ``copy`` that accept both local paths and ``hdfs://`` URIs (the latter through the ``hdfs``
command-line client, when one is installed).

Parity target: ``verl/utils/hdfs_io.py`` (``exists`` :27, ``makedirs`` :50, ``copy`` :84, ``_run_cmd`` :140).
"""

from __future__ import annotations

import os
import shutil
import subprocess
from typing import Optional

__all__ = ["exists", "makedirs", "copy"]

_HDFS_PREFIX = "hdfs://"
_HDFS_BIN = os.environ.get("HDFS_BIN", "hdfs")


def _is_non_local(path: str) -> bool:
    return str(path).startswith(_HDFS_PREFIX)


def _run_cmd(cmd: list[str], timeout: Optional[float] = None) -> int:
    try:
        return subprocess.run(cmd, timeout=timeout, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL).returncode
    except (FileNotFoundError, subprocess.TimeoutExpired):
        return 127


def _hdfs(*args: str) -> list[str]:
    return [_HDFS_BIN, "dfs", *args]


def exists(path: str, **kwargs) -> bool:
    return _run_cmd(_hdfs("-test", "-e", path)) == 0 if _is_non_local(path) else os.path.exists(path)


def makedirs(name: str, mode: int = 0o777, exist_ok: bool = False, **kwargs) -> None:
    if _is_non_local(name):
        if _run_cmd(_hdfs("-mkdir", "-p", name)) != 0:
            raise IOError(f"hdfs mkdir failed for {name}")
        return
    os.makedirs(name, mode=mode, exist_ok=exist_ok)


def copy(src: str, dst: str, timeout: Optional[float] = None, **kwargs) -> bool:
    """Any combination of local and remote endpoints; directories are copied recursively. Returns success."""
    if _is_non_local(src) and not _is_non_local(dst):
        return _run_cmd(_hdfs("-get", src, dst), timeout) == 0
    if not _is_non_local(src) and _is_non_local(dst):
        return _run_cmd(_hdfs("-put", "-f", src, dst), timeout) == 0
    if _is_non_local(src):
        return _run_cmd(_hdfs("-cp", "-f", src, dst), timeout) == 0
    try:
        if os.path.isdir(src):
            shutil.copytree(src, dst, dirs_exist_ok=True)
        else:
            os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
            shutil.copy2(src, dst)
        return True
    except OSError:
        return False

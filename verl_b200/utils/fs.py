"""File-system helpers (reference: ``verl/utils/fs.py``, ``verl/utils/hdfs_io.py``): ``copy_to_local`` with an optional
shared-memory staging area, md5-based cache names, ``hdfs://`` paths through the ``hdfs`` command line when present."""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import tempfile
from typing import Optional

__all__ = ["is_non_local", "md5_encode", "get_local_temp_path", "copy_to_local", "copy_local_path_from_hdfs", "local_mkdir_safe", "exists", "makedirs", "copy"]

_HDFS_PREFIX = "hdfs://"


def is_non_local(path: str) -> bool:
    return isinstance(path, str) and path.startswith(_HDFS_PREFIX)


def md5_encode(path: str) -> str:
    return hashlib.md5(path.encode()).hexdigest()


def get_local_temp_path(hdfs_path: str, cache_dir: str) -> str:
    return os.path.join(cache_dir, md5_encode(hdfs_path), os.path.basename(hdfs_path.rstrip("/")))


def _hdfs(*args) -> int:
    exe = shutil.which("hdfs")
    if exe is None:
        raise RuntimeError("an hdfs:// path was given but the `hdfs` command is not installed")
    return subprocess.run([exe, "dfs", *args], check=False).returncode


def exists(path: str) -> bool:
    return _hdfs("-test", "-e", path) == 0 if is_non_local(path) else os.path.exists(path)


def makedirs(path: str, exist_ok: bool = True):
    if is_non_local(path):
        _hdfs("-mkdir", "-p", path)
    else:
        os.makedirs(path, exist_ok=exist_ok)


def local_mkdir_safe(path: str) -> str:
    os.makedirs(os.path.abspath(path), exist_ok=True)
    return path


def copy(src: str, dst: str):
    if is_non_local(src) or is_non_local(dst):
        rc = _hdfs("-get", src, dst) if is_non_local(src) else _hdfs("-put", "-f", src, dst)
        if rc != 0:
            raise RuntimeError(f"hdfs copy {src} -> {dst} failed with code {rc}")
    elif os.path.isdir(src):
        shutil.copytree(src, dst, dirs_exist_ok=True)
    else:
        shutil.copy(src, dst)


def copy_local_path_from_hdfs(src: str, cache_dir: Optional[str] = None, always_recopy: bool = False) -> str:
    cache_dir = cache_dir or os.path.join(tempfile.gettempdir(), "verl_b200_cache")
    if not is_non_local(src):
        return src
    local = get_local_temp_path(src, cache_dir)
    if always_recopy and os.path.exists(local):
        shutil.rmtree(local, ignore_errors=True)
    if not os.path.exists(local):
        os.makedirs(os.path.dirname(local), exist_ok=True)
        copy(src, local)
    return local


def copy_to_local(src: str, cache_dir: Optional[str] = None, always_recopy: bool = False, use_shm: bool = False) -> str:
    """Local path of ``src``: remote paths are fetched into a cache; ``use_shm`` additionally stages a local directory in
    ``/dev/shm`` so that many processes of one box load the checkpoint from memory."""
    local = copy_local_path_from_hdfs(src, cache_dir, always_recopy)
    if use_shm and os.path.isdir("/dev/shm") and os.path.exists(local):
        dst = os.path.join("/dev/shm", "verl_b200_cache", md5_encode(os.path.abspath(local)), os.path.basename(local.rstrip("/")))
        if always_recopy or not os.path.exists(dst):
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            copy(local, dst)
        return dst
    return local

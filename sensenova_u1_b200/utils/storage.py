"""Checkpoint storage back-ends behind one ``"<scheme>:<path>"`` spelling.

The reference routes every checkpoint read/write through a storage manager with ``local:``,
boto3 S3, Volcano TOS and Ali OSS clients, uploading asynchronously from a ``/dev/shm`` staging
file (training/sensenovalm/utils/storage_manager.py:105-1281).  Here the same interface has two
built-in back-ends — ``local:`` and ``file:`` — an asynchronous writer (a background thread that
moves staged files into place, so the training loop only pays for the serialisation), and a
registry for remote clients: ``register_backend("s3", client)`` with an object that implements
``upload(local_path, remote_path)``, ``download(remote_path, local_path)``, ``exists`` and
``listdir``.  boto3 is not a dependency; an ``S3Backend`` adapter is provided for environments
that have it.
"""
from __future__ import annotations

import hashlib
import os
import queue
import shutil
import tempfile
import threading
from typing import Callable, Dict, List, Optional, Tuple

import torch


class LocalBackend:
    def upload(self, local_path: str, remote_path: str) -> None:
        os.makedirs(os.path.dirname(remote_path) or ".", exist_ok=True)
        tmp = remote_path + ".tmp"
        shutil.copyfile(local_path, tmp)
        os.replace(tmp, remote_path)                 # readers never see a half-written file

    def download(self, remote_path: str, local_path: str) -> None:
        shutil.copyfile(remote_path, local_path)

    def exists(self, remote_path: str) -> bool:
        return os.path.exists(remote_path)

    def listdir(self, remote_path: str) -> List[str]:
        return sorted(os.listdir(remote_path)) if os.path.isdir(remote_path) else []


class S3Backend:
    """``s3:bucket/key`` through boto3 (imported on first use)."""

    def __init__(self, endpoint_url: Optional[str] = None):
        self.endpoint_url, self._client = endpoint_url, None

    def _c(self):
        if self._client is None:
            import boto3                       # not a dependency of the package
            self._client = boto3.client("s3", endpoint_url=self.endpoint_url)
        return self._client

    @staticmethod
    def _split(path: str) -> Tuple[str, str]:
        bucket, _, key = path.lstrip("/").partition("/")
        return bucket, key

    def upload(self, local_path, remote_path):
        b, k = self._split(remote_path)
        self._c().upload_file(local_path, b, k)

    def download(self, remote_path, local_path):
        b, k = self._split(remote_path)
        self._c().download_file(b, k, local_path)

    def exists(self, remote_path):
        b, k = self._split(remote_path)
        try:
            self._c().head_object(Bucket=b, Key=k)
            return True
        except Exception:
            return False

    def listdir(self, remote_path):
        b, k = self._split(remote_path)
        out = self._c().list_objects_v2(Bucket=b, Prefix=k.rstrip("/") + "/", Delimiter="/")
        names = [p["Prefix"].rstrip("/").rsplit("/", 1)[-1] for p in out.get("CommonPrefixes", [])]
        return sorted(names + [o["Key"].rsplit("/", 1)[-1] for o in out.get("Contents", [])])


# "s3:bucket/key" needs boto3 at first use only; other object stores register their client with register_backend
_BACKENDS: Dict[str, object] = {"local": LocalBackend(), "file": LocalBackend(), "s3": S3Backend(os.environ.get("S3_ENDPOINT_URL"))}


def register_backend(scheme: str, backend) -> None:
    _BACKENDS[scheme] = backend


def split_url(url: str) -> Tuple[object, str]:
    """``"local:/a/b"`` -> (backend, "/a/b"); a bare path is local."""
    scheme, sep, rest = url.partition(":")
    if sep and scheme in _BACKENDS:
        return _BACKENDS[scheme], rest
    if sep and scheme.isalpha() and len(scheme) > 1 and not os.path.exists(url):
        raise KeyError(f"no storage back-end registered for {scheme!r} (known: {sorted(_BACKENDS)})")
    return _BACKENDS["local"], url


def md5_of(path: str) -> str:
    h = hashlib.md5()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return h.hexdigest()


class AsyncWriter:
    """Serialises on the caller's thread into a staging directory (``/dev/shm`` when present) and
    moves the file to its destination on a background thread."""

    def __init__(self, staging: Optional[str] = None):
        base = staging or ("/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else None)
        self.staging = tempfile.mkdtemp(prefix="snu1_ckpt_", dir=base)
        self.q: "queue.Queue" = queue.Queue()
        self.errors: List[str] = []
        self.t = threading.Thread(target=self._loop, daemon=True)
        self.t.start()

    def _loop(self):
        while True:
            item = self.q.get()
            if item is None:
                return
            staged, url = item
            try:
                backend, path = split_url(url)
                backend.upload(staged, path)
            except Exception as e:                   # reported by wait(); the loop keeps serving
                self.errors.append(f"{url}: {type(e).__name__}: {e}")
            finally:
                try:
                    os.unlink(staged)
                except OSError:
                    pass
                self.q.task_done()

    def save(self, obj, url: str) -> None:
        fd, staged = tempfile.mkstemp(dir=self.staging)
        os.close(fd)
        torch.save(obj, staged)
        self.q.put((staged, url))

    def wait(self) -> None:
        self.q.join()
        if self.errors:
            errs, self.errors = self.errors, []
            raise IOError("asynchronous checkpoint upload failed: " + "; ".join(errs))

    def close(self) -> None:
        self.q.join()
        self.q.put(None)
        self.t.join(timeout=5)
        shutil.rmtree(self.staging, ignore_errors=True)


def llm_save(url: str, obj) -> None:
    backend, path = split_url(url)
    fd, tmp = tempfile.mkstemp()
    os.close(fd)
    try:
        torch.save(obj, tmp)
        backend.upload(tmp, path)
    finally:
        os.unlink(tmp)


def llm_load(url: str, map_location="cpu"):
    backend, path = split_url(url)
    if isinstance(backend, LocalBackend):
        return torch.load(path, map_location=map_location)
    fd, tmp = tempfile.mkstemp()
    os.close(fd)
    try:
        backend.download(path, tmp)
        return torch.load(tmp, map_location=map_location)
    finally:
        os.unlink(tmp)

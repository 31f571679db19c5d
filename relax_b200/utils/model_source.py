"""Where model files come from: local directories, ``file://`` URLs and object stores (``s3://bucket/prefix``),
fetched once per node into a cache directory with parallel ranged reads, resume and an atomic completion marker.

Covers the reference's model-source helpers (relax/utils/s3_model_loader.py: parallel chunked download,
manifest, per-node lock and wait; relax/utils/model_source.py: URI resolution; relax/utils/hf_page_cache.py:
page-cache warm-up before many ranks open the same safetensors files).

The object-store client is an interface (:class:`ObjectStore`): ``S3Store`` wraps ``boto3`` when it is installed,
``DirStore`` serves a directory (``file://`` URLs; also what the tests use as a stand-in bucket).
"""
from __future__ import annotations

import fnmatch
import json
import os
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence, Tuple

DEFAULT_PATTERNS = ("*.safetensors", "*.json", "*.txt", "*.model", "*.tiktoken", "*.jinja", "*.py")
_MARKER = ".complete.json"


@dataclass(frozen=True)
class ObjectInfo:
    key: str        # relative to the prefix
    size: int
    etag: str = ""


class ObjectStore:
    def list(self, prefix: str) -> List[ObjectInfo]:
        raise NotImplementedError

    def read(self, prefix: str, key: str, offset: int, length: int) -> bytes:
        raise NotImplementedError


class DirStore(ObjectStore):
    """A directory tree presented as a bucket: ``prefix`` is a path under ``root``."""

    def __init__(self, root: str = "/"):
        self.root = root

    def _p(self, prefix, key=""):
        return os.path.join(self.root, prefix.lstrip("/"), key)

    def list(self, prefix):
        base = self._p(prefix)
        out = []
        for d, _, files in os.walk(base):
            for f in files:
                full = os.path.join(d, f)
                st = os.stat(full)
                out.append(ObjectInfo(os.path.relpath(full, base), st.st_size, f"{st.st_size:x}-{int(st.st_mtime_ns):x}"))
        return sorted(out, key=lambda o: o.key)

    def read(self, prefix, key, offset, length):
        with open(self._p(prefix, key), "rb") as f:
            f.seek(offset)
            return f.read(length)


class S3Store(ObjectStore):
    """``boto3`` client wrapper; the import is deferred so the package works without it."""

    def __init__(self, bucket: str, endpoint_url: Optional[str] = None, client=None):
        self.bucket = bucket
        if client is None:
            try:
                import boto3  # type: ignore
            except ImportError as e:   # pragma: no cover - depends on the image
                raise RuntimeError("s3:// model sources need boto3; install it or pre-download the model "
                                   "and pass a local path") from e
            client = boto3.client("s3", endpoint_url=endpoint_url or os.environ.get("AWS_ENDPOINT_URL"))
        self.client = client

    def list(self, prefix):
        prefix = prefix.strip("/") + "/"
        out, token = [], None
        while True:
            kw = dict(Bucket=self.bucket, Prefix=prefix)
            if token:
                kw["ContinuationToken"] = token
            r = self.client.list_objects_v2(**kw)
            for o in r.get("Contents", []):
                if not o["Key"].endswith("/"):
                    out.append(ObjectInfo(o["Key"][len(prefix):], int(o["Size"]), str(o.get("ETag", "")).strip('"')))
            token = r.get("NextContinuationToken")
            if not token:
                return sorted(out, key=lambda o: o.key)

    def read(self, prefix, key, offset, length):
        k = prefix.strip("/") + "/" + key
        r = self.client.get_object(Bucket=self.bucket, Key=k, Range=f"bytes={offset}-{offset + length - 1}")
        return r["Body"].read()


# --------------------------------------------------------------------------- URIs
def parse_model_uri(uri: str) -> Tuple[str, str, str]:
    """``(scheme, bucket, path)``: scheme is ``local`` / ``file`` / ``s3``."""
    if uri.startswith("s3://"):
        rest = uri[5:]
        bucket, _, path = rest.partition("/")
        if not bucket:
            raise ValueError(f"no bucket in {uri!r}")
        return "s3", bucket, path.strip("/")
    if uri.startswith("file://"):
        return "file", "", uri[7:]
    if "://" in uri:
        raise ValueError(f"unsupported model source {uri!r} (local path, file:// or s3://)")
    return "local", "", uri


def cache_subdir(uri: str) -> str:
    scheme, bucket, path = parse_model_uri(uri)
    safe = "".join(c if c.isalnum() or c in "-_." else "_" for c in f"{bucket}_{path}".strip("_"))
    return f"{scheme}_{safe}"


# --------------------------------------------------------------------------- download
def _select(objs: Iterable[ObjectInfo], patterns: Sequence[str]) -> List[ObjectInfo]:
    return [o for o in objs if any(fnmatch.fnmatch(os.path.basename(o.key), p) for p in patterns)]


def _ranges(size: int, chunk: int):
    off = 0
    while off < size:
        yield off, min(chunk, size - off)
        off += chunk
    if size == 0:
        yield 0, 0


def is_complete(dest: str, objs: Optional[Sequence[ObjectInfo]] = None) -> bool:
    m = os.path.join(dest, _MARKER)
    if not os.path.exists(m):
        return False
    try:
        rec = json.load(open(m))["files"]
    except (ValueError, KeyError):
        return False
    if objs is not None and {o.key: [o.size, o.etag] for o in objs} != rec:
        return False     # the source changed since the marker was written
    return all(os.path.exists(os.path.join(dest, k)) and os.path.getsize(os.path.join(dest, k)) == v[0] for k, v in rec.items())


def download_model(store: ObjectStore, prefix: str, dest: str, patterns: Sequence[str] = DEFAULT_PATTERNS,
                   workers: int = 8, chunk_bytes: int = 64 << 20, retries: int = 3) -> dict:
    """Mirror ``prefix`` into ``dest``.  Files already present with the listed size are kept (resume); each file
    is written as ``<name>.part`` by ranged reads issued from a thread pool and renamed when whole; the
    completion marker is written last, so a killed download is never mistaken for a finished one."""
    objs = _select(store.list(prefix), patterns)
    if not objs:
        raise FileNotFoundError(f"nothing matching {list(patterns)} under {prefix!r}")
    os.makedirs(dest, exist_ok=True)
    if is_complete(dest, objs):
        return {"files": len(objs), "bytes": 0, "skipped": len(objs), "seconds": 0.0}
    t0 = time.monotonic()
    todo, skipped = [], 0
    for o in objs:
        final = os.path.join(dest, o.key)
        if os.path.exists(final) and os.path.getsize(final) == o.size and _recorded_etag(dest, o.key) in ("", o.etag):
            skipped += 1
            continue
        os.makedirs(os.path.dirname(final) or dest, exist_ok=True)
        with open(final + ".part", "wb") as f:
            f.truncate(o.size)
        todo.append(o)
    lock = threading.Lock()
    moved = [0]

    def fetch(job):
        o, off, n = job
        err = None
        for attempt in range(retries):
            try:
                data = store.read(prefix, o.key, off, n) if n else b""
                if len(data) != n:
                    raise IOError(f"short read of {o.key} at {off}: {len(data)} of {n}")
                with open(os.path.join(dest, o.key) + ".part", "r+b") as f:
                    f.seek(off)
                    f.write(data)
                with lock:
                    moved[0] += n
                return
            except Exception as e:   # retried; the last one is raised
                err = e
                time.sleep(0.05 * (attempt + 1))
        raise err

    jobs = [(o, off, n) for o in todo for off, n in _ranges(o.size, chunk_bytes)]
    with ThreadPoolExecutor(max_workers=max(1, workers)) as ex:
        list(ex.map(fetch, jobs))
    for o in todo:
        os.replace(os.path.join(dest, o.key) + ".part", os.path.join(dest, o.key))
    tmp = os.path.join(dest, _MARKER + ".tmp")
    with open(tmp, "w") as f:
        json.dump({"files": {o.key: [o.size, o.etag] for o in objs}, "prefix": prefix}, f)
    os.replace(tmp, os.path.join(dest, _MARKER))
    return {"files": len(objs), "bytes": moved[0], "skipped": skipped, "seconds": time.monotonic() - t0}


def _recorded_etag(dest: str, key: str) -> str:
    try:
        return json.load(open(os.path.join(dest, _MARKER)))["files"][key][1]
    except (OSError, ValueError, KeyError, IndexError):
        return ""


def wait_for_complete(dest: str, timeout_s: float = 3600.0, poll_s: float = 0.5) -> None:
    """What the non-downloading ranks of a node do while local rank 0 fetches."""
    end = time.monotonic() + timeout_s
    while not is_complete(dest):
        if time.monotonic() > end:
            raise TimeoutError(f"model files under {dest} did not complete within {timeout_s:.0f} s")
        time.sleep(poll_s)


def resolve_model_path(uri: str, cache_dir: Optional[str] = None, local_rank: int = 0, store: Optional[ObjectStore] = None,
                       patterns: Sequence[str] = DEFAULT_PATTERNS, timeout_s: float = 3600.0, **kw) -> str:
    """Local directory holding the model named by ``uri``.  Local paths are returned as they are; remote ones are
    mirrored under ``cache_dir`` by local rank 0 of each node while the other local ranks wait for the marker."""
    scheme, bucket, path = parse_model_uri(uri)
    if scheme == "local":
        if not os.path.isdir(path):
            raise FileNotFoundError(path)
        return path
    cache_dir = cache_dir or os.environ.get("RELAX_B200_MODEL_CACHE", os.path.expanduser("~/.cache/relax_b200/models"))
    dest = os.path.join(cache_dir, cache_subdir(uri))
    if local_rank == 0:
        if store is None:
            store = DirStore("/") if scheme == "file" else S3Store(bucket)
        download_model(store, path, dest, patterns, **kw)
    else:
        wait_for_complete(dest, timeout_s)
    return dest


def warm_page_cache(path: str, patterns: Sequence[str] = ("*.safetensors",), block: int = 16 << 20, workers: int = 4) -> int:
    """Read the weight files once, sequentially per file, so that the ranks which open them next are served from
    the page cache instead of each hitting the disk (relax/utils/hf_page_cache.py).  Returns the bytes read."""
    files = [os.path.join(d, f) for d, _, fs in os.walk(path) for f in fs if any(fnmatch.fnmatch(f, p) for p in patterns)]

    def rd(p):
        n = 0
        with open(p, "rb", buffering=0) as f:
            while True:
                b = f.read(block)
                if not b:
                    return n
                n += len(b)

    with ThreadPoolExecutor(max_workers=max(1, workers)) as ex:
        return sum(ex.map(rd, sorted(files)))

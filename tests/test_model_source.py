"""Model source resolution and the object-store mirror (CPU; a directory stands in for the bucket)."""
import os
import threading

import pytest

from relax_b200.utils import model_source as MS


def _bucket(tmp_path):
    root = tmp_path / "bucket" / "models" / "m1"
    root.mkdir(parents=True)
    (root / "config.json").write_text('{"a": 1}')
    (root / "model-00001.safetensors").write_bytes(os.urandom(300_000))
    (root / "model-00002.safetensors").write_bytes(os.urandom(70_001))
    (root / "empty.txt").write_bytes(b"")
    (root / "notes.bin").write_bytes(b"skip me")
    return MS.DirStore(str(tmp_path / "bucket")), "models/m1", root


def test_uri_parsing():
    assert MS.parse_model_uri("s3://bkt/a/b/") == ("s3", "bkt", "a/b")
    assert MS.parse_model_uri("file:///x/y") == ("file", "", "/x/y")
    assert MS.parse_model_uri("/x/y") == ("local", "", "/x/y")
    with pytest.raises(ValueError):
        MS.parse_model_uri("gs://b/x")
    with pytest.raises(ValueError):
        MS.parse_model_uri("s3:///x")
    assert MS.cache_subdir("s3://bkt/a/b") == "s3_bkt_a_b"


def test_mirror_resume_and_marker(tmp_path):
    store, prefix, root = _bucket(tmp_path)
    dest = str(tmp_path / "cache")
    st = MS.download_model(store, prefix, dest, workers=4, chunk_bytes=65536)
    assert st["files"] == 4 and st["bytes"] == 300_000 + 70_001 + 8 and MS.is_complete(dest)
    assert not os.path.exists(os.path.join(dest, "notes.bin"))
    for n in ("config.json", "model-00001.safetensors", "model-00002.safetensors", "empty.txt"):
        assert open(os.path.join(dest, n), "rb").read() == (root / n).read_bytes()
    again = MS.download_model(store, prefix, dest)
    assert again["bytes"] == 0 and again["skipped"] == 4
    # a damaged copy (wrong size, marker gone) is re-fetched; intact files are kept
    os.remove(os.path.join(dest, ".complete.json"))
    with open(os.path.join(dest, "model-00002.safetensors"), "wb") as f:
        f.write(b"x")
    fix = MS.download_model(store, prefix, dest, chunk_bytes=1 << 20)
    assert fix["skipped"] == 3 and fix["bytes"] == 70_001 and MS.is_complete(dest)
    # the source changed: the marker no longer matches
    (root / "config.json").write_text('{"a": 22}')
    assert not MS.is_complete(dest, MS._select(store.list(prefix), MS.DEFAULT_PATTERNS))
    MS.download_model(store, prefix, dest)
    assert open(os.path.join(dest, "config.json")).read() == '{"a": 22}'


def test_transient_errors_are_retried_and_hard_ones_leave_no_marker(tmp_path):
    store, prefix, _ = _bucket(tmp_path)

    class Flaky(MS.DirStore):
        def __init__(self, root, fail):
            super().__init__(root)
            self.fail, self.lock = fail, threading.Lock()

        def read(self, prefix, key, off, n):
            with self.lock:
                if self.fail > 0:
                    self.fail -= 1
                    raise IOError("connection reset")
            return super().read(prefix, key, off, n)

    ok = MS.download_model(Flaky(store.root, 2), prefix, str(tmp_path / "c1"), workers=1, chunk_bytes=100_000)
    assert ok["files"] == 4
    with pytest.raises(IOError):
        MS.download_model(Flaky(store.root, 10 ** 6), prefix, str(tmp_path / "c2"), workers=2, retries=2)
    assert not MS.is_complete(str(tmp_path / "c2"))


def test_resolve_and_wait(tmp_path):
    store, prefix, root = _bucket(tmp_path)
    assert MS.resolve_model_path(str(root)) == str(root)
    with pytest.raises(FileNotFoundError):
        MS.resolve_model_path(str(tmp_path / "nope"))
    cache = str(tmp_path / "cache")
    got = {}
    waiter = threading.Thread(target=lambda: got.setdefault("p", MS.resolve_model_path("s3://bucket/models/m1", cache, local_rank=1, timeout_s=20)))
    waiter.start()
    p0 = MS.resolve_model_path("s3://bucket/models/m1", cache, local_rank=0, store=store, patterns=MS.DEFAULT_PATTERNS)
    waiter.join(20)
    assert got["p"] == p0 and os.path.exists(os.path.join(p0, "config.json"))
    with pytest.raises(TimeoutError):
        MS.wait_for_complete(str(tmp_path / "never"), timeout_s=0.2, poll_s=0.05)
    assert MS.warm_page_cache(p0) == 370_001
    # file:// goes through the same mirror
    p1 = MS.resolve_model_path("file://" + str(root), cache)
    assert p1 != p0 and MS.is_complete(p1)


def test_s3_store_against_a_fake_client():
    class Body:
        def __init__(self, b): self.b = b
        def read(self): return self.b

    class Fake:
        data = {"m/a.json": b"0123456789", "m/sub/b.safetensors": b"abcdef", "m/": b""}

        def list_objects_v2(self, Bucket, Prefix, ContinuationToken=None):
            keys = sorted(k for k in self.data if k.startswith(Prefix))
            if ContinuationToken is None:
                return {"Contents": [{"Key": k, "Size": len(self.data[k]), "ETag": '"e"'} for k in keys[:2]], "NextContinuationToken": "t"}
            return {"Contents": [{"Key": k, "Size": len(self.data[k]), "ETag": '"e"'} for k in keys[2:]]}

        def get_object(self, Bucket, Key, Range):
            lo, hi = map(int, Range.split("=")[1].split("-"))
            return {"Body": Body(self.data[Key][lo:hi + 1])}

    s = MS.S3Store("bkt", client=Fake())
    objs = s.list("m")
    assert [(o.key, o.size, o.etag) for o in objs] == [("a.json", 10, "e"), ("sub/b.safetensors", 6, "e")]
    assert s.read("m", "a.json", 2, 4) == b"2345"

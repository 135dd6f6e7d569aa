"""Dataset download with a checksummed cache (crates/data/src/fetch.rs).

Environment: RUSTRAL_CACHE_DIR (default ~/.cache/rustral), RUSTRAL_DATASET_OFFLINE=1 (never touch the network: a
missing file is an error), RUSTRAL_DATASET_SKIP_CHECKSUM=1.  Downloads go to `<name>.partial` and are renamed
once the SHA-256 matches."""
from __future__ import annotations

import gzip
import hashlib
import os
import shutil
import urllib.request


class FetchError(RuntimeError):
    pass


def cache_root() -> str:
    root = os.environ.get("RUSTRAL_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "rustral")
    os.makedirs(root, exist_ok=True)
    return root


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def fetch_url(url: str, sha256: str | None, subdir: str, filename: str | None = None) -> str:
    d = os.path.join(cache_root(), subdir)
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, filename or url.rsplit("/", 1)[-1])
    skip = os.environ.get("RUSTRAL_DATASET_SKIP_CHECKSUM") == "1"
    if os.path.exists(path):
        if sha256 and not skip and _sha256(path) != sha256:
            raise FetchError(f"checksum mismatch for cached file {path}")
        return path
    if os.environ.get("RUSTRAL_DATASET_OFFLINE") == "1":
        raise FetchError(f"{path} is not cached and RUSTRAL_DATASET_OFFLINE=1 forbids downloading {url}")
    tmp = path + ".partial"
    try:
        with urllib.request.urlopen(url, timeout=60) as r, open(tmp, "wb") as f:
            shutil.copyfileobj(r, f)
    except OSError as e:
        raise FetchError(f"download of {url} failed: {e}") from e
    if sha256 and not skip and _sha256(tmp) != sha256:
        os.remove(tmp)
        raise FetchError(f"checksum mismatch for {url}")
    os.replace(tmp, path)
    return path


def ungzip(src: str, dst: str) -> str:
    with gzip.open(src, "rb") as f, open(dst + ".partial", "wb") as g:
        shutil.copyfileobj(f, g)
    os.replace(dst + ".partial", dst)
    return dst


def fnv1a64(data: bytes) -> int:
    """FNV-1a, the dataset fingerprint written into run manifests (crates/runtime/examples/wikitext2_lm.rs:618-656)."""
    h = 0xCBF29CE484222325
    for b in data:
        h ^= b
        h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h

"""Local cache for model archives and vocabularies.

Counterpart of the reference's ``examples/BertPretraining/file_utils.py`` (``cached_path`` :87-114,
``url_to_filename`` :43-58, ``filename_to_url`` :61-84, ``get_from_cache`` :184-237), which
downloads from HTTP / S3 into ``~/.pytorch_pretrained_bert``.  The machines this library is built
for have no network, so the cache is local-first: a path that exists is returned as it is, a URL
is looked up in the cache directory under a file name derived from the URL (and ETag), and only
when it is absent there is a download attempted (``urllib``; S3 URLs are not supported) - which
fails with a clear message when the machine is offline.  ``add_to_cache`` puts a file that was
brought in by other means under the name a later ``cached_path(url)`` will look for.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import tempfile
from typing import Optional, Tuple
from urllib.parse import urlparse

CACHE_DIR = os.environ.get("CONEF_CACHE", os.path.join(os.path.expanduser("~"), ".cache", "conef_b200"))


def url_to_filename(url: str, etag: Optional[str] = None) -> str:
    """sha256(url) [+ '.' + sha256(etag)]: the same URL with a new ETag is a new file."""
    name = hashlib.sha256(url.encode("utf-8")).hexdigest()
    if etag:
        name += "." + hashlib.sha256(etag.encode("utf-8")).hexdigest()
    return name


def filename_to_url(filename: str, cache_dir: Optional[str] = None) -> Tuple[str, Optional[str]]:
    """(url, etag) recorded next to a cached file."""
    cache_dir = cache_dir or CACHE_DIR
    path = os.path.join(cache_dir, filename)
    meta = path + ".json"
    if not os.path.exists(path):
        raise FileNotFoundError(f"file {path} not found")
    if not os.path.exists(meta):
        raise FileNotFoundError(f"file {meta} not found")
    with open(meta, encoding="utf-8") as f:
        d = json.load(f)
    return d["url"], d.get("etag")


def add_to_cache(url: str, local_file: str, etag: Optional[str] = None, cache_dir: Optional[str] = None) -> str:
    """Copy ``local_file`` into the cache as the content of ``url``; returns the cached path."""
    cache_dir = cache_dir or CACHE_DIR
    os.makedirs(cache_dir, exist_ok=True)
    path = os.path.join(cache_dir, url_to_filename(url, etag))
    fd, tmp = tempfile.mkstemp(dir=cache_dir)
    os.close(fd)
    shutil.copyfile(local_file, tmp)
    os.replace(tmp, path)
    with open(path + ".json", "w", encoding="utf-8") as f:
        json.dump({"url": url, "etag": etag}, f)
    return path


def _find_cached(url: str, cache_dir: str) -> Optional[str]:
    prefix = url_to_filename(url)
    if not os.path.isdir(cache_dir):
        return None
    hits = sorted(n for n in os.listdir(cache_dir) if n.startswith(prefix) and not n.endswith(".json"))
    return os.path.join(cache_dir, hits[-1]) if hits else None


def get_from_cache(url: str, cache_dir: Optional[str] = None) -> str:
    cache_dir = cache_dir or CACHE_DIR
    hit = _find_cached(url, cache_dir)
    if hit is not None:
        return hit
    if urlparse(url).scheme == "s3":
        raise EnvironmentError(f"{url}: S3 downloads are not supported; fetch the file and add_to_cache() it")
    import urllib.error
    import urllib.request
    try:
        with urllib.request.urlopen(url, timeout=30) as resp:
            etag = resp.headers.get("ETag")
            os.makedirs(cache_dir, exist_ok=True)
            fd, tmp = tempfile.mkstemp(dir=cache_dir)
            with os.fdopen(fd, "wb") as out:
                shutil.copyfileobj(resp, out)
    except (urllib.error.URLError, OSError) as exc:
        raise EnvironmentError(f"{url} is not in the cache ({cache_dir}) and could not be downloaded: {exc}") from exc
    path = os.path.join(cache_dir, url_to_filename(url, etag))
    os.replace(tmp, path)
    with open(path + ".json", "w", encoding="utf-8") as f:
        json.dump({"url": url, "etag": etag}, f)
    return path


def cached_path(url_or_filename, cache_dir: Optional[str] = None) -> str:
    """A local path for ``url_or_filename``: existing paths pass through, URLs go through the cache."""
    s = os.fspath(url_or_filename)
    scheme = urlparse(s).scheme
    if scheme in ("http", "https", "s3"):
        return get_from_cache(s, cache_dir)
    if os.path.exists(s):
        return s
    if scheme == "":
        raise EnvironmentError(f"file {s} not found")
    raise ValueError(f"unable to parse {s} as a URL or as a local path")

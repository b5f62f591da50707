"""Download helpers with the reference's names (python/fastdeploy/download.py:30-230:
``download``, ``download_and_decompress``, ``download_model``, ``get_model_list``). This build runs without network
access: a request is served from a local directory of pre-fetched files (``FASTDEPLOY_MODEL_CACHE``,
default ``~/.fastdeploy/models``) when the file is there and fails with a clear error otherwise, and
``file://`` / plain paths are copied. Archives are unpacked with the standard library."""
from __future__ import annotations

import os
import shutil
import tarfile
import zipfile
from typing import Optional

CACHE_ENV = "FASTDEPLOY_MODEL_CACHE"


def cache_dir() -> str:
    return os.environ.get(CACHE_ENV, os.path.join(os.path.expanduser("~"), ".fastdeploy", "models"))


def download(url: str, path: Optional[str] = None, rename: Optional[str] = None, show_progress: bool = True) -> str:
    name = rename or os.path.basename(url.split("?")[0])
    dst_dir = path or "."
    os.makedirs(dst_dir, exist_ok=True)
    dst = os.path.join(dst_dir, name)
    src = url[len("file://"):] if url.startswith("file://") else url
    if os.path.exists(src):
        if os.path.abspath(src) != os.path.abspath(dst):
            shutil.copyfile(src, dst)
        return dst
    cached = os.path.join(cache_dir(), os.path.basename(url.split("?")[0]))
    if os.path.exists(cached):
        shutil.copyfile(cached, dst)
        return dst
    raise RuntimeError(f"cannot fetch {url}: no network access in this build; place the file at {cached}")


def decompress(fname: str, path: Optional[str] = None) -> str:
    out = path or os.path.dirname(os.path.abspath(fname))
    if tarfile.is_tarfile(fname):
        with tarfile.open(fname) as t:
            t.extractall(out, filter="data")
            top = t.getnames()[0].split("/")[0] if t.getnames() else ""
    elif zipfile.is_zipfile(fname):
        with zipfile.ZipFile(fname) as z:
            z.extractall(out)
            top = z.namelist()[0].split("/")[0] if z.namelist() else ""
    else:
        raise ValueError(f"unsupported archive: {fname}")
    return os.path.join(out, top)


def download_and_decompress(url: str, path: str = ".", rename: Optional[str] = None) -> str:
    return decompress(download(url, path, rename), path)


def download_model(name: str, path: Optional[str] = None, format: Optional[str] = None, version: Optional[str] = None) -> str:
    """Looks the model up in the local cache (``<cache>/<name>[.tgz|.tar|.zip]``)."""
    base = os.path.join(cache_dir(), name)
    if os.path.isdir(base):
        return base
    for ext in (".tgz", ".tar.gz", ".tar", ".zip"):
        if os.path.exists(base + ext):
            return decompress(base + ext, path or cache_dir())
    raise RuntimeError(f"model {name!r} is not in {cache_dir()} and there is no network access in this build")


def get_model_list(category: Optional[str] = None) -> dict:
    """The models :func:`download_model` can serve, by category (python/fastdeploy/download.py:216-237). The reference
    asks its model hub; here the list is what the local cache holds: ``<cache>/index.json`` (``{category: [{"name": ...,
    "format": ..., "version": ...}]}``) when present, else every directory or archive of the cache under the category
    ``"local"``."""
    import json
    root = cache_dir()
    index = os.path.join(root, "index.json")
    if os.path.exists(index):
        with open(index) as f:
            listing = json.load(f)
    else:
        names = set()
        for entry in sorted(os.listdir(root)) if os.path.isdir(root) else []:
            stem = entry
            for ext in (".tar.gz", ".tgz", ".tar", ".zip"):
                if entry.endswith(ext):
                    stem = entry[:-len(ext)]
            if stem != "index.json":
                names.add(stem)
        listing = {"local": [{"name": n} for n in sorted(names)]} if names else {}
    if category is None:
        return listing
    if category in listing:
        return {category: listing[category]}
    raise ValueError(f"No pretrained model in category {category} can be downloaded now.")

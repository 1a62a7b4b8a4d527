"""Model registry client and local model cache in the Ollama layout.

Parity with ``crates/runtime/src/ollama.rs:12-249``: ``name[:tag]`` parsing (default tag ``latest``), Docker-v2
manifest at ``registry.ollama.ai/v2/library/{name}/manifests/{tag}``, the layer whose media type contains
"model" is the GGUF blob, blobs cached as ``<cache>/ollama/blobs/sha256_<digest>.gguf``, ``list_cached`` /
``delete_cached`` / ``get_cached_path`` / ``is_cached``, progress callback every 10 MB.  The cache root honours
``UNILLM_CACHE_DIR`` (documented but not implemented in the reference).  Downloads resume from a partial
file with an HTTP range request and verify the sha256 digest.  Machines without network (the GPU boxes) use
``register_local`` / the cache only; ``pull`` then raises ``NetworkError`` unless the model is cached.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

from .types import FileSystemError, NetworkError

OLLAMA_REGISTRY = "https://registry.ollama.ai"
PROGRESS_EVERY = 10 * 1024 * 1024


@dataclass
class ModelInfo:
    name: str
    tag: str
    digest: str
    size: int
    path: Optional[str] = None


def parse_model_name(model: str) -> Tuple[str, str]:
    name, _, tag = model.partition(":")
    return name, (tag or "latest")


def default_cache_dir() -> str:
    root = os.environ.get("UNILLM_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "unillm")
    return os.path.join(root, "ollama")


class OllamaRegistry:
    def __init__(self, cache_dir: Optional[str] = None, registry: str = OLLAMA_REGISTRY):
        self.cache_dir = cache_dir or default_cache_dir()
        self.registry = registry.rstrip("/")
        os.makedirs(os.path.join(self.cache_dir, "blobs"), exist_ok=True)
        self._index_path = os.path.join(self.cache_dir, "index.json")

    @staticmethod
    def new() -> "OllamaRegistry":
        return OllamaRegistry()

    # ---- cache ----
    def _index(self) -> Dict[str, dict]:
        if os.path.isfile(self._index_path):
            try:
                return json.loads(open(self._index_path).read())
            except json.JSONDecodeError:
                return {}
        return {}

    def _save_index(self, idx: Dict[str, dict]) -> None:
        tmp = self._index_path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(idx, f, indent=1)
        os.replace(tmp, self._index_path)

    def blob_path(self, digest: str) -> str:
        return os.path.join(self.cache_dir, "blobs", digest.replace(":", "_") + ".gguf")

    def get_cached_path(self, model: str) -> Optional[str]:
        name, tag = parse_model_name(model)
        e = self._index().get(f"{name}:{tag}")
        if e and os.path.isfile(e["path"]):
            return e["path"]
        return None

    def is_cached(self, model: str) -> bool:
        return self.get_cached_path(model) is not None

    def list_cached(self) -> List[ModelInfo]:
        out = []
        for key, e in sorted(self._index().items()):
            if os.path.isfile(e["path"]):
                n, t = parse_model_name(key)
                out.append(ModelInfo(n, t, e.get("digest", ""), os.path.getsize(e["path"]), e["path"]))
        return out

    def delete_cached(self, model: str) -> bool:
        name, tag = parse_model_name(model)
        idx = self._index()
        e = idx.pop(f"{name}:{tag}", None)
        if e is None:
            return False
        if os.path.isfile(e["path"]) and not any(x["path"] == e["path"] for x in idx.values()):
            os.remove(e["path"])
        self._save_index(idx)
        return True

    def register_local(self, model: str, gguf_path: str, copy: bool = False) -> str:
        """Adds an existing GGUF file to the cache under ``name:tag`` (offline installs)."""
        if not os.path.isfile(gguf_path):
            raise FileSystemError(f"no such file: {gguf_path}")
        name, tag = parse_model_name(model)
        h = hashlib.sha256()
        with open(gguf_path, "rb") as f:
            for chunk in iter(lambda: f.read(1 << 20), b""):
                h.update(chunk)
        digest = "sha256:" + h.hexdigest()
        path = gguf_path
        if copy:
            path = self.blob_path(digest)
            if not os.path.isfile(path):
                shutil.copyfile(gguf_path, path)
        idx = self._index()
        idx[f"{name}:{tag}"] = {"path": os.path.abspath(path), "digest": digest}
        self._save_index(idx)
        return path

    # ---- network ----
    def get_manifest(self, model: str) -> dict:
        import urllib.error
        import urllib.request

        name, tag = parse_model_name(model)
        url = f"{self.registry}/v2/library/{name}/manifests/{tag}"
        req = urllib.request.Request(url, headers={"Accept": "application/vnd.docker.distribution.manifest.v2+json"})
        try:
            with urllib.request.urlopen(req, timeout=15) as r:
                return json.loads(r.read().decode("utf-8"))
        except (urllib.error.URLError, OSError) as e:
            raise NetworkError(f"cannot reach {url}: {e}")

    @staticmethod
    def model_layer(manifest: dict) -> dict:
        for layer in manifest.get("layers", []):
            if "model" in layer.get("mediaType", ""):
                return layer
        raise NetworkError("manifest has no model layer")

    def get_model_info(self, model: str) -> ModelInfo:
        name, tag = parse_model_name(model)
        layer = self.model_layer(self.get_manifest(model))
        return ModelInfo(name, tag, layer["digest"], int(layer.get("size", 0)), self.get_cached_path(model))

    def pull(self, model: str, progress: Optional[Callable[[int, int], None]] = None) -> str:
        cached = self.get_cached_path(model)
        if cached:
            return cached
        import urllib.error
        import urllib.request

        name, tag = parse_model_name(model)
        layer = self.model_layer(self.get_manifest(model))
        digest, size = layer["digest"], int(layer.get("size", 0))
        dest = self.blob_path(digest)
        part = dest + ".part"
        have = os.path.getsize(part) if os.path.isfile(part) else 0
        url = f"{self.registry}/v2/library/{name}/blobs/{digest}"
        req = urllib.request.Request(url, headers={"Range": f"bytes={have}-"} if have else {})
        try:
            with urllib.request.urlopen(req, timeout=60) as r, open(part, "ab" if have else "wb") as f:
                done, mark = have, have
                while True:
                    chunk = r.read(1 << 20)
                    if not chunk:
                        break
                    f.write(chunk)
                    done += len(chunk)
                    if progress and done - mark >= PROGRESS_EVERY:
                        progress(done, size)
                        mark = done
        except (urllib.error.URLError, OSError) as e:
            raise NetworkError(f"download of {model} failed: {e}")
        h = hashlib.sha256()
        with open(part, "rb") as f:
            for chunk in iter(lambda: f.read(1 << 20), b""):
                h.update(chunk)
        if digest.startswith("sha256:") and h.hexdigest() != digest[7:]:
            os.remove(part)
            raise NetworkError(f"digest mismatch for {model}")
        os.replace(part, dest)
        idx = self._index()
        idx[f"{name}:{tag}"] = {"path": dest, "digest": digest}
        self._save_index(idx)
        return dest

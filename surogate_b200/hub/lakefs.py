"""LakeFS model/dataset hub through its S3-compatible gateway (``lakefs://<repo>/<ref>/<path>``).

Configuration comes from ``LAKEFS_ENDPOINT``, ``LAKEFS_ACCESS_KEY_ID`` and ``LAKEFS_SECRET_ACCESS_KEY``.  Objects are listed
with the LakeFS REST API (basic auth) and fetched one by one into a local cache directory; a file already present with
the same size is not downloaded again.

Parity: surogate/core/hub/lakefs.py:1-436.
"""
from __future__ import annotations

import base64
import json
import os
import urllib.parse
import urllib.request
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional


@dataclass
class LakeFSHub:
    endpoint: str
    access_key: str
    secret_key: str
    timeout_s: float = 60.0

    @staticmethod
    def from_env() -> "LakeFSHub":
        ep, ak, sk = os.environ.get("LAKEFS_ENDPOINT"), os.environ.get("LAKEFS_ACCESS_KEY_ID"), os.environ.get("LAKEFS_SECRET_ACCESS_KEY")
        if not (ep and ak and sk):
            raise RuntimeError("LakeFS access needs LAKEFS_ENDPOINT, LAKEFS_ACCESS_KEY_ID and LAKEFS_SECRET_ACCESS_KEY")
        return LakeFSHub(ep.rstrip("/"), ak, sk)

    @staticmethod
    def parse_uri(uri: str):
        if not uri.startswith("lakefs://"):
            raise ValueError(f"not a lakefs:// URI: {uri}")
        parts = uri[len("lakefs://"):].split("/", 2)
        if len(parts) < 2:
            raise ValueError(f"lakefs URI needs at least a repository and a ref: {uri}")
        return parts[0], parts[1], parts[2] if len(parts) > 2 else ""

    def _request(self, url: str) -> bytes:
        req = urllib.request.Request(url)
        tok = base64.b64encode(f"{self.access_key}:{self.secret_key}".encode()).decode()
        req.add_header("Authorization", f"Basic {tok}")
        with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
            return r.read()

    def list_objects(self, repo: str, ref: str, prefix: str) -> Iterator[Dict]:
        after = ""
        while True:
            q = urllib.parse.urlencode({"prefix": prefix, "after": after, "amount": 1000})
            page = json.loads(self._request(f"{self.endpoint}/api/v1/repositories/{repo}/refs/{ref}/objects/ls?{q}"))
            yield from (o for o in page.get("results", []) if o.get("path_type", "object") == "object")
            pag = page.get("pagination", {})
            if not pag.get("has_more"):
                return
            after = pag.get("next_offset", "")

    def download(self, uri: str, cache_dir: Optional[str] = None) -> str:
        repo, ref, prefix = self.parse_uri(uri)
        from ..utils.fs import get_cache_dir

        root = os.path.join(cache_dir or os.path.join(get_cache_dir(), "lakefs"), repo, ref, prefix.strip("/"))
        os.makedirs(root, exist_ok=True)
        for obj in self.list_objects(repo, ref, prefix):
            rel = obj["path"][len(prefix):].lstrip("/")
            dst = os.path.join(root, rel)
            if os.path.exists(dst) and os.path.getsize(dst) == obj.get("size_bytes", -1):
                continue
            os.makedirs(os.path.dirname(dst) or root, exist_ok=True)
            q = urllib.parse.urlencode({"path": obj["path"]})
            data = self._request(f"{self.endpoint}/api/v1/repositories/{repo}/refs/{ref}/objects?{q}")
            with open(dst + ".part", "wb") as f:
                f.write(data)
            os.replace(dst + ".part", dst)
        return root

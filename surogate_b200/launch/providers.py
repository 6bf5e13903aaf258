"""Saved compute targets: SSH GPU servers, Modal workspaces, dstack cloud backends.

Only non-secret metadata lives in this store (label, host, backend, region, preferred GPU).  Credentials go to each tool's own
store when the target is connected (Modal: its token file; SSH: the user's keys; dstack: its server config, ``dstack.py``), so no
key is duplicated into a file this package owns.

Parity: jackalope/src/providers.ts.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional

KINDS = ("ssh", "modal", "dstack")

# what each dstack backend needs in order to connect: (key, label, secret, may be a file path or pasted contents)
DSTACK_BACKEND_FIELDS: Dict[str, List[tuple]] = {
    "runpod": [("api_key", "API key", True, False)],
    "lambda": [("api_key", "API key", True, False)],
    "vastai": [("api_key", "API key", True, False)],
    "aws": [("access_key", "access key id", False, False), ("secret_key", "secret access key", True, False)],
    "gcp": [("project_id", "project id", False, False), ("data_file", "service-account JSON (path or contents)", True, True)],
    "azure": [("tenant_id", "tenant id", False, False), ("subscription_id", "subscription id", False, False), ("client_id", "client id", False, False),
              ("client_secret", "client secret", True, False)],
    "nebius": [("service_account_id", "service account id", False, False), ("public_key_id", "public key id", False, False),
               ("private_key_file", "private key (path or contents)", True, True)],
    "oci": [("user", "user OCID", False, False), ("tenancy", "tenancy OCID", False, False), ("region", "region", False, False),
            ("fingerprint", "fingerprint", False, False), ("key_file", "private key (path or contents)", True, True)],
}


@dataclass
class ProviderRecord:
    id: str
    kind: str
    label: str
    host: Optional[str] = None         # ssh: user@host[:port] or an alias of the user's ssh config
    workspace: Optional[str] = None    # modal
    environment: Optional[str] = None  # modal
    backend: Optional[str] = None      # dstack: which cloud
    region: Optional[str] = None       # dstack
    gpu: Optional[str] = None          # preferred GPU, "B200" or "B200:8"
    added_at: str = ""


def provider_id(kind: str, key: str) -> str:
    """Stable id from kind + key (host / workspace / backend): adding the same target again updates it in place.  The key is kept
    as typed (trimmed only): ids are JSON strings, never paths, and folding characters would merge distinct hosts."""
    return f"{kind}:{key.strip() or 'default'}"


class ProviderStore:
    def __init__(self, path: Optional[str] = None):
        self.path = path or os.path.join(os.path.expanduser("~"), ".surogate-watch", "providers.json")

    def load(self) -> List[ProviderRecord]:
        try:
            with open(self.path) as f:
                raw = json.load(f)
        except (OSError, ValueError):
            return []
        known = set(ProviderRecord.__dataclass_fields__)
        out = []
        for p in raw if isinstance(raw, list) else []:
            if isinstance(p, dict) and p.get("id") and p.get("kind") in KINDS and p.get("label"):
                out.append(ProviderRecord(**{k: v for k, v in p.items() if k in known}))
        return out

    def _write(self, records: List[ProviderRecord]) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump([asdict(r) for r in records], f, indent=2)
        os.replace(tmp, self.path)

    def save(self, rec: ProviderRecord) -> List[ProviderRecord]:
        """Insert or update (matched by id); the newest entry sorts last."""
        if rec.kind not in KINDS:
            raise ValueError(f"provider kind must be one of {KINDS}, got {rec.kind!r}")
        if rec.kind == "dstack" and rec.backend and rec.backend not in DSTACK_BACKEND_FIELDS:
            raise ValueError(f"unknown dstack backend {rec.backend!r} ({', '.join(DSTACK_BACKEND_FIELDS)})")
        rec.added_at = rec.added_at or time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())
        records = [r for r in self.load() if r.id != rec.id] + [rec]
        self._write(records)
        return records

    def delete(self, pid: str) -> List[ProviderRecord]:
        records = [r for r in self.load() if r.id != pid]
        self._write(records)
        return records

    def get(self, pid: str) -> Optional[ProviderRecord]:
        return next((r for r in self.load() if r.id == pid), None)

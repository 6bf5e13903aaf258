"""Model / dataset download: local paths pass through, HuggingFace Hub and LakeFS are used when reachable.

``download_model("Qwen/Qwen3-8B")`` returns a local directory.  Resolution order: an existing path; the HuggingFace
cache (``HF_HOME``), which works offline; a Hub download through ``huggingface_hub`` (honours ``HF_TOKEN``,
``HF_ENDPOINT``, ``HF_HUB_OFFLINE``); a ``lakefs://repo/ref/path`` URI through the LakeFS S3 gateway.

Parity: surogate/core/hub/huggingface.py, lakefs.py:1-436, model_info.py.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Sequence

WEIGHT_PATTERNS = ["*.safetensors", "*.json", "*.jinja", "tokenizer.model", "*.txt"]


class HubError(RuntimeError):
    pass


def _hf_cached(repo_id: str, revision: Optional[str]) -> Optional[str]:
    try:
        from huggingface_hub import snapshot_download

        return snapshot_download(repo_id, revision=revision, local_files_only=True, allow_patterns=WEIGHT_PATTERNS)
    except Exception:  # noqa: BLE001
        return None


def download_model(name: str, revision: Optional[str] = None, cache_dir: Optional[str] = None, token: Optional[str] = None) -> str:
    if os.path.exists(name):
        return name
    if name.startswith("lakefs://"):
        from .lakefs import LakeFSHub

        return LakeFSHub.from_env().download(name, cache_dir)
    cached = _hf_cached(name, revision)
    if cached:
        return cached
    if os.environ.get("HF_HUB_OFFLINE") == "1":
        raise HubError(f"model '{name}' is not a local path, not in the HuggingFace cache, and HF_HUB_OFFLINE=1")
    try:
        from huggingface_hub import snapshot_download

        return snapshot_download(name, revision=revision, cache_dir=cache_dir, token=token or os.environ.get("HF_TOKEN"), allow_patterns=WEIGHT_PATTERNS)
    except Exception as e:  # noqa: BLE001
        raise HubError(f"cannot fetch model '{name}': {type(e).__name__}: {e}") from e


def download_dataset(name: str, revision: Optional[str] = None, cache_dir: Optional[str] = None) -> str:
    if os.path.exists(name):
        return name
    try:
        from huggingface_hub import snapshot_download

        return snapshot_download(name, repo_type="dataset", revision=revision, cache_dir=cache_dir, token=os.environ.get("HF_TOKEN"))
    except Exception as e:  # noqa: BLE001
        raise HubError(f"cannot fetch dataset '{name}': {type(e).__name__}: {e}") from e


def model_info(model_dir: str) -> Dict[str, Any]:
    """Size / architecture summary of a local model directory (parameter count from the safetensors headers, no weights read)."""
    from ..models.registry import describe_config

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    info = describe_config(cfg)
    n_params, nbytes, files = 0, 0, []
    for fn in sorted(os.listdir(model_dir)):
        if fn.endswith(".safetensors"):
            path = os.path.join(model_dir, fn)
            files.append(fn)
            with open(path, "rb") as f:
                hlen = int.from_bytes(f.read(8), "little")
                header = json.loads(f.read(hlen))
            for k, v in header.items():
                if k == "__metadata__":
                    continue
                n = 1
                for d in v["shape"]:
                    n *= d
                n_params += n
                nbytes += v["data_offsets"][1] - v["data_offsets"][0]
    info.update(num_parameters=n_params, weight_bytes=nbytes, weight_files=files)
    return info


def try_login(token: Optional[str] = None) -> bool:
    """True when the hub accepts the token (``token``, else ``HF_TOKEN``, else the stored login)."""
    try:
        from huggingface_hub import HfApi

        HfApi().whoami(token=token or os.environ.get("HF_TOKEN"))
        return True
    except Exception:  # noqa: BLE001 - not installed, offline, or refused
        return False


def push_to_hub(repo_id: str, folder_path: str, path_in_repo: Optional[str] = None, commit_message: Optional[str] = None, private: bool = False,
                revision: Optional[str] = None, ignore_patterns: Optional[Sequence[str]] = None, token: Optional[str] = None, api=None) -> Any:
    """Upload a directory (an exported model or adapter) to a model repository, creating it when missing.  ``revision`` ``master`` /
    None means ``main``.  ``api``: an object with ``create_repo`` / ``upload_folder`` (tests inject one; default ``huggingface_hub.HfApi``).
    Parity: surogate/core/hub/huggingface.py (create_model_repo, push_to_hub)."""
    if not os.path.isdir(folder_path):
        raise HubError(f"nothing to upload: {folder_path} is not a directory")
    if api is None:
        try:
            from huggingface_hub import HfApi
        except ImportError as e:
            raise HubError("pushing to the hub needs the `huggingface_hub` package") from e
        api = HfApi()
    token = token or os.environ.get("HF_TOKEN")
    api.create_repo(repo_id, token=token, private=private, exist_ok=True)
    return api.upload_folder(repo_id=repo_id, folder_path=folder_path, path_in_repo=path_in_repo, commit_message=commit_message or f"Upload {os.path.basename(folder_path.rstrip('/'))}",
                             token=token, revision="main" if revision in (None, "master") else revision,
                             ignore_patterns=list(ignore_patterns) if ignore_patterns else ["tokens/*", "step_*", "*.log", "log.jsonl"])

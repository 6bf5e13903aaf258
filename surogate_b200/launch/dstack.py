"""Cloud GPUs through dstack (one open-source CLI that provisions AWS / GCP / Azure / Lambda / Vast / RunPod / Nebius / OCI).

dstack has no "download a file of the run" command, so the run's metrics come back over the task's standard output: the
generated task writes the config on the instance from a here-document (nothing is uploaded), starts the trainer in the background
with its output in a log, and follows the feed file on stdout.  ``dstack apply`` runs attached and streams that output; the pump
keeps the feed records and appends them to the run's local feed.

Credentials: dstack reads backend credentials from its own server config (``~/.dstack/server/config.yml``).  ``configure_backend``
merges one backend into the ``main`` project of that file and leaves every other project and backend as it is; a file this
package cannot parse is refused (after a one-time ``.bak`` copy), never overwritten.

Parity: jackalope/src/dstack.ts.
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
from dataclasses import dataclass
from typing import Any, Dict, Optional

import yaml

from .configs import load_overlaid
from .providers import DSTACK_BACKEND_FIELDS
from .runs import new_run
from .stream import pump_metrics, register

HEREDOC_TAG = "SUROGATE_CONFIG_YAML"


def server_config_path() -> str:
    return os.path.join(os.path.expanduser("~"), ".dstack", "server", "config.yml")


def _file_or_text(key: str, raw: str) -> str:
    """A credential given either as a path or as pasted contents.  A one-line value that looks like a path (``~``, ``/``, ``./``,
    ``../`` at its start) but names no file is a mistyped path: refuse it rather than store the path string as the key."""
    value = raw.strip()
    path = os.path.expanduser(value) if value.startswith("~") else value
    if "\n" not in value and os.path.isfile(path):
        with open(path) as f:
            return f.read().replace("\r", "").rstrip()
    if "\n" not in value and re.match(r"^(~|\.{0,2}/)", value):
        raise ValueError(f"could not read {key}: {value}")
    return value.replace("\r", "").rstrip()


def backend_entry(backend: str, fields: Dict[str, str]) -> Dict[str, Any]:
    """The backend object of dstack's server config for one cloud, from the fields ``DSTACK_BACKEND_FIELDS`` lists."""
    spec = DSTACK_BACKEND_FIELDS.get(backend)
    if spec is None:
        raise ValueError(f"unknown backend {backend}")
    v = {k: (fields.get(k) or "").strip() for k, *_ in spec}
    for k, label, _secret, _file in spec:
        if not v[k]:
            raise ValueError(f"missing {label}")
    if backend in ("runpod", "lambda", "vastai"):
        return {"type": backend, "creds": {"type": "api_key", "api_key": v["api_key"]}}
    if backend == "aws":
        return {"type": "aws", "creds": {"type": "access_key", "access_key": v["access_key"], "secret_key": v["secret_key"]}}
    if backend == "gcp":
        return {"type": "gcp", "project_id": v["project_id"], "creds": {"type": "service_account", "filename": "", "data": _file_or_text("data_file", v["data_file"])}}
    if backend == "azure":
        return {"type": "azure", "tenant_id": v["tenant_id"], "subscription_id": v["subscription_id"],
                "creds": {"type": "client", "client_id": v["client_id"], "client_secret": v["client_secret"]}}
    if backend == "nebius":
        return {"type": "nebius", "creds": {"type": "service_account", "service_account_id": v["service_account_id"], "public_key_id": v["public_key_id"],
                                            "private_key_content": _file_or_text("private_key_file", v["private_key_file"])}}
    if backend == "oci":
        return {"type": "oci", "region": v["region"], "creds": {"type": "client", "user": v["user"], "tenancy": v["tenancy"], "fingerprint": v["fingerprint"],
                                                                "key_content": _file_or_text("key_file", v["key_file"])}}
    raise ValueError(f"unsupported backend {backend}")


def merge_backend(existing: Optional[Dict[str, Any]], backend: str, fields: Dict[str, str]) -> Dict[str, Any]:
    """``existing`` with the backend placed in project ``main``: a backend of the same type is replaced (configuring twice is
    idempotent), everything else is kept.  A ``projects`` / ``backends`` entry of the wrong shape means the file is not what
    this code thinks it is: raise instead of clobbering it."""
    entry = backend_entry(backend, fields)
    doc = existing if isinstance(existing, dict) else {}
    if doc.get("projects") is None:
        doc["projects"] = []
    projects = doc["projects"]
    if not isinstance(projects, list):
        raise ValueError("existing dstack config has a `projects` entry that is not a list; not overwriting")
    main = next((p for p in projects if isinstance(p, dict) and p.get("name") == "main"), None)
    if main is None:
        main = {"name": "main", "backends": []}
        projects.append(main)
    if main.get("backends") is None:
        main["backends"] = []
    if not isinstance(main["backends"], list):
        raise ValueError("project `main` of the existing dstack config has `backends` that is not a list; not overwriting")
    for i, b in enumerate(main["backends"]):
        if isinstance(b, dict) and b.get("type") == entry["type"]:
            main["backends"][i] = entry
            break
    else:
        main["backends"].append(entry)
    return doc


def configure_backend(backend: str, fields: Dict[str, str], path: Optional[str] = None) -> Dict[str, Any]:
    path = path or server_config_path()
    try:
        os.makedirs(os.path.dirname(path), exist_ok=True)
        existing = None
        if os.path.exists(path):
            if not os.path.exists(path + ".bak"):
                shutil.copyfile(path, path + ".bak")
            try:
                with open(path) as f:
                    existing = yaml.safe_load(f)
                if existing is not None and not isinstance(existing, dict):
                    raise ValueError("not a mapping")
            except (yaml.YAMLError, ValueError) as e:
                return {"ok": False, "reason": f"existing {path} is not a valid dstack config ({e}); a copy is at {os.path.basename(path)}.bak: fix or remove it"}
        doc = merge_backend(existing, backend, fields)
        fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
        with os.fdopen(fd, "w") as f:
            yaml.safe_dump(doc, f, sort_keys=False)
        os.chmod(path, 0o600)
        return {"ok": True, "path": path}
    except (OSError, ValueError) as e:
        return {"ok": False, "reason": f"{backend}: {e}"}


@dataclass
class DstackConfig:
    gpu: str = "B200"
    count: int = 1
    image: str = "surogate-b200:latest"
    backend: Optional[str] = None  # pin one cloud; None = whichever offer is cheapest
    region: Optional[str] = None


def task_spec(name: str, cfg: DstackConfig, config_text: str, mode: str = "sft", surogate_bin: str = "surogate") -> Dict[str, Any]:
    """The dstack task as a mapping.  One literal shell block = one shell session: write the config, run the trainer in the
    background into a log, follow the feed on stdout."""
    if HEREDOC_TAG in config_text:
        raise ValueError(f"the config contains the here-document tag {HEREDOC_TAG}")
    script = "\n".join([
        f"cat > config.yaml <<'{HEREDOC_TAG}'",
        config_text.rstrip(),
        HEREDOC_TAG,
        f"SUROGATE_METRICS_PATH=metrics.jsonl {surogate_bin} {mode} config.yaml > train.log 2>&1 &",
        "sleep 3",
        "tail -n +1 -F metrics.jsonl",
    ]) + "\n"
    spec: Dict[str, Any] = {"type": "task", "name": name, "image": cfg.image}
    if cfg.backend:
        spec["backends"] = [cfg.backend]
    if cfg.region:
        spec["regions"] = [cfg.region]
    spec["commands"] = [script]
    spec["resources"] = {"gpu": f"{cfg.gpu}:{max(1, cfg.count)}"}
    return spec


class _Literal(str):
    pass


def task_yaml(name: str, cfg: DstackConfig, config_text: str, mode: str = "sft", surogate_bin: str = "surogate") -> str:
    spec = task_spec(name, cfg, config_text, mode, surogate_bin)
    spec["commands"] = [_Literal(c) for c in spec["commands"]]

    class Dumper(yaml.SafeDumper):
        pass

    Dumper.add_representer(_Literal, lambda d, s: d.represent_scalar("tag:yaml.org,2002:str", str(s), style="|"))
    return yaml.dump(spec, Dumper=Dumper, sort_keys=False)


def available(run=subprocess.run) -> bool:
    try:
        return run(["dstack", "--version"], capture_output=True, timeout=8).returncode == 0
    except (OSError, subprocess.TimeoutExpired):
        return False


def run_name(run_id: str) -> str:
    return re.sub(r"[^a-z0-9-]", "-", f"sur-{run_id}".lower())[:40]


def launch_dstack(cfg: DstackConfig, config_text: str, label: str, mode: str = "sft", surogate_bin: str = "surogate", root: Optional[str] = None,
                  popen=subprocess.Popen) -> Dict[str, Any]:
    rd = new_run(f"dstack-{label}", root)
    name = run_name(rd.id)
    task_file = os.path.join(rd.dir, "task.dstack.yml")
    try:
        with open(rd.config, "w") as f:
            f.write(config_text)
        with open(task_file, "w") as f:
            f.write(task_yaml(name, cfg, config_text, mode, surogate_bin))
        proc = popen(["dstack", "apply", "-y", "--name", name, "-f", task_file], cwd=rd.dir, stdin=subprocess.DEVNULL, stdout=subprocess.PIPE,
                     stderr=subprocess.PIPE)
    except (OSError, ValueError) as e:
        return {"ok": False, "reason": f'could not run "dstack" ({e}); is the CLI installed? (pip install dstack)', "run": rd}
    pump_metrics(proc, rd.feed, rd.log)
    register(proc)
    c = load_overlaid(config_text)
    rd.write_meta(mode=mode, label=f"dstack-{label}", model=c.get("model"), recipe=c.get("recipe"), max_steps=c.get("max_steps"),
                  remote={"kind": "dstack", "host": f"dstack · {cfg.backend or 'cheapest'} · {cfg.gpu}:{cfg.count}", "session": name, "dir": "(cloud)"})
    return {"ok": True, "run": rd, "feed": rd.feed, "name": name, "proc": proc}


def stop_dstack(name: str, proc: Optional[subprocess.Popen] = None, popen=subprocess.Popen) -> bool:
    """Stop the cloud run by name and end the local attached stream."""
    if proc is not None and proc.poll() is None:
        proc.terminate()
    try:
        popen(["dstack", "stop", "-y", name], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, stdin=subprocess.DEVNULL, start_new_session=True)
    except OSError:
        return False
    return True

"""``surogate launch``: start, list, stop and fetch training runs on this machine, an SSH host, dstack cloud GPUs or Modal.

    surogate launch run cfg.yaml --target local --gpus 0,1
    surogate launch run --model Qwen/Qwen3-0.6B --dataset data.jsonl --target ssh:user@host
    surogate launch run cfg.yaml --target dstack --gpu B200 --count 8 --backend runpod
    surogate launch run cfg.yaml --target modal --gpu B200
    surogate launch runs | stop <run> | fetch <run> | fit --model ... | providers [add|remove] | dstack-backend <cloud> key=value ...

Every run gets a directory of its own with its feed, config, log and outputs; ``surogate monitor --feed <run>/metrics.jsonl``
follows it, ``--watch`` does so right after the start.

Parity: jackalope/src/ui/Launch.tsx and its back ends (jackalope/src/{launch,ssh,dstack,modal,artifacts,providers}.ts).
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List, Optional


def _table(rows) -> str:
    from .monitor import table

    return table(rows) if rows else "(none)"


def _resolve_run(name: str, root: Optional[str]):
    from ..launch.runs import RunDir, runs_root

    for cand in (name, os.path.join(runs_root(root), name)):
        if os.path.isdir(cand):
            return RunDir(os.path.abspath(cand))
        if os.path.isfile(cand):
            return RunDir.of_feed(cand)
    raise SystemExit(f"no such run: {name}")


def _config_text(a) -> str:
    from ..launch.configs import LaunchFields, build_config

    if a.config:
        with open(a.config) as f:
            return f.read()
    fields = LaunchFields(model=a.model or "", dataset_path=a.dataset or "", dataset_type=a.dataset_type, recipe=a.recipe, max_steps=a.max_steps,
                          learning_rate=a.learning_rate, per_device_batch=a.batch, grad_accum=a.grad_accum, sequence_len=a.sequence_len, lora=not a.full,
                          optimizer=a.optimizer, output_dir=a.output_dir)
    bad = fields.problems()
    if bad:
        raise SystemExit("cannot build a config: " + "; ".join(bad))
    return build_config(fields, n_gpus=max(1, len(a.gpu_ids) or a.count))


def main(argv: List[str], command: str = "launch") -> int:
    p = argparse.ArgumentParser(prog="surogate launch")
    p.add_argument("--runs-dir", default=None, help="run history root (default ~/.surogate-watch/runs or $SUROGATE_RUNS_DIR)")
    sub = p.add_subparsers(dest="action", required=True)

    r = sub.add_parser("run", help="start a run")
    r.add_argument("config", nargs="?", help="a training config; without one the config is built from --model / --dataset / ...")
    r.add_argument("--target", default="local", help="local | ssh:<user@host[:port]> | dstack | modal | a saved provider id")
    r.add_argument("--mode", default="sft", choices=["sft", "pt", "dpo", "grpo-train", "grpo-colocate"])
    r.add_argument("--gpus", dest="gpu_ids", default="", help="local / ssh: comma-separated GPU indices")
    r.add_argument("--gpu", default="B200", help="dstack / modal: GPU type")
    r.add_argument("--count", type=int, default=1, help="dstack / modal: number of GPUs")
    r.add_argument("--image", default=None)
    r.add_argument("--backend", default=None)
    r.add_argument("--region", default=None)
    r.add_argument("--label", default=None)
    r.add_argument("--surogate-bin", default=None)
    r.add_argument("--watch", action="store_true", help="open the monitor on the run's feed after starting it")
    r.add_argument("--dry-run", action="store_true", help="print the config (and the task / command) instead of starting anything")
    for flag, kw in (("--model", {}), ("--dataset", {}), ("--dataset-type", {"default": "auto"}), ("--recipe", {"default": "fp8-hybrid"}),
                     ("--max-steps", {"type": int, "default": 200}), ("--learning-rate", {"type": float, "default": 2e-4}),
                     ("--batch", {"type": int, "default": 2}), ("--grad-accum", {"type": int, "default": 4}), ("--sequence-len", {"type": int, "default": 2048}),
                     ("--optimizer", {"default": "adamw_8bit"}), ("--output-dir", {"default": "./watch-out"})):
        r.add_argument(flag, **kw)
    r.add_argument("--full", action="store_true", help="full fine-tuning instead of LoRA")

    sub.add_parser("runs", help="run history")
    for name in ("stop", "fetch"):
        s = sub.add_parser(name)
        s.add_argument("run")
    f = sub.add_parser("fit", help="rough memory estimate of a run against the GPUs of this machine")
    f.add_argument("--model", required=True)
    f.add_argument("--recipe", default="fp8-hybrid")
    f.add_argument("--full", action="store_true")
    f.add_argument("--qlora", default="none")
    f.add_argument("--optimizer", default="adamw_8bit")
    f.add_argument("--batch", type=int, default=2)
    f.add_argument("--sequence-len", type=int, default=2048)
    f.add_argument("--gpus", type=int, default=1)
    f.add_argument("--zero-level", type=int, default=1)
    pr = sub.add_parser("providers", help="saved compute targets")
    pr.add_argument("op", nargs="?", default="list", choices=["list", "add", "remove"])
    pr.add_argument("--kind", choices=["ssh", "modal", "dstack"])
    pr.add_argument("--key", help="host (ssh), workspace (modal) or backend (dstack)")
    pr.add_argument("--label")
    pr.add_argument("--region")
    pr.add_argument("--gpu")
    pr.add_argument("--store", default=None)
    db = sub.add_parser("dstack-backend", help="merge one cloud backend's credentials into dstack's own server config")
    db.add_argument("backend")
    db.add_argument("fields", nargs="*", help="key=value ...")
    db.add_argument("--config-path", default=None)
    a = p.parse_args(argv)

    if a.action == "runs":
        from ..launch.runs import list_runs

        print(_table([{k: v for k, v in row.items() if k != "dir"} for row in list_runs(a.runs_dir)]))
        return 0
    if a.action == "fit":
        from ..launch.fit import estimate_run_memory_gb, fit_verdict
        from .monitor import live_gpus

        est = estimate_run_memory_gb(a.model, a.recipe, not a.full, a.qlora, a.optimizer, a.batch, a.sequence_len, True, a.gpus, a.zero_level)
        print(f"estimate: {'unknown (no parameter count in the name)' if est is None else f'~{est} GB per GPU'}")
        for g in live_gpus():
            free = (float(g.get("mem_total", 0)) - float(g.get("mem_used", 0))) / 2**30 if g.get("mem_total") else None
            print(f"gpu{g.get('index')}: {'?' if free is None else f'{free:.0f} GB free'}  {fit_verdict(est, free)}")
        return 0
    if a.action == "providers":
        from ..launch.providers import ProviderRecord, ProviderStore, provider_id

        store = ProviderStore(a.store)
        if a.op == "add":
            if not a.kind or not a.key:
                p.error("providers add needs --kind and --key")
            rec = ProviderRecord(id=provider_id(a.kind, a.key), kind=a.kind, label=a.label or a.key, region=a.region, gpu=a.gpu,
                                 host=a.key if a.kind == "ssh" else None, workspace=a.key if a.kind == "modal" else None,
                                 backend=a.key if a.kind == "dstack" else None)
            store.save(rec)
        elif a.op == "remove":
            if not a.key:
                p.error("providers remove needs --key (the provider id, or --kind with the key)")
            store.delete(a.key if ":" in a.key or not a.kind else provider_id(a.kind, a.key))
        print(_table([{"id": r.id, "kind": r.kind, "label": r.label, "gpu": r.gpu or "", "region": r.region or ""} for r in store.load()]))
        return 0
    if a.action == "dstack-backend":
        from ..launch.dstack import configure_backend

        fields = dict(kv.split("=", 1) for kv in a.fields if "=" in kv)
        res = configure_backend(a.backend, fields, a.config_path)
        print(f"written: {res['path']}" if res["ok"] else f"refused: {res['reason']}", file=sys.stderr if not res["ok"] else sys.stdout)
        return 0 if res["ok"] else 1
    if a.action == "stop":
        run = _resolve_run(a.run, a.runs_dir)
        remote = run.read_meta().get("remote") or {}
        if remote.get("kind") == "ssh":
            from ..launch.ssh import parse_target, stop_remote

            ok = stop_remote(parse_target(remote["host"]), remote["session"])
        elif remote.get("kind") == "dstack":
            from ..launch.dstack import stop_dstack

            ok = stop_dstack(remote["session"])
        elif remote.get("kind") == "modal":
            from ..launch.modal import stop_modal

            ok = stop_modal(run)
        else:
            from ..launch.local import stop_local

            ok = stop_local(run)
        print("stop sent" if ok else "nothing to stop")
        return 0 if ok else 1
    if a.action == "fetch":
        from ..launch.artifacts import fetch_artifacts

        res = fetch_artifacts(_resolve_run(a.run, a.runs_dir), on_line=lambda l: print(l, file=sys.stderr))
        print(res["dest"] if res["ok"] else res["reason"])
        return 0 if res["ok"] else 1

    # run
    a.gpu_ids = [int(g) for g in a.gpu_ids.split(",") if g.strip() != ""]
    text = _config_text(a)
    label = a.label or os.path.splitext(os.path.basename(a.config or a.model or "run"))[0]
    target = a.target
    if ":" in target and not target.startswith("ssh:"):
        from ..launch.providers import ProviderStore

        rec = ProviderStore().get(target)
        if rec is None:
            raise SystemExit(f"no saved provider {target}")
        target = {"ssh": f"ssh:{rec.host}", "modal": "modal", "dstack": "dstack"}[rec.kind]
        a.backend, a.region = a.backend or rec.backend, a.region or rec.region
        if rec.gpu:
            a.gpu, _, n = rec.gpu.partition(":")
            a.count = int(n) if n else a.count
    if a.dry_run:
        print(text)
        if target == "dstack":
            from ..launch.dstack import DstackConfig, task_yaml

            print("# --- dstack task ---\n" + task_yaml("sur-preview", DstackConfig(a.gpu, a.count, a.image or "surogate-b200:latest", a.backend, a.region), text, a.mode,
                                                         a.surogate_bin or "surogate"))
        else:
            from ..launch.configs import build_command

            print("# " + build_command(a.gpu_ids, "config.yaml", a.mode, a.surogate_bin or "surogate"))
        return 0
    if target == "local":
        from ..launch.local import launch_local

        res = launch_local(text, label, a.gpu_ids, a.mode, a.runs_dir, a.surogate_bin)
    elif target.startswith("ssh:"):
        from ..launch.ssh import launch_remote, parse_target, recent_hosts

        res = launch_remote(parse_target(target[4:]), text, label, a.mode, a.surogate_bin or "surogate", a.gpu_ids, a.runs_dir)
        if res["ok"]:
            recent_hosts(remember=target[4:])
    elif target == "dstack":
        from ..launch.dstack import DstackConfig, launch_dstack

        res = launch_dstack(DstackConfig(a.gpu, a.count, a.image or "surogate-b200:latest", a.backend, a.region), text, label, a.mode, a.surogate_bin or "surogate",
                            a.runs_dir)
    elif target == "modal":
        from ..launch.modal import ModalConfig, launch_modal

        res = launch_modal(ModalConfig(a.gpu, a.count, a.image or "surogate-b200:latest"), text, label, a.mode, a.runs_dir)
    else:
        raise SystemExit(f"unknown target {a.target}")
    if not res["ok"]:
        print(f"launch failed: {res['reason']}", file=sys.stderr)
        return 1
    print(res["feed"])
    streaming = res.get("proc") is not None or res.get("mirrors")
    if a.watch or streaming:  # cloud / ssh runs stream through this process: stay attached
        from . import monitor

        try:
            return monitor.main(["watch", "--feed", res["feed"]])
        finally:
            from ..launch.stream import stop_all

            stop_all()
    return 0

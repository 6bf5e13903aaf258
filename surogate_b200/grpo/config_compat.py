"""Orchestrator configs written in the nested schema (``model: {name}``, ``client: {base_url: [...]}``, ``sampling: {...}``,
``env: [{id, args}]``, ``buffer``, ``rollout_depth``, ``advantage``, ``filters``, ``ckpt``, ``eval``, ``weight_broadcast: {type}``,
``rollout_transport: {type}``, ``batch_size`` / ``rollouts_per_example`` ...) translated to this package's flat orchestrator keys.

``flatten_orchestrator_config(raw)`` returns ``(flat, notes)``: ``flat`` is a dict the ``grpo-orch`` command reads like a config file
of its own schema (it selects the asynchronous loop, which is the one the nested schema describes), ``notes`` lists every key
that was dropped or approximated, so nothing is ignored silently.  A config already in the flat schema is returned unchanged.

Parity: surogate/core/config/grpo_orch_config.py (GRPOOrchestratorConfig and its sections).
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Tuple

NESTED_MARKERS = ("client", "sampling", "env", "rollout_transport", "rollout_depth", "ckpt", "rollouts_per_example")


def is_nested_schema(raw: Dict[str, Any]) -> bool:
    return isinstance(raw.get("model"), dict) or isinstance(raw.get("weight_broadcast"), dict) or any(k in raw for k in NESTED_MARKERS)


def _take(section: Dict[str, Any], known: Dict[str, str], notes: List[str], where: str) -> Dict[str, Any]:
    """``known``: their key -> our key ("" = accepted, nothing to set).  Unknown keys are reported."""
    out = {}
    for k, v in (section or {}).items():
        if k in known:
            if known[k] and v is not None:
                out[known[k]] = v
        elif v not in (None, {}, [], False):
            notes.append(f"{where}.{k}: not supported here, ignored")
    return out


def flatten_orchestrator_config(raw: Dict[str, Any]) -> Tuple[Dict[str, Any], List[str]]:
    if not is_nested_schema(raw):
        return dict(raw), []
    notes: List[str] = []
    flat: Dict[str, Any] = {"scheduler": "async"}
    out_dir = raw.get("output_dir") or "outputs/run_default"

    model = raw.get("model")
    if isinstance(model, dict):
        flat["model"] = model.get("name") or ""
        if model.get("lora_adapter"):
            flat["served_model"] = model["lora_adapter"]  # requests name the adapter, the tokenizer comes from the base model
    elif model:
        flat["model"] = model

    client = raw.get("client") or {}
    urls = client.get("base_url") or ["http://localhost:8000/v1"]
    urls = [urls] if isinstance(urls, str) else list(urls)
    flat["base_url"], flat["base_urls"] = urls[0], urls
    if client.get("timeout") is not None:
        flat["request_timeout_s"] = float(client["timeout"])
    if client.get("api_key_var"):
        flat["api_key_var"] = client["api_key_var"]
    if client.get("headers"):
        flat["headers"] = dict(client["headers"])
    _take({k: v for k, v in client.items() if k not in ("base_url", "timeout", "api_key_var", "headers")}, {"skip_model_check": ""}, notes, "client")

    s = raw.get("sampling") or {}
    extra = dict(s.get("extra_body") or {})
    if s.get("temp_scheduler"):
        ts = s["temp_scheduler"]
        flat["temperature_schedule"] = {"type": ts.get("type") or "linear", "start": ts.get("start_temperature"), "end": ts.get("end_temperature"),
                                        "total_steps": ts.get("total_steps")}
        if s.get("temperature") is not None:
            raise ValueError("sampling: set temperature or temp_scheduler, not both")
    flat["temperature"] = 1.0 if s.get("temperature") is None else float(s["temperature"])
    flat["top_p"] = 1.0 if s.get("top_p") is None else float(s["top_p"])
    if s.get("max_tokens") is not None:
        flat["max_tokens"] = int(s["max_tokens"])
    for k in ("repetition_penalty", "min_tokens", "seed"):
        if s.get(k) not in (None, 0 if k == "min_tokens" else None, 1.0 if k == "repetition_penalty" else None):
            extra[k] = s[k]
    if extra:
        flat["extra_sampling"] = extra
    _take({k: v for k, v in s.items() if k not in ("temperature", "temp_scheduler", "top_p", "max_tokens", "repetition_penalty", "min_tokens", "seed", "extra_body")},
          {}, notes, "sampling")

    envs = raw.get("env") or []
    envs = [envs] if isinstance(envs, dict) else list(envs)
    if envs:
        e0 = envs[0]
        flat["environment"] = e0.get("id") or e0.get("name") or ""
        flat["environment_args"] = dict(e0.get("args") or {}, **(e0.get("extra_env_kwargs") or {}))
        if e0.get("path"):
            flat["environment_import_path"] = e0["path"]
        if e0.get("address"):
            notes.append("env[0].address: environments run inside the orchestrator process here, no environment server is contacted")
        if len(envs) > 1:
            flat["environments"] = [{"id": e.get("id") or e.get("name"), "name": e.get("name"), "args": dict(e.get("args") or {}), "path": e.get("path"),
                                     "extra_env_kwargs": dict(e.get("extra_env_kwargs") or {})} for e in envs]

    rollouts = int(raw.get("rollouts_per_example") or 1)
    batch = int(raw.get("batch_size") or 128)
    flat["group_size"] = rollouts
    flat["batch_size"] = batch
    flat["prompts_per_step"] = max(1, batch // max(1, rollouts))
    if raw.get("token_batch_size"):
        flat["token_batch_size"] = int(raw["token_batch_size"])
    seq = int(raw.get("sequence_len") or raw.get("seq_len") or 2048)
    flat["sequence_len"] = seq
    if raw.get("rows_per_step"):
        flat["rows_per_step"] = int(raw["rows_per_step"])
    else:  # as many packed rows as a step's rollouts need; the trainer pads them to a multiple of its micro-batch
        flat["rows_per_step"] = 0
    for theirs, ours in (("max_steps", "max_steps"), ("max_off_policy_steps", "max_off_policy_steps"), ("max_async_level", "max_async_level"), ("seed", "seed"),
                         ("max_inflight_rollouts", "max_inflight"), ("max_concurrent", "workers")):
        if raw.get(theirs) is not None:
            flat[ours] = int(raw[theirs])
    if "max_inflight" in flat:  # theirs counts rollouts, ours counts group requests
        flat["max_inflight"] = max(1, flat["max_inflight"] // max(1, rollouts))
    if raw.get("oversampling_factor"):
        flat.setdefault("max_inflight", max(1, int(flat["prompts_per_step"] * float(raw["oversampling_factor"]))))

    if raw.get("buffer"):
        flat["buffer"] = _take(raw["buffer"], {"seed": "seed", "env_ratios": "env_ratios", "easy_threshold": "easy_threshold", "hard_threshold": "hard_threshold",
                                               "easy_fraction": "easy_fraction", "hard_fraction": "hard_fraction", "online_difficulty_filtering": "online_difficulty_filtering",
                                               "normal_pool_min_examples": "min_normal", "hash_keys": "", "recycle_easy_fraction": "", "recycle_hard_fraction": "",
                                               "sample_without_replacement": ""}, notes, "buffer")
    if raw.get("rollout_depth"):
        flat["depth"] = _take(raw["rollout_depth"], {"enabled": "enabled", "quantile": "quantile", "min_depth": "min_cap", "max_depth": "max_cap",
                                                     "probe_interval": "probe_every", "min_observations": "min_observations", "ema": "", "warmup_steps": ""}, notes, "rollout_depth")
    adv = raw.get("advantage") or {}
    if adv.get("type") == "custom":
        path = adv.get("import_path") or ""
        flat["advantage"] = path if ":" in path else ":".join(path.rsplit(".", 1))
        if adv.get("kwargs"):
            flat["advantage_kwargs"] = dict(adv["kwargs"])
    elif adv:
        flat["advantage"] = "default"
        flat["length_weighted_mean"] = bool(adv.get("length_weighted_mean", False))
    if raw.get("filters"):
        flat["filters"] = [dict(f) for f in raw["filters"]]
        for f in flat["filters"]:
            f.setdefault("enforce", False)  # their default: count only

    ck = raw.get("ckpt") or {}
    if ck.get("interval"):
        flat["checkpoint_every"] = int(ck["interval"])
        flat["checkpoint_dir"] = os.path.join(out_dir, "orch_checkpoints")
    if ck.get("keep_last"):
        flat["keep_checkpoints"] = int(ck["keep_last"])
    if ck.get("resume_step") is not None:
        flat["resume_step"] = int(ck["resume_step"])
    _take({k: v for k, v in ck.items() if k not in ("interval", "keep_last", "resume_step")}, {"wait_for_weights_timeout": "", "keep_interval": "", "skip_progress": "", "skip_buffer": ""},
          notes, "ckpt")

    ev = raw.get("eval") or {}
    if ev:
        flat["eval_every"] = int(ev.get("interval") or 100)
        flat["eval_samples"] = int(ev.get("rollouts_per_example") or 1)
        if ev.get("num_examples") not in (None, -1):
            flat["eval_examples"] = int(ev["num_examples"])
        if ev.get("env"):
            flat["eval_environments"] = [{"id": e.get("id") or e.get("name"), "name": e.get("name"), "args": dict(e.get("args") or {}), "path": e.get("path"),
                                          "num_examples": e.get("num_examples")} for e in ev["env"]]

    wb = raw.get("weight_broadcast") or {}
    flat["weight_broadcast"] = (wb.get("type") if isinstance(wb, dict) else wb) or "filesystem"
    flat["weight_dir"] = raw.get("weight_dir") or os.path.join(out_dir, "weights")
    rt = raw.get("rollout_transport") or {}
    flat["transport"] = (rt.get("type") if isinstance(rt, dict) else rt) or "filesystem"
    flat["transport_dir"] = raw.get("transport_dir") or os.path.join(out_dir, "rollouts")
    if flat["transport"] == "zmq":
        flat["zmq_endpoint"] = f"tcp://{rt.get('host') or 'localhost'}:{int(rt.get('port') or 5555)}"

    if raw.get("ruler"):
        flat["ruler"] = dict(raw["ruler"])
    if raw.get("teacher_model"):
        flat["teacher"] = dict(raw["teacher_model"])
    if raw.get("tasks_per_minute"):
        flat["tasks_per_minute"] = float(raw["tasks_per_minute"])
    if raw.get("dump_metrics"):
        flat["metrics_file"] = os.path.join(out_dir, "orchestrator_metrics.jsonl")
    val = raw.get("val") or {}
    if val:
        flat.update(val_every=int(val.get("interval") or 10), val_examples=int(val.get("num_examples") or 16), val_samples=int(val.get("rollouts_per_example") or 1))
    for k in ("verification", "strict_async_level", "bench", "use_token_client", "learning_rate", "log", "report_to"):
        v = raw.get(k)
        if v not in (None, {}, [], False) and not (k == "verification" and v == {"enabled": True}) and k not in ("log", "report_to", "learning_rate", "use_token_client"):
            notes.append(f"{k}: not supported by this orchestrator, ignored")
    return flat, notes


def temperature_at(step: int, schedule: Dict[str, Any], max_steps: int) -> float:
    """Temperature of a step under ``{type: linear | cosine, start, end, total_steps}``; constant ``end`` after ``total_steps``."""
    import math

    total = max(1, int(schedule.get("total_steps") or max_steps))
    start, end = float(schedule["start"]), float(schedule["end"])
    f = min(1.0, max(0.0, step / total))
    if (schedule.get("type") or "linear") == "cosine":
        f = 0.5 * (1.0 - math.cos(math.pi * f))
    return start + (end - start) * f

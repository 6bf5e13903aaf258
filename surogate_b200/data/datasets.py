"""Dataset loading and row preprocessing for ``surogate sft|pt|dpo``.

A dataset is a local file or directory (``.jsonl`` / ``.json`` / ``.parquet`` / ``.csv`` / ``.txt``) or, when the
``datasets`` package and a network are available, a HuggingFace dataset name.  Each row is normalised by a
preprocessor chosen from the dataset ``type`` (or detected from the columns) into one of

* ``{"text": str}``                                  — plain text (pre-training),
* ``{"messages": [{"role", "content"}...], "tools"}`` — chat (instruction / alpaca / conversation / messages),
* ``{"prompt": [...], "chosen": str, "rejected": str}`` — preference pairs (DPO).

Parity: surogate/core/datasets/loader.py, preprocessor/{auto,text,instruction,alpaca,conversation,messages,preference,row}.py.
"""
from __future__ import annotations

import csv
import glob
import json
import os
from typing import Any, Dict, Iterable, Iterator, List, Optional

ROLE_ALIASES = {"human": "user", "user": "user", "gpt": "assistant", "assistant": "assistant", "bot": "assistant", "model": "assistant",
                "system": "system", "tool": "tool", "function": "tool", "observation": "tool", "function_call": "assistant"}


# ---------------------------------------------------------------------- loading
def _iter_file(path: str) -> Iterator[Dict[str, Any]]:
    ext = os.path.splitext(path)[1].lower()
    if ext in (".jsonl", ".ndjson"):
        with open(path) as f:
            for line in f:
                line = line.strip()
                if line:
                    yield json.loads(line)
    elif ext == ".json":
        with open(path) as f:
            data = json.load(f)
        if isinstance(data, dict):
            data = data.get("data") or data.get("train") or next((v for v in data.values() if isinstance(v, list)), [])
        yield from data
    elif ext == ".parquet":
        import pyarrow.parquet as pq

        for batch in pq.ParquetFile(path).iter_batches():
            yield from batch.to_pylist()
    elif ext in (".csv", ".tsv"):
        with open(path, newline="") as f:
            yield from csv.DictReader(f, delimiter="\t" if ext == ".tsv" else ",")
    elif ext in (".txt", ".md"):
        with open(path) as f:
            for para in f.read().split("\n\n"):
                if para.strip():
                    yield {"text": para.strip()}
    else:
        raise ValueError(f"unsupported dataset file type: {path}")


def fetch_remote(url: str, split: str = "train", cache_dir: Optional[str] = None) -> List[str]:
    """Copy the data files under an object-store URL (``s3://bucket/prefix``, ``gs://...``, any fsspec protocol) into a local
    cache directory and return the local paths.  A URL that names one file fetches that file; a prefix fetches every data file
    below it (those whose name contains ``split`` when any does).  Files already present with the same size are reused."""
    import hashlib

    try:
        import fsspec
    except ImportError as e:  # pragma: no cover - fsspec ships with the image
        raise RuntimeError(f"{url}: object-store datasets need the `fsspec` package") from e
    proto = url.split("://", 1)[0]
    try:
        fs = fsspec.filesystem(proto)
    except (ImportError, ValueError) as e:
        raise RuntimeError(f"{url}: no fsspec backend for '{proto}://' is installed (s3 needs s3fs, gs needs gcsfs)") from e
    exts = (".jsonl", ".ndjson", ".json", ".parquet", ".csv", ".tsv", ".txt")
    if fs.isdir(url):
        names = sorted(n for n in fs.find(url) if os.path.splitext(n)[1].lower() in exts)
        names = [n for n in names if split in os.path.basename(n)] or names
    else:
        names = [url]
    if not names:
        raise FileNotFoundError(f"{url}: no data files ({', '.join(exts)}) found")
    from ..utils.fs import get_cache_dir

    root = cache_dir or os.path.join(get_cache_dir(), "datasets", hashlib.sha1(url.encode()).hexdigest()[:16])
    os.makedirs(root, exist_ok=True)
    out = []
    for n in names:
        local = os.path.join(root, os.path.basename(n))
        size = fs.size(n)
        if not (os.path.exists(local) and os.path.getsize(local) == size):
            fs.get(n, local + ".part")
            os.replace(local + ".part", local)
        out.append(local)
    return out


def load_rows(cfg, max_rows: Optional[int] = None) -> List[Dict[str, Any]]:
    """Rows of one dataset config (``DatasetConfig``) as a list of dicts."""
    path = cfg.path
    limit = cfg.samples if cfg.samples else max_rows
    rows: List[Dict[str, Any]] = []
    if os.path.isdir(path):
        split = cfg.split or "train"
        files = sorted(f for f in glob.glob(os.path.join(path, "**", "*"), recursive=True)
                       if os.path.splitext(f)[1].lower() in (".jsonl", ".ndjson", ".json", ".parquet", ".csv", ".tsv", ".txt"))
        chosen = [f for f in files if split in os.path.basename(f)] or files
        it: Iterable = (r for f in chosen for r in _iter_file(f))
    elif os.path.exists(path):
        it = _iter_file(path)
    elif "://" in path and not path.startswith(("http://", "https://")):
        it = (r for f in fetch_remote(path, cfg.split or "train") for r in _iter_file(f))
    else:
        try:
            import datasets as hf_datasets  # type: ignore
        except ImportError as e:
            raise FileNotFoundError(f"dataset '{path}' is not a local path and the `datasets` package is not installed") from e
        it = hf_datasets.load_dataset(path, cfg.subset, split=cfg.split or "train")
    for r in it:
        rows.append(dict(r))
        if limit and len(rows) >= limit:
            break
    return rows


# ---------------------------------------------------------------------- type detection
def detect_type(columns: Iterable[str]) -> str:
    c = set(columns)
    if {"chosen", "rejected"} <= c:
        return "preference"
    if "messages" in c:
        return "messages"
    if "conversations" in c or "conversation" in c:
        return "conversation"
    if {"instruction", "output"} <= c:
        return "alpaca" if "input" in c else "instruction"
    if {"prompt", "completion"} <= c or {"prompt", "response"} <= c or {"question", "answer"} <= c:
        return "instruction"
    if "text" in c or "content" in c:
        return "text"
    raise ValueError(f"[E120] cannot detect the dataset type from columns {sorted(c)}; set `type:` explicitly")


# ---------------------------------------------------------------------- preprocessors
def _norm_messages(raw, mappings: Dict[str, str]) -> List[Dict[str, Any]]:
    role_key = mappings.get("role", "role")
    content_key = mappings.get("content", "content")
    out = []
    for m in raw:
        if role_key not in m and "from" in m:
            role_key, content_key = "from", "value"
        role = ROLE_ALIASES.get(str(m.get(role_key, "")).lower(), str(m.get(role_key, "user")))
        msg = {"role": role, "content": m.get(content_key) if m.get(content_key) is not None else ""}
        for extra in ("tool_calls", "reasoning_content", "name", "tool_call_id", "loss"):
            if m.get(extra) is not None:
                msg[extra] = m[extra]
        out.append(msg)
    return out


def _system(cfg, row) -> Optional[str]:
    kind = cfg.system_prompt_type or ("fixed" if cfg.system_prompt else ("field" if cfg.system_prompt_field else None))
    if kind == "fixed":
        return cfg.system_prompt
    if kind == "field" and cfg.system_prompt_field:
        return row.get(cfg.system_prompt_field)
    return None


def preprocess_text(cfg, row) -> Optional[Dict[str, Any]]:
    t = row.get(cfg.text_field) if cfg.text_field in row else row.get("content")
    return {"text": t} if t else None


def preprocess_instruction(cfg, row) -> Optional[Dict[str, Any]]:
    pick = lambda *names: next((row[n] for n in names if n and row.get(n) not in (None, "")), None)  # noqa: E731
    instruction = pick(cfg.instruction_field, "instruction", "prompt", "question")
    output = pick(cfg.output_field, "output", "completion", "response", "answer")
    extra = pick(cfg.input_field) if cfg.input_field else None
    if instruction is None or output is None:
        return None
    system = _system(cfg, row)
    if cfg.prompt_format and (extra or not cfg.prompt_format_no_input):
        user = cfg.prompt_format.format(system=system or "", instruction=instruction, input=extra or "", output="")
    elif cfg.prompt_format_no_input and not extra:
        user = cfg.prompt_format_no_input.format(system=system or "", instruction=instruction, output="")
    else:
        user = f"{instruction}\n\n{extra}" if extra else str(instruction)
    msgs = ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": user}, {"role": "assistant", "content": str(output)}]
    return {"messages": msgs}


ALPACA_WITH_INPUT = ("Below is an instruction that describes a task, paired with an input that provides further context. "
                     "Write a response that appropriately completes the request.\n\n### Instruction:\n{instruction}\n\n### Input:\n{input}\n\n### Response:\n")
ALPACA_NO_INPUT = ("Below is an instruction that describes a task. Write a response that appropriately completes the request.\n\n"
                   "### Instruction:\n{instruction}\n\n### Response:\n")


def preprocess_alpaca(cfg, row) -> Optional[Dict[str, Any]]:
    ins, inp, out = row.get(cfg.instruction_field), row.get(cfg.input_field or "input"), row.get(cfg.output_field)
    if not ins or out is None:
        return None
    user = (ALPACA_WITH_INPUT if inp else ALPACA_NO_INPUT).format(instruction=ins, input=inp or "")
    return {"messages": [{"role": "user", "content": user}, {"role": "assistant", "content": str(out)}]}


def preprocess_conversation(cfg, row) -> Optional[Dict[str, Any]]:
    field = cfg.messages_field if cfg.messages_field in row else next((k for k in ("messages", "conversations", "conversation") if k in row), None)
    if field is None:
        return None
    raw = row[field]
    if isinstance(raw, str):
        raw = json.loads(raw)
    msgs = _norm_messages(raw, cfg.message_property_mappings)
    if cfg.completion_field and row.get(cfg.completion_field) is not None:
        comp = row[cfg.completion_field]
        msgs += _norm_messages(comp, cfg.message_property_mappings) if isinstance(comp, list) else [{"role": "assistant", "content": str(comp)}]
    sysmsg = row.get(cfg.system_field) if cfg.system_field else None
    if sysmsg and (not msgs or msgs[0]["role"] != "system"):
        msgs = [{"role": "system", "content": sysmsg}] + msgs
    if not any(m["role"] == "assistant" for m in msgs):
        return None
    out: Dict[str, Any] = {"messages": msgs}
    if cfg.tools_field and row.get(cfg.tools_field):
        tools = row[cfg.tools_field]
        out["tools"] = json.loads(tools) if isinstance(tools, str) else tools
    return out


def preprocess_preference(cfg, row) -> Optional[Dict[str, Any]]:
    chosen, rejected = row.get(cfg.chosen_field), row.get(cfg.rejected_field)
    if chosen is None or rejected is None:
        return None
    prompt = row.get(cfg.prompt_field)
    if isinstance(chosen, list):  # full conversations: the shared prefix is the prompt, the last message the answer
        c, r = _norm_messages(chosen, {}), _norm_messages(rejected, {})
        prompt_msgs = c[:-1]
        chosen, rejected = c[-1]["content"], r[-1]["content"]
    else:
        prompt_msgs = _norm_messages(prompt, {}) if isinstance(prompt, list) else [{"role": "user", "content": str(prompt or "")}]
    system = _system(cfg, row)
    if system and (not prompt_msgs or prompt_msgs[0]["role"] != "system"):
        prompt_msgs = [{"role": "system", "content": system}] + prompt_msgs
    out = {"prompt": prompt_msgs, "chosen": str(chosen), "rejected": str(rejected)}
    field = getattr(cfg, "enable_thinking_field", None)
    if field and field not in row:
        raise ValueError(f"enable-thinking field '{field}' is missing from the dataset; columns: {sorted(row)}")
    flag = row.get(field or "enable_thinking")
    if flag is not None:
        out["enable_thinking"] = bool(flag) if not isinstance(flag, str) else flag.strip().lower() in ("1", "true", "yes")
    return out


PREPROCESSORS = {"text": preprocess_text, "instruction": preprocess_instruction, "alpaca": preprocess_alpaca, "conversation": preprocess_conversation,
                 "messages": preprocess_conversation, "preference": preprocess_preference}


def preprocess_rows(cfg, rows: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
    if not rows:
        return []
    kind = cfg.type if cfg.type and cfg.type != "auto" else detect_type(rows[0].keys())
    if kind not in PREPROCESSORS:
        raise ValueError(f"[E121] unknown dataset type '{kind}' (known: {sorted(PREPROCESSORS)})")
    fn = PREPROCESSORS[kind]
    out = []
    for r in rows:
        p = fn(cfg, r)
        if p is not None:
            out.append(p)
    return out


def load_dataset_rows(cfg) -> List[Dict[str, Any]]:
    return preprocess_rows(cfg, load_rows(cfg))

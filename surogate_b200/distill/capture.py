"""Teacher capture (``surogate distill-capture``): run a teacher over token shards and store its top-K log-probs.

Teachers: a model trained / loadable by this framework (forward through the Trainer's executor with a hook on the
logits), a HuggingFace ``transformers`` model (local directory), or an OpenAI-compatible API that returns
``top_logprobs`` for a prompt (vLLM's ``prompt_logprobs``).  One ``.kd`` file is written next to each shard.

Parity: surogate/distill/capture.py.
"""
from __future__ import annotations

import json
import os
import urllib.request
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

from ..data.tokfile import read_token_file
from .sidecar import SidecarWriter, sidecar_path

TeacherFn = Callable[[np.ndarray], torch.Tensor]  # int32 [rows, T] -> logits [rows, T, V]


def topk_logprobs(logits: torch.Tensor, k: int, temperature: float = 1.0) -> Tuple[np.ndarray, np.ndarray]:
    lp = torch.log_softmax(logits.float() / temperature, dim=-1)
    v, i = lp.topk(k, dim=-1)
    return i.to(torch.int32).cpu().numpy(), v.cpu().numpy()


def hf_teacher(model_dir: str, device: str = "cuda", dtype=torch.bfloat16) -> TeacherFn:
    from transformers import AutoModelForCausalLM

    model = AutoModelForCausalLM.from_pretrained(model_dir, torch_dtype=dtype).to(device).eval()

    @torch.no_grad()
    def fn(tokens: np.ndarray) -> torch.Tensor:
        return model(torch.from_numpy(tokens.astype(np.int64)).to(device)).logits

    return fn


def native_teacher(trainer) -> TeacherFn:
    """A model held by this framework's Trainer: logits = final hidden states x LM head (computed in row chunks)."""

    @torch.no_grad()
    def fn(tokens: np.ndarray) -> torch.Tensor:
        return trainer.logits(tokens)

    return fn


def api_teacher_rows(base_url: str, model: str, k: int, timeout_s: float = 600.0, workers: int = 8, retries: int = 3, api_key: str = "EMPTY"):
    """vLLM-style ``prompt_logprobs``: returns a function rows -> (indices, logprobs) directly (no logits leave the server).

    Rows of a call are requested concurrently (``workers`` threads: the server batches them), a failed request is retried with
    back-off, and a position for which the server returned fewer than ``k`` entries is padded with log-prob -30 on token 0
    (weightless in the distillation term)."""
    import time
    from concurrent.futures import ThreadPoolExecutor

    url = base_url.rstrip("/") + "/completions"

    def one(row):
        body = {"model": model, "prompt": [int(t) for t in row], "max_tokens": 1, "prompt_logprobs": k, "temperature": 0.0}
        req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json", "Authorization": f"Bearer {api_key}"})
        last = None
        for attempt in range(retries):
            try:
                with urllib.request.urlopen(req, timeout=timeout_s) as resp:
                    return json.loads(resp.read())["choices"][0]["prompt_logprobs"]
            except Exception as e:  # noqa: BLE001 -- connection reset, 5xx, malformed body: all retried
                last = e
                time.sleep(min(2.0 ** attempt * 0.1, 5.0))
        raise RuntimeError(f"teacher at {url} failed {retries} times: {last}")

    def fn(tokens: np.ndarray):
        idx = np.zeros(tokens.shape + (k,), np.int32)
        lp = np.full(tokens.shape + (k,), -30.0, np.float32)
        with ThreadPoolExecutor(max_workers=max(1, min(workers, len(tokens)))) as pool:
            results = list(pool.map(one, tokens))
        for r, pl in enumerate(results):
            # entry t (t >= 1) is the distribution that predicted token t: store it at position t-1
            for t in range(1, min(len(pl), tokens.shape[1])):
                items = sorted(((int(tok), d["logprob"] if isinstance(d, dict) else float(d)) for tok, d in (pl[t] or {}).items()), key=lambda x: -x[1])[:k]
                for j, (tok, l) in enumerate(items):
                    idx[r, t - 1, j], lp[r, t - 1, j] = tok, l
        return idx, lp

    return fn


def sidecar_complete(shard: str, seq_len: int, top_k: int, path: Optional[str] = None) -> bool:
    """True when a sidecar with the expected K and number of positions already stands next to the shard (resume skips it)."""
    from ..data.tokfile import read_header
    from .sidecar import SidecarReader

    p = path or sidecar_path(shard)
    if not os.path.exists(p):
        return False
    try:
        r = SidecarReader(p)
        return r.K == top_k and r.N == (read_header(shard)["n_tokens"] // seq_len) * seq_len
    except Exception:  # noqa: BLE001 -- truncated or foreign file: capture again
        return False


def capture_shard(shard: str, teacher: TeacherFn, seq_len: int, top_k: int, vocab: int, temperature: float = 1.0, rows_per_call: int = 4,
                  out_path: Optional[str] = None, direct=None) -> str:
    tok, _, _, h = read_token_file(shard)
    n_rows = h["n_tokens"] // seq_len
    w = SidecarWriter(out_path or sidecar_path(shard), top_k, vocab, temperature)
    for s in range(0, n_rows, rows_per_call):
        rows = np.stack([np.asarray(tok[r * seq_len:(r + 1) * seq_len]) for r in range(s, min(n_rows, s + rows_per_call))])
        if direct is not None:
            idx, lp = direct(rows)
        else:
            idx, lp = topk_logprobs(teacher(rows), top_k, temperature)
        w.add(idx.reshape(-1, top_k), lp.reshape(-1, top_k))
    w.close()
    return w.path


def capture(shards: Iterable[str], teacher: TeacherFn, seq_len: int, top_k: int, vocab: int, resume: bool = True, out_dir: Optional[str] = None,
            **kw) -> List[str]:
    """One sidecar per shard, next to it or (``out_dir``) under another directory with the same file name; with ``resume`` a
    complete sidecar of the expected K and length is kept."""
    out = []
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
    for s in shards:
        path = kw.get("out_path") or (os.path.join(out_dir, os.path.basename(sidecar_path(s))) if out_dir else None)
        if resume and sidecar_complete(s, seq_len, top_k, path):
            out.append(path or sidecar_path(s))
            continue
        out.append(capture_shard(s, teacher, seq_len, top_k, vocab, **dict(kw, out_path=path)))
    return out

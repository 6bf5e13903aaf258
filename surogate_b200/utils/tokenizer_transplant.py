"""Vocabulary transplantation for cross-tokenizer distillation: give a student model the teacher's tokenizer.

The student's embedding and LM-head rows are rebuilt for the teacher's vocabulary.  Tokens both vocabularies contain keep their
rows exactly; a token only the teacher has is approximated, by default with orthogonal matching pursuit (OMP, arXiv:2506.06607):
the token's embedding in the TEACHER's space is written as a sparse combination of ``k`` shared tokens' teacher embeddings, and
the same coefficients applied to those tokens' STUDENT embeddings give the new row (the shared tokens are the bridge between
the two spaces).  Afterwards the student uses the teacher's tokenizer, so the same-tokenizer pipeline (tokenize ->
distill-capture -> sft) runs unchanged.  A ``transplant_manifest.json`` beside the output records both models, the method and
``k``; ``restore`` reads it to move a distilled model back to the student's own tokenizer.

Two engines:

* ``builtin`` (this file): exact-match sharing on the token strings of ``tokenizer.json``, methods ``omp`` / ``subword`` / ``mean`` /
  ``zero``; OMP runs batched in PyTorch (GPU when given a device) with the candidate atoms of each target pruned to the
  ``candidates`` shared tokens most correlated with it, which bounds the work at one full correlation pass;
* ``mergekit``: the external ``mergekit-tokensurgeon`` command (LGPL, never imported), when it is on PATH.

Parity: surogate/transplant/transplant.py (run_transplant, run_transplant_back, transplant_manifest.json), surogate/cli/transplant.py.
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

MANIFEST = "transplant_manifest.json"
BUILTIN_METHODS = ("omp", "subword", "mean", "zero")
MERGEKIT_METHODS = ("omp", "common_interpolation", "subword", "mean", "zero", "randn", "john_hewitt", "landmark_pca", "sparse_token_basis", "mp_rope")
TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "vocab.json", "merges.txt", "added_tokens.json",
                   "chat_template.jinja", "chat_template.json", "tokenizer.model", "generation_config.json")
EMBED_KEYS = ("model.embed_tokens.weight", "model.language_model.embed_tokens.weight", "transformer.wte.weight", "embed_tokens.weight")
HEAD_KEYS = ("lm_head.weight", "model.lm_head.weight", "output.weight")


# ---------------------------------------------------------------------- vocabularies
def load_vocab(model_dir: str) -> Dict[str, int]:
    """token string -> id from ``tokenizer.json`` (model vocabulary plus added tokens)."""
    with open(os.path.join(model_dir, "tokenizer.json")) as f:
        tj = json.load(f)
    vocab = tj.get("model", {}).get("vocab", {})
    if isinstance(vocab, list):  # unigram models store [piece, score] pairs
        vocab = {p[0]: i for i, p in enumerate(vocab)}
    out = {str(t): int(i) for t, i in vocab.items()}
    for a in tj.get("added_tokens", []) or []:
        out[str(a["content"])] = int(a["id"])
    return out


def vocab_size_of(model_dir: str, vocab: Dict[str, int]) -> int:
    """Rows the embedding needs: the config's (possibly padded) vocabulary size, at least the largest id + 1."""
    n = max(vocab.values()) + 1 if vocab else 0
    try:
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        n = max(n, int((cfg.get("text_config") or cfg).get("vocab_size", 0)))
    except (OSError, ValueError):
        pass
    return n


# ---------------------------------------------------------------------- approximations
def omp_rows(targets: torch.Tensor, atoms_ref: torch.Tensor, atoms_out: torch.Tensor, k: int = 64, candidates: int = 1024,
             batch: int = 32) -> torch.Tensor:
    """For every row ``t`` of ``targets`` [N, d_ref]: a ``k``-sparse least-squares fit ``t ~ c @ atoms_ref[S]`` chosen greedily
    (orthogonal matching pursuit) and returned as ``c @ atoms_out[S]`` [N, d_out].  ``atoms_ref`` [S, d_ref] and ``atoms_out``
    [S, d_out] are the shared tokens in the reference and the output space."""
    N, S = targets.shape[0], atoms_ref.shape[0]
    out = torch.zeros(N, atoms_out.shape[1], dtype=torch.float32, device=targets.device)
    if N == 0 or S == 0:
        return out
    k = max(1, min(k, S, atoms_ref.shape[1]))
    M = max(k, min(candidates, S))
    A = atoms_ref.float()
    A_unit = A / A.norm(dim=1, keepdim=True).clamp_min(1e-12)
    for s in range(0, N, batch):
        T = targets[s:s + batch].float()                                    # [B, d]
        B = T.shape[0]
        cand = (T @ A_unit.t()).abs().topk(M, dim=1).indices                 # [B, M] candidate atoms of each target
        D = A[cand]                                                          # [B, M, d]
        D_unit = A_unit[cand]
        chosen = torch.zeros(B, 0, dtype=torch.long, device=T.device)
        taken = torch.zeros(B, M, dtype=torch.bool, device=T.device)
        R = T.clone()
        coef = None
        for _ in range(k):
            corr = torch.einsum("bmd,bd->bm", D_unit, R).abs().masked_fill(taken, -1.0)
            pick = corr.argmax(dim=1, keepdim=True)
            taken.scatter_(1, pick, True)
            chosen = torch.cat([chosen, pick], dim=1)
            sel = torch.gather(D, 1, chosen[..., None].expand(-1, -1, D.shape[2]))          # [B, j, d]
            # least squares of T on the chosen atoms through the normal equations (j <= k is small); ridge for safety
            G = sel @ sel.transpose(1, 2)
            G = G + 1e-6 * G.diagonal(dim1=1, dim2=2).mean(dim=1).clamp_min(1e-12)[:, None, None] * torch.eye(G.shape[1], device=G.device)
            coef = torch.linalg.solve(G, (sel @ T[..., None])).squeeze(-1)                   # [B, j]
            R = T - torch.einsum("bj,bjd->bd", coef, sel)
        atom_ids = torch.gather(cand, 1, chosen)                                             # [B, k] indices into the shared set
        out[s:s + B] = torch.einsum("bj,bjd->bd", coef, atoms_out.float()[atom_ids])
    return out


def subword_rows(new_tokens: Sequence[str], encode, embed: torch.Tensor) -> torch.Tensor:
    """Mean of the student's embeddings of the pieces its own tokenizer cuts each new token's text into."""
    out = torch.zeros(len(new_tokens), embed.shape[1], dtype=torch.float32)
    mean = embed.float().mean(0)
    for i, t in enumerate(new_tokens):
        ids = [j for j in encode(t) if 0 <= j < embed.shape[0]]
        out[i] = embed[ids].float().mean(0) if ids else mean
    return out


def rebuild_matrix(student: torch.Tensor, teacher: Optional[torch.Tensor], s_vocab: Dict[str, int], t_vocab: Dict[str, int], rows: int,
                   method: str = "omp", k: int = 64, candidates: int = 1024, device: Optional[str] = None, encode=None, text_of=None) -> Tuple[torch.Tensor, Dict[str, int]]:
    """The student's matrix re-indexed by the teacher's vocabulary: ``rows`` x d_student.  ``subword`` needs ``text_of(teacher id)
    -> text`` and ``encode(text) -> student ids``."""
    dt = student.dtype
    out = torch.zeros(rows, student.shape[1], dtype=torch.float32)
    shared = [(t_vocab[tok], s_vocab[tok]) for tok in t_vocab if tok in s_vocab and s_vocab[tok] < student.shape[0] and t_vocab[tok] < rows]
    t_ids = torch.tensor([a for a, _ in shared], dtype=torch.long)
    s_ids = torch.tensor([b for _, b in shared], dtype=torch.long)
    out[t_ids] = student[s_ids].float()
    have = torch.zeros(rows, dtype=torch.bool)
    have[t_ids] = True
    new_ids = (~have).nonzero().squeeze(1)
    stats = {"rows": rows, "shared": len(shared), "new": int(new_ids.numel())}
    if new_ids.numel() == 0:
        return out.to(dt), stats
    mean_row = student.float().mean(0)
    if method == "zero":
        pass
    elif method == "mean" or not shared:
        out[new_ids] = mean_row
    elif method == "subword":
        if encode is None or text_of is None:
            raise ValueError("subword needs both tokenizers")
        out[new_ids] = subword_rows([text_of(int(i)) for i in new_ids], encode, student)
    elif method == "omp":
        if teacher is None:
            raise ValueError("omp needs the teacher's matrix as the reference space")
        in_teacher = new_ids[new_ids < teacher.shape[0]]
        dev = torch.device(device) if device else torch.device("cpu")
        ok = t_ids < teacher.shape[0]
        fit = omp_rows(teacher[in_teacher].to(dev), teacher[t_ids[ok]].to(dev), student[s_ids[ok]].to(dev), k, candidates).cpu()
        out[in_teacher] = fit
        rest = new_ids[new_ids >= teacher.shape[0]]  # padding rows beyond the teacher's matrix
        out[rest] = mean_row
    else:
        raise ValueError(f"unknown method '{method}' for the built-in engine ({', '.join(BUILTIN_METHODS)})")
    return out.to(dt), stats


# ---------------------------------------------------------------------- model directories
def _weight_files(model_dir: str) -> List[str]:
    return sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors") and "adapter" not in f)


def _find(model_dir: str, keys: Sequence[str]) -> Tuple[Optional[str], Optional[str]]:
    from safetensors import safe_open

    for fn in _weight_files(model_dir):
        with safe_open(os.path.join(model_dir, fn), framework="pt") as f:
            names = set(f.keys())
        for k in keys:
            if k in names:
                return fn, k
    return None, None


def _read(model_dir: str, fn: str, key: str) -> torch.Tensor:
    from safetensors import safe_open

    with safe_open(os.path.join(model_dir, fn), framework="pt") as f:
        return f.get_tensor(key)


def resolve_model_dir(model: str) -> str:
    if os.path.isdir(model):
        return model
    from ..hub import download_model

    return download_model(model)


def validate_output_model(out_dir: str) -> Dict[str, Any]:
    """The transplanted directory must be loadable: config, tokenizer and at least one weight file, with an embedding that
    covers the tokenizer."""
    for need in ("config.json", "tokenizer.json"):
        if not os.path.exists(os.path.join(out_dir, need)):
            raise RuntimeError(f"transplant output {out_dir} lacks {need}")
    if not _weight_files(out_dir):
        raise RuntimeError(f"transplant output {out_dir} has no safetensors weights")
    with open(os.path.join(out_dir, "config.json")) as f:
        cfg = json.load(f)
    vocab = load_vocab(out_dir)
    size = int((cfg.get("text_config") or cfg).get("vocab_size", 0))
    if vocab and size < max(vocab.values()) + 1:
        raise RuntimeError(f"config vocab_size {size} does not cover the tokenizer's largest id {max(vocab.values())}")
    return cfg


def builtin_transplant(student_dir: str, teacher_dir: str, out_dir: str, method: str = "omp", k: int = 64, device: Optional[str] = None,
                       candidates: int = 1024) -> Dict[str, Any]:
    from safetensors import safe_open
    from safetensors.torch import save_file

    if method not in BUILTIN_METHODS:
        raise ValueError(f"unknown method '{method}' for the built-in engine ({', '.join(BUILTIN_METHODS)}); the mergekit engine also has "
                         f"{', '.join(m for m in MERGEKIT_METHODS if m not in BUILTIN_METHODS)}")
    if k < 1:
        raise ValueError(f"k must be >= 1, got {k}")
    s_vocab, t_vocab = load_vocab(student_dir), load_vocab(teacher_dir)
    rows = vocab_size_of(teacher_dir, t_vocab)
    s_embed_file, s_embed_key = _find(student_dir, EMBED_KEYS)
    if s_embed_key is None:
        raise RuntimeError(f"no embedding matrix ({', '.join(EMBED_KEYS)}) in {student_dir}")
    s_head_file, s_head_key = _find(student_dir, HEAD_KEYS)
    t_embed_file, t_embed_key = _find(teacher_dir, EMBED_KEYS)
    t_head_file, t_head_key = _find(teacher_dir, HEAD_KEYS)
    encode = text_of = None
    if method == "subword":
        from ..data.tokenizer import Tokenizer

        s_tok, t_tok = Tokenizer.from_pretrained(student_dir), Tokenizer.from_pretrained(teacher_dir)
        known = set(t_vocab.values())
        encode = s_tok.encode_ordinary
        text_of = lambda i: t_tok.decode([i]) if i in known else ""  # noqa: E731
    t_embed = _read(teacher_dir, t_embed_file, t_embed_key) if (t_embed_key and method == "omp") else None
    new_embed, stats = rebuild_matrix(_read(student_dir, s_embed_file, s_embed_key), t_embed, s_vocab, t_vocab, rows, method, k, candidates, device, encode, text_of)
    new_head = None
    if s_head_key is not None:
        t_head = (_read(teacher_dir, t_head_file, t_head_key) if t_head_key else t_embed) if method == "omp" else None
        new_head, _ = rebuild_matrix(_read(student_dir, s_head_file, s_head_key), t_head, s_vocab, t_vocab, rows, method, k, candidates, device, encode, text_of)

    os.makedirs(out_dir, exist_ok=True)
    for fn in sorted(os.listdir(student_dir)):
        src = os.path.join(student_dir, fn)
        if fn.endswith(".safetensors") and "adapter" not in fn:
            tensors = {}
            with safe_open(src, framework="pt") as f:
                meta = f.metadata() or {"format": "pt"}
                for key in f.keys():
                    t = f.get_tensor(key)
                    if fn == s_embed_file and key == s_embed_key:
                        t = new_embed
                    elif new_head is not None and fn == s_head_file and key == s_head_key:
                        t = new_head
                    tensors[key] = t.contiguous()
            save_file(tensors, os.path.join(out_dir, fn), metadata=meta)
        elif os.path.isfile(src) and fn not in TOKENIZER_FILES and fn != MANIFEST:
            shutil.copy2(src, os.path.join(out_dir, fn))
    for fn in TOKENIZER_FILES:  # the teacher's tokenizer, chat template and special-token ids
        if fn != "generation_config.json" and os.path.exists(os.path.join(teacher_dir, fn)):
            shutil.copy2(os.path.join(teacher_dir, fn), os.path.join(out_dir, fn))
    with open(os.path.join(student_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(teacher_dir, "config.json")) as f:
        t_cfg = json.load(f)
    tgt, src_cfg = (cfg.get("text_config") or cfg), (t_cfg.get("text_config") or t_cfg)
    tgt["vocab_size"] = rows
    for key in ("bos_token_id", "eos_token_id", "pad_token_id"):
        if key in src_cfg:
            tgt[key] = src_cfg[key]
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    index = os.path.join(out_dir, "model.safetensors.index.json")
    if os.path.exists(index):  # total size changed with the two matrices
        with open(index) as f:
            ix = json.load(f)
        ix.setdefault("metadata", {})["total_size"] = sum(os.path.getsize(os.path.join(out_dir, fn)) for fn in _weight_files(out_dir))
        with open(index, "w") as f:
            json.dump(ix, f, indent=2)
    return stats


# ---------------------------------------------------------------------- mergekit engine
def find_tokensurgeon() -> Optional[List[str]]:
    if shutil.which("mergekit-tokensurgeon"):
        return ["mergekit-tokensurgeon"]
    return None


def mergekit_command(base: str, donor: str, out_dir: str, method: str = "omp", k: int = 64, device: Optional[str] = None, trust_remote_code: bool = False,
                     extra: Optional[Sequence[str]] = None, exe: Sequence[str] = ("mergekit-tokensurgeon",)) -> List[str]:
    if method not in MERGEKIT_METHODS:
        raise ValueError(f"unknown approximation method '{method}' ({', '.join(MERGEKIT_METHODS)})")
    if k < 1:
        raise ValueError(f"k must be >= 1, got {k}")
    cmd = list(exe) + [base, donor, out_dir, "--approximation-method", method, "--k", str(k)]
    if device:
        cmd += ["--device", device]
    if trust_remote_code:
        cmd += ["--trust-remote-code"]
    return cmd + list(extra or [])


def _run(base_dir: str, donor_dir: str, out_dir: str, method: str, k: int, device: Optional[str], trust_remote_code: bool, extra, engine: str,
         runner=subprocess.run) -> Dict[str, Any]:
    exe = find_tokensurgeon() if engine in ("auto", "mergekit") else None
    if engine == "mergekit" and exe is None:
        raise RuntimeError("mergekit-tokensurgeon was not found on PATH (pip install mergekit, in an environment of its own if its pins clash); "
                           "`--engine builtin` needs no external tool")
    if exe is not None and (engine == "mergekit" or method not in BUILTIN_METHODS):
        cmd = mergekit_command(base_dir, donor_dir, out_dir, method, k, device, trust_remote_code, extra, exe)
        r = runner(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            tail = (r.stderr or r.stdout or "").strip().splitlines()[-15:]
            raise RuntimeError(f"mergekit-tokensurgeon failed (exit {r.returncode}):\n" + "\n".join(tail))
        return {"engine": "mergekit", "command": cmd}
    return dict(builtin_transplant(base_dir, donor_dir, out_dir, method, k, device), engine="builtin")


def run_transplant(student_model: str, teacher_model: str, out_dir: str, method: str = "omp", k: int = 64, device: Optional[str] = None,
                   trust_remote_code: bool = False, extra_args: Optional[Sequence[str]] = None, engine: str = "auto", runner=subprocess.run) -> Dict[str, Any]:
    """The teacher's tokenizer on the student: ``out_dir`` holds the student's weights with embedding / LM-head rows rebuilt for
    the teacher's vocabulary, the teacher's tokenizer files and the manifest.  ``engine``: auto (built-in for the methods it
    has, else mergekit) | builtin | mergekit."""
    student_dir, teacher_dir = resolve_model_dir(student_model), resolve_model_dir(teacher_model)
    info = _run(student_dir, teacher_dir, out_dir, method, k, device, trust_remote_code, extra_args, engine, runner)
    validate_output_model(out_dir)
    manifest = {"version": 1, "student_model": student_model, "student_dir": os.path.abspath(student_dir), "teacher_model": teacher_model,
                "teacher_dir": os.path.abspath(teacher_dir), "method": method, "k": k, "engine": info["engine"], "created_unix": int(time.time())}
    with open(os.path.join(out_dir, MANIFEST), "w") as f:
        json.dump(manifest, f, indent=2)
    return dict(info, out_dir=out_dir, manifest=os.path.join(out_dir, MANIFEST))


def run_transplant_back(distilled_model: str, manifest_path: str, out_dir: str, device: Optional[str] = None, trust_remote_code: bool = False,
                        extra_args: Optional[Sequence[str]] = None, engine: str = "auto", runner=subprocess.run) -> Dict[str, Any]:
    """A distilled model (teacher vocabulary) back on the original student's tokenizer; the original student is the donor.  A short
    fine-tune on data in the native chat template afterwards is advisable: template semantics move back with the tokenizer."""
    with open(manifest_path) as f:
        manifest = json.load(f)
    donor = manifest.get("student_dir") or manifest.get("student_model")
    if not donor:
        raise ValueError(f"manifest {manifest_path} names no student model")
    if not os.path.isdir(donor):
        donor = resolve_model_dir(manifest["student_model"])
    info = _run(resolve_model_dir(distilled_model), donor, out_dir, manifest.get("method", "omp"), int(manifest.get("k", 64)), device, trust_remote_code,
                extra_args, engine, runner)
    validate_output_model(out_dir)
    return dict(info, out_dir=out_dir)

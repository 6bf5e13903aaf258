"""Introspection helpers that write JSON-lines reports.

* ``audit_weights``   — static comparison of a checkpoint's tensor names / shapes with what the DSL model maps.
* ``registry_report`` — architectures, parameters, ops of the forward / backward graphs.
* ``activation_stats`` / ``gradient_stats`` — per-tensor mean / std / abs-max / non-finite counts for one batch.
* ``diff_against_transformers`` — layer-by-layer hidden-state comparison with the HuggingFace implementation.

Parity: surogate/debug/{weights,registry,activations,gradients,diff,tensor_*}.py, cli/debug.py.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterable, List, Optional

import numpy as np
import torch


def _stats(t: torch.Tensor) -> Dict[str, float]:
    f = t.detach().float()
    finite = torch.isfinite(f)
    g = f[finite] if not bool(finite.all()) else f
    return {"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", ""), "mean": float(g.mean()) if g.numel() else 0.0,
            "std": float(g.std()) if g.numel() > 1 else 0.0, "absmax": float(g.abs().max()) if g.numel() else 0.0,
            "nonfinite": int((~finite).sum()), "norm": float(g.norm()) if g.numel() else 0.0}


def write_jsonl(path: Optional[str], rows: Iterable[Dict[str, Any]]) -> List[Dict[str, Any]]:
    rows = list(rows)
    if path:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    return rows


def audit_weights(model_dir: str, out: Optional[str] = None) -> Dict[str, Any]:
    from ..dsl.compiler import compile_model, load_hf_config, model_from_hf_config
    from ..io.hf_checkpoint import LazyCheckpoint

    cfg = load_hf_config(model_dir)
    cm = compile_model(model_from_hf_config(cfg))
    ckpt = LazyCheckpoint(model_dir)
    have = set(ckpt.names())
    used, missing, rows = set(), [], []
    for p in cm.params:
        m = p.spec.hf
        if m is None or p.tied_to:
            continue
        names = m.hf_names(p.layer)
        absent = [n for n in names if n not in have]
        used.update(n for n in names if n in have)
        rows.append({"param": p.name, "hf": names, "shape": list(p.spec.shape), "status": "missing" if absent else "ok", "absent": absent})
        if absent:
            missing.append(p.name)
    unused = sorted(have - used)
    rows.append({"summary": True, "mapped": len(rows), "missing": missing, "unused_checkpoint_tensors": unused})
    write_jsonl(out, rows)
    return {"mapped": len(rows) - 1, "missing": missing, "unused": unused}


def registry_report(arch_or_dir: Optional[str] = None, out: Optional[str] = None) -> List[Dict[str, Any]]:
    from ..dsl import models  # noqa: F401
    from ..dsl.nn import registered_architectures, registered_models

    rows: List[Dict[str, Any]] = [{"architectures": registered_architectures()}]
    if arch_or_dir:
        from ..dsl.compiler import compile_model, load_hf_config, model_from_hf_config

        if os.path.isdir(arch_or_dir):
            cm = compile_model(model_from_hf_config(load_hf_config(arch_or_dir)))
            rows += [{"param": p.name, "shape": list(p.spec.shape), "layer": p.layer, "group": p.group, "tied_to": p.tied_to} for p in cm.params]
            for gname, g in [("forward", cm.fwd), ("backward", cm.bwd)] + [(f"block:{k}", v) for k, v in cm.block_fwd.items()]:
                rows.append({"graph": gname, "ops": [op.kind for op in g.ops]})
        else:
            rows.append({"model_class": registered_models()[arch_or_dir].__name__})
    return write_jsonl(out, rows)


def activation_stats(trainer, inputs: np.ndarray, targets: np.ndarray, out: Optional[str] = None) -> List[Dict[str, Any]]:
    rows: List[Dict[str, Any]] = []

    def hook(name, layer, val):
        if torch.is_tensor(val) and val.is_floating_point():
            rows.append({"tensor": name, "layer": layer, **_stats(val)})

    prev = trainer.executor.options.dump_tensors
    trainer.executor.options.dump_tensors = hook
    try:
        trainer.validate(inputs, targets)
    finally:
        trainer.executor.options.dump_tensors = prev
    return write_jsonl(out, rows)


def gradient_stats(trainer, inputs: np.ndarray, targets: np.ndarray, out: Optional[str] = None, steps: int = 1) -> List[Dict[str, Any]]:
    """Per-parameter gradient statistics; with ``steps`` > 1 an optimizer update follows each capture, so degradation after a few
    updates shows (rows carry ``step``)."""
    rows: List[Dict[str, Any]] = []
    for step in range(max(1, steps)):
        trainer.forward_backward(inputs, targets)
        now = [{"step": step, "param": name, **_stats(g)} for name, g in trainer.get_gradients().items() if g is not None]
        if getattr(trainer, "lora", None) is not None:  # the base is frozen under LoRA: the adapters carry the gradients
            now += [{"step": step, "param": name, **_stats(g)} for name, g in trainer.lora.named_grads()]
        now.sort(key=lambda r: -r["absmax"])
        rows += now
        if step + 1 < steps:
            trainer.optimizer_step()
        else:
            trainer.store.release_grads()
    return write_jsonl(out, rows)


def diff_against_transformers(model_dir: str, tokens: np.ndarray, device: str = "cpu", out: Optional[str] = None, backend: str = "auto",
                              reference: Optional[str] = None, rtol: float = 1e-2, atol: float = 1e-3):
    """Hidden state after every block (and the logits) from both implementations on the same tokens.  ``reference``: the
    transformers model to compare with (default: ``model_dir``).  Rows carry ``diverged`` by the allclose rule
    ``|a - b| <= atol + rtol |b|`` and the report ends with the first layer that diverged."""
    from transformers import AutoModelForCausalLM

    from ..dsl.compiler import load_hf_config
    from ..runtime.trainer import Trainer, TrainerConfig

    hf = AutoModelForCausalLM.from_pretrained(reference or model_dir, torch_dtype=torch.float32).to(device).eval()
    with torch.no_grad():
        ref = hf(torch.from_numpy(tokens.astype(np.int64)).to(device), output_hidden_states=True)
    cfg = load_hf_config(model_dir)
    tr = Trainer(TrainerConfig(model=cfg, batch_size=tokens.shape[0], seq_len=tokens.shape[1], zero_level=0, backend=backend, param_dtype="fp32" if device == "cpu" else "bf16"),
                 device=torch.device(device))
    tr.import_weights(model_dir)
    mine: Dict[int, torch.Tensor] = {}

    def hook(name, layer, val):
        if layer is not None and name in ("x_out", "residual_out") and torch.is_tensor(val):
            mine.setdefault(layer, {})[name] = val.detach().float()

    prev = tr.executor.options.dump_tensors
    tr.executor.options.dump_tensors = hook
    try:
        logits = tr.logits(tokens)
    finally:
        tr.executor.options.dump_tensors = prev
    rows = []
    for L in sorted(mine):
        h = sum(mine[L].values())  # block output = deferred residual stream + last branch output
        r = ref.hidden_states[L + 1].float()
        if L == len(mine) - 1 and r.shape == h.shape and (r - h).abs().max() > 1.0:
            continue  # transformers applies the final norm to the last hidden state
        rows.append({"layer": L, "max_abs_diff": float((h - r).abs().max()), "rel": float((h - r).norm() / (r.norm() + 1e-12)),
                     "diverged": not bool(torch.allclose(h, r, rtol=rtol, atol=atol))})
    rl = ref.logits.float()
    rows.append({"logits": True, "max_abs_diff": float((logits - rl).abs().max()), "rel": float((logits - rl).norm() / (rl.norm() + 1e-12)),
                 "diverged": not bool(torch.allclose(logits.float(), rl, rtol=rtol, atol=atol))})
    rows.append({"summary": True, "first_diverged_layer": next((r["layer"] for r in rows if r.get("diverged") and "layer" in r), None), "rtol": rtol, "atol": atol})
    return write_jsonl(out, rows)


def determinism_report(make_trainer, inputs: np.ndarray, targets: np.ndarray, steps: int = 2, out: Optional[str] = None) -> Dict[str, Any]:
    """Run the same ``steps`` optimizer steps twice from the same seed and compare, step by step, the loss, the gradient norm
    and (after the last step's forward + backward) every parameter gradient.  On the PyTorch backend the two runs are identical
    bit for bit.  The CUDA kernels accumulate a few gradients with atomics (embedding rows, norm weights), so small differences
    there are expected; a large relative difference in any other tensor points at a race or at uninitialised memory.
    ``make_trainer()`` must return a freshly initialised trainer each time.
    Parity: the reference's deterministic-replay self-checks (SUROGATE_CHECK_REPLAY_SCOPE and friends)."""
    runs = []
    for _ in range(2):
        tr = make_trainer()
        hist = [tr.step(inputs, targets) for _ in range(max(0, steps - 1))]
        r = tr.forward_backward(inputs, targets)
        hist.append({"loss": float(r["loss_sum"] / r["n_valid"].clamp_min(1.0) if torch.is_tensor(r["n_valid"]) else r["loss_sum"] / max(1.0, r["n_valid"])),
                     "norm": float(tr.grad_norm())})
        runs.append((hist, {k: v.detach().float().cpu().clone() for k, v in tr.get_gradients().items()}))
    (ha, ga), (hb, gb) = runs
    rows = []
    for name in ga:
        den = float(ga[name].norm()) + 1e-30
        rows.append({"param": name, "max_abs_diff": float((ga[name] - gb[name]).abs().max()), "rel_diff": float((ga[name] - gb[name]).norm()) / den,
                     "bitwise_equal": bool(torch.equal(ga[name], gb[name]))})
    rows.sort(key=lambda r: -r["rel_diff"])
    write_jsonl(out, rows)
    return {"steps": [{"loss_a": a["loss"], "loss_b": b["loss"], "norm_a": a["norm"], "norm_b": b["norm"]} for a, b in zip(ha, hb)],
            "bitwise_equal": all(r["bitwise_equal"] for r in rows) and all(a["loss"] == b["loss"] for a, b in zip(ha, hb)),
            "worst": rows[:5], "n_params": len(rows)}

"""Step checkpoints: per-rank shards of weights and optimizer state + run metadata.

Layout: ``<dir>/step_%08d/`` with ``weights.shard_RRR_of_NNN.safetensors``, ``adam.m.shard_*``, ``adam.v.shard_*`` and, for
8-bit state, ``adam.m.scales.*`` / ``adam.v.scales.*`` (the reference's directory and file names); ``rng.rank_RRR.pt`` holds each
rank's complete CPU and CUDA generator state; ``checkpoint.json`` (written by rank 0 once every rank has reported a successful
write) holds run state, the data-loader cursor and the distributed shape.  Inside the files there is ONE flat tensor per
parameter bucket, keyed by bucket name: the files are this framework's own and are not interchangeable with the reference's
per-parameter checkpoints (``export_model`` writes HF-format weights for that).  LoRA runs store the adapter, its optimizer
state and only the TRAINABLE base buckets; frozen (possibly block-quantised) base weights are re-imported or re-initialised
from the seed before the checkpoint is applied.  Loading under a different world size is supported: shards are re-cut from
the flat bucket layout (padding included) because every rank's slice is a contiguous range.

A write error on any rank (full disk, lost mount) fails the checkpoint on ALL ranks together: every rank runs the same
sequence of collectives whether or not its own write succeeded, nobody writes ``checkpoint.json``, and
``CheckpointWriteError`` is raised everywhere.

Parity: csrc/src/runtime/training/checkpoint.cpp:31-380 (save :56, load :186, retention :317-380).
"""
from __future__ import annotations

import glob
import json
import os
import re
import shutil
from typing import Any, Dict, List, Optional

import torch
from safetensors import safe_open
from safetensors.torch import save_file

STEP_RE = re.compile(r"step_(\d{8})$")


def step_dir(root: str, step: int) -> str:
    return os.path.join(root, f"step_{step:08d}")


def find_latest_checkpoint(root: str) -> Optional[int]:
    best = None
    for d in glob.glob(os.path.join(root, "step_*")):
        m = STEP_RE.search(d)
        if m and os.path.exists(os.path.join(d, "checkpoint.json")):
            best = max(best or -1, int(m.group(1)))
    return best


def clean_old_checkpoints(root: str, keep: int, major_every: int = 0) -> List[int]:
    """Keep the newest ``keep`` checkpoints (and every ``major_every``-th step); returns the removed steps."""
    steps = sorted(int(STEP_RE.search(d).group(1)) for d in glob.glob(os.path.join(root, "step_*")) if STEP_RE.search(d))
    removed = []
    for s in steps[:-keep] if keep > 0 else []:
        if major_every and s % major_every == 0:
            continue
        shutil.rmtree(step_dir(root, s), ignore_errors=True)
        removed.append(s)
    return removed


def _shard_name(kind: str, rank: int, world: int) -> str:
    return f"{kind}.shard_{rank:03d}_of_{world:03d}.safetensors"


class CheckpointWriteError(OSError):
    """Raised on every rank when at least one rank could not write its part of a checkpoint."""


def _write_rank_files(trainer, d: str) -> None:
    os.makedirs(d, exist_ok=True)
    store, opt = trainer.store, trainer.optimizer
    rank, world = trainer.rank, trainer.world
    shard_world = world if store.sharded else 1
    if store.sharded or rank == 0:
        r = rank if store.sharded else 0
        adapter_only = trainer.lora is not None
        weights = {b.name: b.master.detach().cpu().contiguous() for b in store.buckets.values() if b.trainable or not adapter_only}
        if not weights:  # safetensors needs at least the header; an empty file still marks the shard as written
            weights = {"__empty__": torch.zeros(1)}
        save_file(weights, os.path.join(d, _shard_name("weights", r, shard_world)))
        kinds: Dict[str, Dict[str, torch.Tensor]] = {}
        for b in store.trainable_buckets():
            for k, t in opt.state_tensors(b).items():
                kinds.setdefault(k, {})[b.name] = t.detach().cpu().contiguous()
        for k, tensors in kinds.items():
            save_file(tensors, os.path.join(d, _shard_name(f"adam.{k}", r, shard_world)))
        extra_state = getattr(opt, "mom", None)
        if extra_state:
            save_file({k: v.cpu() for k, v in {**opt.mom, **{f"second::{k}": v for k, v in opt.second.items()}}.items()},
                      os.path.join(d, _shard_name("normuon", r, shard_world)))
    if trainer.lora is not None:
        trainer.lora.save_state(d, rank)
    rng = {"cpu": torch.get_rng_state()}
    if store.device.type == "cuda":
        rng["cuda"] = torch.cuda.get_rng_state(store.device)
    torch.save(rng, os.path.join(d, f"rng.rank_{rank:03d}.pt"))
    rs = trainer.recipe.state_dict()
    if rs and rank == 0:
        torch.save({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in rs.items()}, os.path.join(d, "recipe_state.pt"))


def save_checkpoint(trainer, root: str, step: int, extra: Dict[str, Any]) -> str:
    d = step_dir(root, step)
    store = trainer.store
    rank, world = trainer.rank, trainer.world
    error: Optional[BaseException] = None
    try:
        _write_rank_files(trainer, d)
    except OSError as e:  # kept until every rank has voted, so the ranks stay on the same collective sequence
        error = e
    failed = torch.tensor([0.0 if error is None else 1.0], dtype=torch.float32, device=store.device)
    if world > 1:
        trainer.comm.all_reduce(failed, "sum")  # doubles as the barrier before rank 0 publishes the checkpoint
    n_failed = int(failed.item())
    if n_failed == 0 and rank == 0:
        try:
            meta = {
                "run": {"step": step, "optimizer_step": trainer.step_index, "past_losses": extra.get("past_losses", []),
                        "past_norms": extra.get("past_norms", [])},
                "data-loader": extra.get("data_loader", {}),
                "distributed": {"world": world, "ep_size": trainer.cfg.ep_size, "zero_level": store.zero_level, "sharded": store.sharded},
                "layout": {b.name: {"numel": b.numel, "shard_numel": b.shard_numel} for b in store.buckets.values()},
                "optimizer": trainer.cfg.optimizer, "recipe": trainer.cfg.recipe,
                "frozen_base_omitted": trainer.lora is not None,
                # which (rank, slot) holds each global expert of each layer (identity unless experts were re-placed for load balance)
                "ep_placement": {str(k): v for k, v in getattr(trainer.store, "expert_placement", {}).items()},
            }
            tmp = os.path.join(d, "checkpoint.json.tmp")
            with open(tmp, "w") as f:
                json.dump(meta, f, indent=1)
            os.replace(tmp, os.path.join(d, "checkpoint.json"))  # atomic: a directory without checkpoint.json is incomplete
        except OSError as e:
            error = e
    published = torch.tensor([1.0 if (rank == 0 and n_failed == 0 and error is None) else 0.0], dtype=torch.float32, device=store.device)
    if world > 1:
        trainer.comm.all_reduce(published, "sum")  # second rendezvous: nobody returns before checkpoint.json exists (or is known not to)
    if n_failed or published.item() < 1:
        why = f"{n_failed} of {world} ranks could not write their shard" if n_failed else "rank 0 could not write checkpoint.json"
        raise CheckpointWriteError(f"checkpoint step {step} abandoned on all ranks: {why}" + (f" (this rank: {error})" if error else ""))
    return d


def _read_flat(d: str, kind: str, bucket: str, saved_world: int, lo: int, hi: int, shard_numel: int) -> torch.Tensor:
    """Elements [lo, hi) of a bucket-flat tensor reassembled from the shards saved under ``saved_world``."""
    parts = []
    for r in range(saved_world):
        a, z = r * shard_numel, (r + 1) * shard_numel
        if z <= lo or a >= hi:
            continue
        with safe_open(os.path.join(d, _shard_name(kind, r, saved_world)), framework="pt") as f:
            t = f.get_tensor(bucket)
        parts.append(t[max(lo, a) - a:min(hi, z) - a])
    return torch.cat(parts) if len(parts) != 1 else parts[0]


def load_checkpoint(trainer, root: str, step: Optional[int] = None) -> Dict[str, Any]:
    if step is None:
        step = find_latest_checkpoint(root)
        if step is None:
            raise FileNotFoundError(f"no complete checkpoint under {root}")
    d = step_dir(root, step)
    with open(os.path.join(d, "checkpoint.json")) as f:
        meta = json.load(f)
    dist_meta = meta["distributed"]
    if dist_meta.get("ep_size", 1) != trainer.cfg.ep_size:
        raise ValueError(f"checkpoint was written with ep_size={dist_meta.get('ep_size')} but the run uses {trainer.cfg.ep_size}")
    saved_world = dist_meta["world"] if dist_meta.get("sharded") else 1
    store, opt = trainer.store, trainer.optimizer
    placement = {int(k): list(v) for k, v in (meta.get("ep_placement") or {}).items()}
    if placement and trainer.ep is not None:
        store.expert_placement = dict(placement)
        trainer.ep.placement_host = dict(placement)
        trainer.ep.placement = {L: torch.tensor(v, dtype=torch.int32, device=store.device) for L, v in placement.items()}
    for b in store.buckets.values():
        lay = meta["layout"][b.name]
        if not b.trainable and meta.get("frozen_base_omitted"):
            continue  # adapter-only checkpoint: the frozen base is whatever the caller imported / re-initialised
        if b.expert:  # whole experts live on one rank: each rank reads back exactly what it wrote
            if dist_meta["world"] != trainer.world:
                raise ValueError("expert-parallel checkpoints must be loaded with the world size they were written with")
            with safe_open(os.path.join(d, _shard_name("weights", trainer.rank, saved_world)), framework="pt") as f:
                b.master.copy_(f.get_tensor(b.name).to(b.master.dtype))
            for k, t in opt.state_tensors(b).items():
                fn = os.path.join(d, _shard_name(f"adam.{k}", trainer.rank, saved_world))
                if os.path.exists(fn):
                    with safe_open(fn, framework="pt") as f:
                        if b.name in f.keys():
                            t.copy_(f.get_tensor(b.name).to(t.dtype))
            continue
        lo, hi = store.shard_range(b)
        total_saved = lay["shard_numel"] * saved_world
        hi_c = min(hi, total_saved)
        w = _read_flat(d, "weights", b.name, saved_world, lo, hi_c, lay["shard_numel"])
        b.master[: hi_c - lo].copy_(w.to(b.master.dtype))
        if not b.trainable:
            continue
        for k, t in opt.state_tensors(b).items():
            kind = f"adam.{k}"
            if not os.path.exists(os.path.join(d, _shard_name(kind, 0, saved_world))):
                continue
            per = 32 if k.endswith("scales") else 1
            if per == 32 and (lo % 32 or lay["shard_numel"] % 32):
                raise ValueError("8-bit optimizer scales cannot be re-sharded at this alignment")
            s = _read_flat(d, kind, b.name, saved_world, lo // per, (hi_c + per - 1) // per, max(1, lay["shard_numel"] // per))
            t[: s.numel()].copy_(s.to(t.dtype))
    nm = os.path.join(d, _shard_name("normuon", trainer.rank if store.sharded else 0, saved_world))
    if hasattr(opt, "mom") and os.path.exists(nm):
        with safe_open(nm, framework="pt") as f:
            for k in f.keys():
                (opt.second if k.startswith("second::") else opt.mom)[k.replace("second::", "")] = f.get_tensor(k).to(store.device)
    if trainer.lora is not None:
        trainer.lora.load_state(d, trainer.rank)
    rng_file = os.path.join(d, f"rng.rank_{trainer.rank:03d}.pt")
    if os.path.exists(rng_file) and dist_meta["world"] == trainer.world:
        rng = torch.load(rng_file, map_location="cpu")
        torch.set_rng_state(rng["cpu"])
        if "cuda" in rng and store.device.type == "cuda":
            torch.cuda.set_rng_state(rng["cuda"], store.device)
    rp = os.path.join(d, "recipe_state.pt")
    if os.path.exists(rp):
        trainer.recipe.load_state_dict(torch.load(rp, map_location=store.device))
    trainer.step_index = meta["run"].get("optimizer_step", step)
    store.sync_work_from_master()
    trainer.recipe.on_weights_updated(store)
    return meta

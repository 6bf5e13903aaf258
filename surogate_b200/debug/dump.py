"""Dump named activations of a run to files, switched on by the environment (no code change, works under every command):

    SUROGATE_DEBUG_DUMP_TENSORS   comma-separated names: ``blocks[3].ln1`` (one layer), ``ln1`` (every layer), ``loss`` (model level),
                                  ``d_blocks[3].d_ln1`` / ``d_ln1`` (backward graph), or ``all``
    SUROGATE_DEBUG_DUMP_DIR       where the files go (created)
    SUROGATE_DEBUG_DUMP_LAYER     optional: only this layer

Each tensor becomes ``<sanitised name>.bin`` (float32, C order) + ``<sanitised name>.json`` (``{"name", "dtype": "float32", "shape"}``); a
tensor produced several times (micro-batches, recomputation) keeps its last value.  Dumping synchronises the device at every dumped
tensor, so it is a debugging aid, not something to leave on.

Parity: csrc/src/runtime/executor/graph_executor.cpp:170-260 (debug_dump_tensor, the same file format and variables).
"""
from __future__ import annotations

import json
import os
import re
from typing import Callable, List, Optional, Set, Tuple

import numpy as np
import torch

NAME_RE = re.compile(r"^(d_)?blocks\[(\d+)\]\.(.+)$")


def sanitise(name: str) -> str:
    return "".join(c if (c.isalnum() or c in "_-.") else "_" for c in name)


def parse_names(text: str) -> Tuple[bool, Set[Tuple[Optional[int], str]]]:
    """(dump everything?, {(layer or None, tensor name)})."""
    wanted: Set[Tuple[Optional[int], str]] = set()
    everything = False
    for raw in (text or "").split(","):
        n = raw.strip()
        if not n:
            continue
        if n == "all":
            everything = True
            continue
        m = NAME_RE.match(n)
        wanted.add((int(m.group(2)), m.group(3)) if m else (None, n))
    return everything, wanted


def qualified(name: str, layer: Optional[int]) -> str:
    if layer is None:
        return name
    return f"{'d_' if name.startswith('d_') else ''}blocks[{layer}].{name}"


def dump_tensor(name: str, t: torch.Tensor, directory: str) -> str:
    os.makedirs(directory, exist_ok=True)
    base = os.path.join(directory, sanitise(name))
    arr = t.detach().float().cpu().contiguous().numpy()
    arr.astype(np.float32).tofile(base + ".bin")
    with open(base + ".json", "w") as f:
        json.dump({"name": name, "dtype": "float32", "shape": list(arr.shape)}, f)
    return base + ".bin"


def load_dump(directory: str, name: str) -> np.ndarray:
    base = os.path.join(directory, sanitise(name))
    with open(base + ".json") as f:
        meta = json.load(f)
    return np.fromfile(base + ".bin", dtype=np.float32).reshape(meta["shape"])


def env_dump_hook(environ=os.environ) -> Optional[Callable[[str, Optional[int], torch.Tensor], None]]:
    """The executor's ``dump_tensors`` hook for the variables above, or None when they are not set."""
    names, directory = environ.get("SUROGATE_DEBUG_DUMP_TENSORS"), environ.get("SUROGATE_DEBUG_DUMP_DIR")
    if not names or not directory:
        return None
    everything, wanted = parse_names(names)
    only = environ.get("SUROGATE_DEBUG_DUMP_LAYER")
    only_layer = int(only) if only not in (None, "") else None
    written: List[str] = []

    def hook(name: str, layer: Optional[int], val: torch.Tensor) -> None:
        if only_layer is not None and layer != only_layer:
            return
        if not (everything or (layer, name) in wanted or (None, name) in wanted):
            return
        if not val.is_floating_point():
            return
        written.append(dump_tensor(qualified(name, layer), val, directory))

    hook.written = written  # type: ignore[attr-defined]
    return hook

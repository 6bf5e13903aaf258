"""``surogate merge --base-model <model dir or hub id> --checkpoint-dir <adapter dir> --output <dir>``: fold a LoRA adapter into the
base weights.  ``--checkpoint-dir`` may be the adapter directory itself or a directory that holds one (``<output_dir>/adapter``);
``--base`` / ``--adapter`` are shorter spellings.

Parity: surogate/cli (merge command), surogate/utils/adapter_merge.py.
"""
from __future__ import annotations

import argparse
import json


def main(argv, command: str = "merge") -> int:
    p = argparse.ArgumentParser(prog="surogate merge")
    p.add_argument("--base-model", "--base", dest="base", required=True, help="base model directory or hub id")
    p.add_argument("--checkpoint-dir", "--adapter", dest="adapter", required=True, help="LoRA adapter directory (adapter_config.json + adapter_model.safetensors)")
    p.add_argument("--output", required=True)
    a = p.parse_args(argv)
    import os

    from ..utils.adapter_merge import merge_adapter

    base = a.base
    if not os.path.isdir(base):
        from ..hub import download_model

        base = download_model(base)
    adapter = a.adapter
    if not os.path.exists(os.path.join(adapter, "adapter_config.json")) and os.path.exists(os.path.join(adapter, "adapter", "adapter_config.json")):
        adapter = os.path.join(adapter, "adapter")
    print(json.dumps(merge_adapter(base, adapter, a.output)))
    return 0

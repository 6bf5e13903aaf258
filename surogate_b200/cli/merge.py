"""``surogate merge --base <model dir> --adapter <adapter dir> --output <dir>``: fold a LoRA adapter into the base weights.

Parity: surogate/cli (merge command), surogate/utils/adapter_merge.py.
"""
from __future__ import annotations

import argparse
import json


def main(argv, command: str = "merge") -> int:
    p = argparse.ArgumentParser(prog="surogate merge")
    p.add_argument("--base", required=True)
    p.add_argument("--adapter", required=True)
    p.add_argument("--output", required=True)
    a = p.parse_args(argv)
    from ..utils.adapter_merge import merge_adapter

    print(json.dumps(merge_adapter(a.base, a.adapter, a.output)))
    return 0

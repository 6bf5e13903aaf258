"""``surogate dpo config.yaml``.  Parity: surogate/cli (dpo command), surogate/dpo/trainer.py."""
from __future__ import annotations

import json
import os

from .sft import build_parser, take_hub_token


def main(argv, command: str = "dpo") -> int:
    a = build_parser(command).parse_args(argv)
    take_hub_token(a)
    from ..dpo.trainer import dpo_main

    r = dpo_main(a.config, **{k: v for k, v in vars(a).items() if k != "config" and v is not None})
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"steps": r["steps"], "final": r["history"][-1] if r["history"] else None}))
    return 0

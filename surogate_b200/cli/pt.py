"""``surogate pt config.yaml`` (pre-training).  Parity: surogate/cli/pt.py:13."""
from __future__ import annotations

from .sft import build_parser, launch


def main(argv, command: str = "pt") -> int:
    from ..train.sft import pt_main

    return launch(build_parser(command).parse_args(argv), command, pt_main)

"""``surogate`` command: argparse front end that dispatches to the workflow modules.

Commands: sft, pt, merge, tokenize, debug, dpo, grpo, grpo-infer, grpo-orch, grpo-train, grpo-colocate, distill-capture,
transplant-tokenizer, eval, export, chat, monitor, vf-init, vf-eval, info.

Parity: surogate/cli/main.py:42-58 (COMMAND_MAPPING), :193-204 (cli_main).
"""
from __future__ import annotations

import argparse
import importlib
import os
import sys
from typing import Dict, List, Optional

COMMAND_MAPPING: Dict[str, str] = {
    "sft": "surogate_b200.cli.sft",
    "pt": "surogate_b200.cli.pt",
    "merge": "surogate_b200.cli.merge",
    "tokenize": "surogate_b200.cli.tokenize",
    "debug": "surogate_b200.cli.debug",
    "dpo": "surogate_b200.cli.dpo",
    "grpo": "surogate_b200.cli.grpo",
    "grpo-infer": "surogate_b200.cli.grpo",
    "grpo-orch": "surogate_b200.cli.grpo",
    "grpo-train": "surogate_b200.cli.grpo",
    "grpo-colocate": "surogate_b200.cli.grpo",
    "distill-capture": "surogate_b200.cli.distill",
    "transplant-tokenizer": "surogate_b200.cli.transplant",
    "export": "surogate_b200.cli.export",
    "eval": "surogate_b200.cli.eval",
    "info": "surogate_b200.cli.info",
    "chat": "surogate_b200.cli.chat",
    "monitor": "surogate_b200.cli.monitor",
    "launch": "surogate_b200.cli.launch",
    "jackalope": "surogate_b200.cli.monitor",  # the dashboard's name in the reference
    "vf-init": "surogate_b200.cli.vf",
    "vf-eval": "surogate_b200.cli.vf",
}

BANNER = r"""
  ___ _   _ _ __ ___   __ _  __ _| |_ ___    | |__|___ \ / _ \ / _ \
 / __| | | | '__/ _ \ / _` |/ _` | __/ _ \   | '_ \ __) | | | | | | |
 \__ \ |_| | | | (_) | (_| | (_| | ||  __/ _ | |_) / __/| |_| | |_| |
 |___/\__,_|_|  \___/ \__, |\__,_|\__\___|(_)|_.__/_____|\___/ \___/
                      |___/        Blackwell-native LLM training
"""


def print_banner(stream=None) -> None:
    print(BANNER, file=stream or sys.stderr)


def mask_gpus_for_grpo(argv: List[str]) -> None:
    """``grpo --trainer-gpus 0,1`` restricts the trainer process before CUDA is initialised."""
    if "--trainer-gpus" in argv:
        i = argv.index("--trainer-gpus")
        if i + 1 < len(argv):
            os.environ["CUDA_VISIBLE_DEVICES"] = argv[i + 1]


def cli_main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print_banner()
        print("usage: surogate <command> [config.yaml] [options]\n\ncommands:\n  " + "\n  ".join(sorted(COMMAND_MAPPING)))
        return 0
    cmd = argv[0]
    if cmd not in COMMAND_MAPPING:
        print(f"unknown command '{cmd}' (known: {', '.join(sorted(COMMAND_MAPPING))})", file=sys.stderr)
        return 2
    if cmd in ("grpo", "grpo-train", "grpo-infer", "grpo-orch") and "--train" not in argv:  # the trainer alone; a supervised run masks per component
        mask_gpus_for_grpo(argv)
    if int(os.environ.get("RANK", "0")) == 0 and os.environ.get("SUROGATE_NO_BANNER") != "1":
        print_banner()
    mod = importlib.import_module(COMMAND_MAPPING[cmd])
    return int(mod.main(argv[1:], command=cmd) or 0)


if __name__ == "__main__":
    sys.exit(cli_main())

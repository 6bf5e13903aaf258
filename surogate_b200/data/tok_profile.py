"""Where data preparation spends its time: ``SUROGATE_TOK_PROFILE=1`` times a tokenizer's chat-template rendering, its BPE encodes
and ``encode_for_training`` as a whole (the remainder is prefix alignment and label building), and prints the breakdown to stderr
when the process ends (every process of a tokenisation pool prints its own).  ``profile().summary()`` returns the numbers and
``profile().reset()`` clears them.  Nothing is wrapped, and nothing costs anything, unless the variable is set.

Parity: csrc/src/tokenizer/tok_profile.h, tok_profile.cpp (the same switch and purpose; the phases are this tokenizer's own).
"""
from __future__ import annotations

import atexit
import os
import sys
import time
from typing import Any, Callable, Dict, Optional

PHASES = ("render", "encode", "encode_for_training")


class TokProfile:
    def __init__(self):
        self.reset()

    def reset(self) -> None:
        self.ms: Dict[str, float] = {p: 0.0 for p in PHASES}
        self.calls: Dict[str, int] = {p: 0 for p in PHASES}
        self.tokens = 0

    def wrap(self, phase: str, fn: Callable[..., Any]) -> Callable[..., Any]:
        def timed(*a, **kw):
            t0 = time.perf_counter()
            out = fn(*a, **kw)
            self.ms[phase] += (time.perf_counter() - t0) * 1e3
            self.calls[phase] += 1
            if phase == "encode_for_training":
                self.tokens += len(out[0])
            return out

        timed.__wrapped__ = fn  # type: ignore[attr-defined]
        return timed

    def summary(self) -> Dict[str, Any]:
        whole = self.ms["encode_for_training"]
        inner = self.ms["render"] + self.ms["encode"]
        return {"calls": dict(self.calls), "ms": dict(self.ms), "tokens": self.tokens,
                # renders and encodes outside encode_for_training (plain text rows) make the remainder meaningless: clamp at zero
                "align_and_label_ms": max(0.0, whole - inner) if whole else 0.0,
                "tokens_per_second": self.tokens / (whole / 1e3) if whole else 0.0}

    def report(self, file=None) -> None:
        if not any(self.calls.values()):
            return
        s = self.summary()
        f = file or sys.stderr
        print(f"[tok-profile] pid {os.getpid()}: encode_for_training breakdown (SUROGATE_TOK_PROFILE=1)", file=f)
        for p in PHASES:
            print(f"  {p:<22}{s['ms'][p]:>12.1f} ms{s['calls'][p]:>10} calls", file=f)
        print(f"  {'align + labels':<22}{s['align_and_label_ms']:>12.1f} ms", file=f)
        print(f"  {s['tokens']} training tokens, {s['tokens_per_second']:.0f} tokens/s", file=f)


_profile: Optional[TokProfile] = None


def enabled(environ=os.environ) -> bool:
    return environ.get("SUROGATE_TOK_PROFILE", "0") not in ("", "0")


def profile() -> TokProfile:
    global _profile
    if _profile is None:
        _profile = TokProfile()
        atexit.register(_profile.report)
    return _profile


def instrument(tokenizer) -> None:
    """Wrap the three methods on this tokenizer object (instance attributes, the class stays as it is)."""
    p = profile()
    tokenizer.apply_chat_template = p.wrap("render", tokenizer.apply_chat_template)
    tokenizer.encode = p.wrap("encode", tokenizer.encode)
    tokenizer.encode_for_training = p.wrap("encode_for_training", tokenizer.encode_for_training)

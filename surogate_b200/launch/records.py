"""Which lines of a text stream are metrics-feed records.

A launcher streams a remote run's standard output back; log lines and feed records arrive interleaved.  A feed record is one
JSON object per line that is a step (``"step"`` present, no ``"type"``), or typed ``config`` / ``gpu`` / ``moe``.

Parity: jackalope/src/records.ts (parseLine).
"""
from __future__ import annotations

import json
from typing import Any, Dict, Optional

FEED_TYPES = ("config", "gpu", "moe")


def parse_feed_line(line: str) -> Optional[Dict[str, Any]]:
    s = line.strip()
    if not s or s[0] != "{":
        return None
    try:
        obj = json.loads(s)
    except ValueError:
        return None
    if not isinstance(obj, dict):
        return None
    kind = obj.get("type")
    if kind is None:
        step = obj.get("step")
        return obj if isinstance(step, (int, float)) and not isinstance(step, bool) else None
    return obj if kind in FEED_TYPES else None

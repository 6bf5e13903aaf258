"""Where downloaded datasets and lakeFS objects are kept, and path normalisation.

Parity: surogate/utils/fs.py (get_cache_dir, to_abspath)."""
from __future__ import annotations

import os
from typing import List, Optional, Union


def get_cache_dir() -> str:
    """``SUROGATE_CACHE_DIR`` (``SUROGATE_CACHE`` is read too), else ``~/.cache/surogate_b200``."""
    return os.environ.get("SUROGATE_CACHE_DIR") or os.environ.get("SUROGATE_CACHE") or os.path.join(os.path.expanduser("~"), ".cache", "surogate_b200")


def to_abspath(path: Union[str, List[str], None], check_path_exist: bool = False) -> Union[str, List[str], None]:
    """``~`` expanded and made absolute; a list is converted element by element; None stays None."""
    if path is None:
        return None
    if isinstance(path, str):
        p = os.path.abspath(os.path.expanduser(path))
        if check_path_exist and not os.path.exists(p):
            raise FileNotFoundError(f"path: '{p}'")
        return p
    return [to_abspath(p, check_path_exist) for p in path]

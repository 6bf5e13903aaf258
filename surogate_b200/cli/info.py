"""``surogate info [model dir]``: system diagnostics (GPUs, driver, extension build) and, optionally, a model summary.

Parity: surogate/utils/system_info.py, core/hub/model_info.py.
"""
from __future__ import annotations

import argparse
import json


def main(argv, command: str = "info") -> int:
    p = argparse.ArgumentParser(prog="surogate info")
    p.add_argument("model", nargs="?")
    a = p.parse_args(argv)
    from ..utils.system_info import system_info

    out = {"system": system_info()}
    if a.model:
        from ..models.presets import is_preset, preset_config

        if is_preset(a.model):   # an architecture preset: its config and parameter count, no files involved
            from ..dsl.compiler import compile_model, model_from_hf_config

            cfg = preset_config(a.model)
            out["model"] = {"preset": a.model, "config": cfg, "parameters": compile_model(model_from_hf_config(cfg)).num_parameters()}
        else:
            from ..hub import download_model, model_info

            out["model"] = model_info(download_model(a.model))
    print(json.dumps(out, indent=1, default=str))
    return 0

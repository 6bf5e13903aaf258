"""Offline block-FP8 quantisation of a HuggingFace checkpoint (the "fp8 block" pre-quantised layout).

Every 2-D projection weight ``W`` becomes ``W`` in E4M3 plus ``W_scale_inv`` (fp32, one value per 128 x 128 tile, multiply to
de-quantise); embeddings, norms, routers and the LM head stay in their dtype; ``config.json`` gains the
``quantization_config`` that loaders look for.  ``python -m surogate_b200.utils.quantize_fp8 --src dir --dst dir``.

Parity: scripts/quantize_fp8.py; csrc/src/kernels/block_quant.cu.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
from typing import Dict

import torch
from safetensors import safe_open
from safetensors.torch import save_file

SKIP = ("embed_tokens", "lm_head", "norm", ".gate.weight", "router")


def quantize_2d(w: torch.Tensor, block: int = 128):
    N, K = w.shape
    pn, pk = (-N) % block, (-K) % block
    wp = torch.nn.functional.pad(w.float(), (0, pk, 0, pn))
    tiles = wp.reshape((N + pn) // block, block, (K + pk) // block, block)
    scale_inv = tiles.abs().amax(dim=(1, 3)).clamp_min(1e-12) / 448.0
    q = (tiles / scale_inv[:, None, :, None]).reshape(N + pn, K + pk)[:N, :K].to(torch.float8_e4m3fn)
    return q.contiguous(), scale_inv.contiguous()


def quantize_checkpoint(src: str, dst: str, block: int = 128) -> Dict:
    os.makedirs(dst, exist_ok=True)
    n_q = n_keep = 0
    for fn in sorted(os.listdir(src)):
        p = os.path.join(src, fn)
        if fn.endswith(".safetensors"):
            out = {}
            with safe_open(p, framework="pt") as f:
                for k in f.keys():
                    t = f.get_tensor(k)
                    if t.dim() == 2 and k.endswith(".weight") and not any(s in k for s in SKIP) and t.dtype in (torch.bfloat16, torch.float16, torch.float32):
                        q, s = quantize_2d(t, block)
                        out[k] = q
                        out[k + "_scale_inv"] = s
                        n_q += 1
                    else:
                        out[k] = t
                        n_keep += 1
            save_file(out, os.path.join(dst, fn), metadata={"format": "pt"})
        elif fn == "config.json":
            with open(p) as f:
                cfg = json.load(f)
            cfg["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "activation_scheme": "dynamic", "weight_block_size": [block, block]}
            with open(os.path.join(dst, fn), "w") as f:
                json.dump(cfg, f, indent=1)
        elif os.path.isfile(p):
            shutil.copy2(p, os.path.join(dst, fn))
    return {"quantized": n_q, "kept": n_keep}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m surogate_b200.utils.quantize_fp8")
    p.add_argument("--src", required=True)
    p.add_argument("--dst", required=True)
    p.add_argument("--block", type=int, default=128)
    a = p.parse_args(argv)
    print(json.dumps(quantize_checkpoint(a.src, a.dst, a.block)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

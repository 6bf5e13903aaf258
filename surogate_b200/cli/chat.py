"""``surogate chat <model dir> [--adapter dir]``: a minimal interactive / one-shot generation loop for checking a trained model.

Decoding re-runs the full prefix every token (no KV cache): fine for a smoke test of a checkpoint, not a serving path.

Parity: scripts/chat.py.
"""
from __future__ import annotations

import argparse
import sys
from typing import List, Optional

import numpy as np


def generate(trainer, tokenizer, prompt_ids: List[int], max_new_tokens: int = 64, temperature: float = 0.0, seed: int = 0, eos_id: Optional[int] = None) -> List[int]:
    import torch

    ids = list(prompt_ids)
    gen = torch.Generator().manual_seed(seed)
    eos = tokenizer.eos_token_id if eos_id is None and tokenizer is not None else eos_id
    for _ in range(max_new_tokens):
        logits = trainer.logits(np.asarray([ids], np.int32))[0, -1].float().cpu()
        if temperature > 0:
            nxt = int(torch.multinomial(torch.softmax(logits / temperature, -1), 1, generator=gen))
        else:
            nxt = int(logits.argmax())
        ids.append(nxt)
        if eos is not None and nxt == eos:
            break
    return ids[len(prompt_ids):]


def main(argv, command: str = "chat") -> int:
    p = argparse.ArgumentParser(prog="surogate chat")
    p.add_argument("model")
    p.add_argument("--adapter", default=None)
    p.add_argument("--prompt", default=None, help="answer this prompt and exit (otherwise read prompts from stdin)")
    p.add_argument("--max-new-tokens", type=int, default=128)
    p.add_argument("--temperature", type=float, default=0.0)
    a = p.parse_args(argv)
    import torch

    from ..data.tokenizer import Tokenizer
    from ..dsl.compiler import load_hf_config
    from ..runtime.trainer import Trainer, TrainerConfig

    tok = Tokenizer.from_pretrained(a.model)
    cfg = load_hf_config(a.model)
    lora = None
    if a.adapter:
        import json
        import os

        with open(os.path.join(a.adapter, "adapter_config.json")) as f:
            ac = json.load(f)
        lora = dict(rank=ac["r"], alpha=ac["lora_alpha"], dropout=0.0, dtype="fp32", targets=ac["target_modules"], rslora=ac.get("use_rslora", False), train_router=False)
    tr = Trainer(TrainerConfig(model=cfg, batch_size=1, seq_len=128, zero_level=0, lora=lora), device=torch.device("cuda" if torch.cuda.is_available() else "cpu"))
    tr.import_weights(a.model)
    if a.adapter:
        tr.lora.load_peft(a.adapter)

    def answer(text: str) -> str:
        ids = tok.apply_chat_template_and_encode([{"role": "user", "content": text}], add_generation_prompt=True)
        return tok.decode(generate(tr, tok, ids, a.max_new_tokens, a.temperature), skip_special_tokens=True)

    if a.prompt is not None:
        print(answer(a.prompt))
        return 0
    for line in sys.stdin:
        if line.strip():
            print(answer(line.strip()), flush=True)
    return 0

"""Tokenizer front end: native byte-level BPE (``csrc/host/bpe_tokenizer.cpp``) + Jinja chat templates + training masks.

``Tokenizer.from_pretrained(dir)`` reads ``tokenizer.json`` (vocabulary, merges, added tokens, pre-tokeniser flavour),
``tokenizer_config.json`` (chat template, bos/eos/pad) and renders conversations with the model's own template.
``encode_for_training`` returns ``(input_ids, labels)`` where only assistant turns carry labels: the span of turn *i* is
found by rendering the conversation up to the turn with a generation prompt (where the assistant starts) and up to
and including it (where it ends), so the mask follows whatever markers the template emits.

Parity: csrc/src/tokenizer/tokenizer.h:39-122 (encode / decode / apply_chat_template / encode_for_training).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

IGNORE = -100
CHATML_TEMPLATE = (
    "{% for message in messages %}{{'<|im_start|>' + message['role'] + '\n' + message['content'] + '<|im_end|>' + '\n'}}{% endfor %}"
    "{% if add_generation_prompt %}{{ '<|im_start|>assistant\n' }}{% endif %}")


def _token_content(v) -> Optional[str]:
    if v is None:
        return None
    return v.get("content") if isinstance(v, dict) else str(v)


class Tokenizer:
    def __init__(self, core, config: Optional[Dict[str, Any]] = None, chat_template: Optional[str] = None):
        self.core = core
        self.config = config or {}
        self.chat_template = chat_template or self.config.get("chat_template")
        if isinstance(self.chat_template, list):  # named templates: take "default"
            named = {t.get("name"): t.get("template") for t in self.chat_template}
            self.chat_template = named.get("default") or next(iter(named.values()))
        self.bos_token = _token_content(self.config.get("bos_token"))
        self.eos_token = _token_content(self.config.get("eos_token"))
        self.pad_token = _token_content(self.config.get("pad_token"))
        self.add_bos = bool(self.config.get("add_bos_token", False))
        self._jinja = None
        if os.environ.get("SUROGATE_TOK_PROFILE"):
            from . import tok_profile

            if tok_profile.enabled():
                tok_profile.instrument(self)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_pretrained(cls, model_dir: str) -> "Tokenizer":
        from ..ops import host

        tj = os.path.join(model_dir, "tokenizer.json")
        if not os.path.exists(tj):
            raise FileNotFoundError(f"{model_dir} has no tokenizer.json")
        core = host().BpeTokenizer.from_file(tj)
        cfg: Dict[str, Any] = {}
        tc = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(tc):
            with open(tc) as f:
                cfg = json.load(f)
        template = None
        for name in ("chat_template.jinja", "chat_template.json"):
            p = os.path.join(model_dir, name)
            if os.path.exists(p):
                with open(p) as f:
                    raw = f.read()
                template = json.loads(raw).get("chat_template") if name.endswith(".json") else raw
                break
        return cls(core, cfg, template)

    @classmethod
    def from_json(cls, tokenizer_json: str, config: Optional[Dict[str, Any]] = None) -> "Tokenizer":
        from ..ops import host

        return cls(host().BpeTokenizer.from_json(tokenizer_json), config)

    # ------------------------------------------------------------------ ids
    def _id(self, tok: Optional[str]) -> int:
        return -1 if tok is None else self.core.token_to_id(tok.encode())

    @property
    def bos_token_id(self) -> int:
        return self._id(self.bos_token)

    @property
    def eos_token_id(self) -> int:
        return self._id(self.eos_token)

    @property
    def pad_token_id(self) -> int:
        p = self._id(self.pad_token)
        return p if p >= 0 else self.eos_token_id

    @property
    def vocab_size(self) -> int:
        return self.core.vocab_size()

    def is_special_token(self, tid: int) -> bool:
        return self.core.is_special(tid)

    # ------------------------------------------------------------------ encode / decode
    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = self.core.encode(text, True)
        if add_special_tokens and self.add_bos and self.bos_token_id >= 0:
            ids = [self.bos_token_id] + ids
        return ids

    def encode_ordinary(self, text: str) -> List[int]:
        """No added-token matching: marker strings in the text are tokenised as plain text."""
        return self.core.encode(text, False)

    def encode_batch(self, texts: Sequence[str], add_special_tokens: bool = False, threads: int = 0) -> List[List[int]]:
        out = self.core.encode_batch(list(texts), True, threads)
        if add_special_tokens and self.add_bos and self.bos_token_id >= 0:
            out = [[self.bos_token_id] + o for o in out]
        return out

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = False) -> str:
        return self.core.decode([int(i) for i in ids], skip_special_tokens).decode("utf-8", errors="replace")

    # ------------------------------------------------------------------ chat
    def _template(self):
        if self._jinja is None:
            import jinja2
            from jinja2.sandbox import ImmutableSandboxedEnvironment

            def raise_exception(msg):
                raise jinja2.exceptions.TemplateError(msg)

            env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])
            env.globals["raise_exception"] = raise_exception
            env.filters["tojson"] = lambda x, **kw: json.dumps(x, ensure_ascii=False, **{k: v for k, v in kw.items() if k == "indent"})
            self._jinja = env.from_string(self.chat_template or CHATML_TEMPLATE)
        return self._jinja

    def apply_chat_template(self, messages: Sequence[Dict[str, Any]], add_generation_prompt: bool = False, enable_thinking: Optional[bool] = None,
                            tools: Optional[List[Dict[str, Any]]] = None) -> str:
        kw: Dict[str, Any] = dict(messages=list(messages), add_generation_prompt=add_generation_prompt, bos_token=self.bos_token or "",
                                  eos_token=self.eos_token or "", pad_token=self.pad_token or "", tools=tools)
        if enable_thinking is not None:
            kw["enable_thinking"] = enable_thinking
        return self._template().render(**kw)

    def apply_chat_template_and_encode(self, messages, add_generation_prompt: bool = False) -> List[int]:
        return self.encode(self.apply_chat_template(messages, add_generation_prompt))

    def encode_for_training(self, messages: Sequence[Dict[str, Any]], train_on: str = "assistant", enable_thinking: Optional[bool] = None,
                            tools=None) -> Tuple[List[int], List[int]]:
        """(input_ids, labels): labels are -100 outside the trained turns. ``train_on``: assistant | last | all."""
        messages = list(messages)
        full = self.apply_chat_template(messages, False, enable_thinking, tools)
        ids = self.encode(full)
        if train_on == "all" and not any(m.get("loss") is not None for m in messages):
            return ids, list(ids)
        if train_on == "all":  # every token except the turns whose ``loss`` field switches them off
            labels = list(ids)
            for i, m in enumerate(messages):
                if m.get("role") == "assistant" and m.get("loss") is not None and not float(m["loss"]):
                    prefix = self.apply_chat_template(messages[:i], True, enable_thinking, tools)
                    upto = os.path.commonprefix([self.apply_chat_template(messages[:i + 1], False, enable_thinking, tools), full])
                    prefix = os.path.commonprefix([prefix, upto])
                    for k in range(len(self.encode(prefix)), min(len(self.encode(upto)), len(ids))):
                        labels[k] = IGNORE
            return ids, labels
        labels = [IGNORE] * len(ids)
        turns = [i for i, m in enumerate(messages) if m.get("role") == "assistant"]
        if train_on == "last":  # the assistant turns after the last user message (the last round)
            users = [i for i, m in enumerate(messages) if m.get("role") == "user"]
            turns = [i for i in turns if not users or i > users[-1]] or turns[-1:]
        # a message's own ``loss`` field overrides the mode: 0 / false leaves the turn out, anything else trains it
        forced = {i: bool(float(m["loss"])) for i, m in enumerate(messages) if m.get("role") == "assistant" and m.get("loss") is not None}
        turns = sorted((set(turns) | {i for i, on in forced.items() if on}) - {i for i, on in forced.items() if not on})
        for i in turns:
            prefix = self.apply_chat_template(messages[:i], True, enable_thinking, tools)
            upto = self.apply_chat_template(messages[:i + 1], False, enable_thinking, tools)
            if not full.startswith(upto):  # the template rewrites earlier turns (e.g. strips old reasoning): align on the common prefix
                upto = os.path.commonprefix([upto, full])
            if not upto.startswith(prefix):
                prefix = os.path.commonprefix([prefix, upto])
            a, b = len(self.encode(prefix)), len(self.encode(upto))
            for k in range(a, min(b, len(ids))):
                labels[k] = ids[k]
        return ids, labels

    def encode_for_training_batch(self, batch: Sequence[Sequence[Dict[str, Any]]], **kw) -> List[Tuple[List[int], List[int]]]:
        return [self.encode_for_training(m, **kw) for m in batch]

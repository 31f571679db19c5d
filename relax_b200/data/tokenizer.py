"""Text <-> token ids for prompts and responses: a Hugging Face tokenizer when a directory with tokenizer files is
given (``--hf-checkpoint`` / ``--tokenizer-path``), else a byte-level fallback that needs no files (tests, synthetic
runs).  Prompts may be strings or chat message lists; chat prompts go through the tokenizer's chat template (the
``--apply-chat-template`` path of relax/utils/data/data.py), with an optional system prompt prepended.
"""
from __future__ import annotations

import os
from typing import Any, List, Optional, Sequence


class ByteCodec:
    """UTF-8 bytes shifted past the special ids; ids beyond the byte range decode to nothing."""

    def __init__(self, vocab_size: int, offset: int = 3):
        self.vocab_size, self.offset = vocab_size, offset
        self.eos_token_id: Optional[int] = None

    def encode(self, text: str) -> List[int]:
        span = max(1, self.vocab_size - self.offset)
        return [self.offset + (b % span) for b in text.encode("utf-8")]

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i - self.offset for i in ids if self.offset <= i < self.offset + 256).decode("utf-8", errors="replace")

    def render(self, messages: Sequence[dict], add_generation_prompt: bool = True, tools=None, **kw) -> str:
        import json as _json

        head = f"<|tools|>\n{_json.dumps(tools)}\n" if tools else ""
        out = head + "".join(f"<|{m['role']}|>\n{_text_of(m.get('content'))}\n" for m in messages)
        return out + ("<|assistant|>\n" if add_generation_prompt else "")


def _text_of(content: Any) -> str:
    if isinstance(content, list):       # multimodal parts: the text ones, in order
        return "".join(p.get("text", "") for p in content if isinstance(p, dict))
    return "" if content is None else str(content)


class HFCodec:
    def __init__(self, path: str):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(path, trust_remote_code=False)
        self.eos_token_id = self.tok.eos_token_id
        self.vocab_size = len(self.tok)

    def encode(self, text: str) -> List[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def decode(self, ids: Sequence[int]) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=True)

    def render(self, messages, add_generation_prompt: bool = True, **kw) -> str:
        return self.tok.apply_chat_template(list(messages), tokenize=False, add_generation_prompt=add_generation_prompt, **kw)


def has_tokenizer_files(path: Optional[str]) -> bool:
    return bool(path) and os.path.isdir(path) and any(
        os.path.exists(os.path.join(path, f)) for f in ("tokenizer.json", "tokenizer.model", "vocab.json", "tokenizer_config.json"))


def build_codec(path: Optional[str], vocab_size: int):
    return HFCodec(path) if has_tokenizer_files(path) else ByteCodec(vocab_size)


class PromptEncoder:
    """``prompt`` (string or message list) -> token ids, honouring ``--apply-chat-template``, its kwargs and
    ``--system-prompt``; over-long prompts are reported by returning None so the loader can drop them."""

    def __init__(self, codec, apply_chat_template: bool = False, template_kwargs: Optional[dict] = None,
                 system_prompt: Optional[str] = None, max_prompt_len: Optional[int] = None):
        self.codec, self.chat, self.kw = codec, apply_chat_template, dict(template_kwargs or {})
        self.system_prompt, self.max_len = system_prompt, max_prompt_len

    def text(self, prompt: Any, tools: Optional[list] = None) -> str:
        if isinstance(prompt, str) and not self.chat and not tools:
            return (self.system_prompt + "\n" if self.system_prompt else "") + prompt
        msgs = [{"role": "user", "content": prompt}] if isinstance(prompt, str) else [dict(m) for m in prompt]
        if self.system_prompt and not (msgs and msgs[0].get("role") == "system"):
            msgs.insert(0, {"role": "system", "content": self.system_prompt})
        kw = dict(self.kw, tools=tools) if tools else self.kw      # tool definitions go through the chat template
        return self.codec.render(msgs, add_generation_prompt=True, **kw)

    def __call__(self, prompt: Any, tools: Optional[list] = None) -> Optional[List[int]]:
        ids = self.codec.encode(self.text(prompt, tools))
        return None if self.max_len and len(ids) > self.max_len else ids


def cut_at_stop_strings(codec, ids: Sequence[int], stops: Sequence[str]) -> Optional[int]:
    """Smallest token count whose decoded text contains one of ``stops`` (None when none occurs): containment is
    monotone in the prefix length, so a bisection over prefixes needs only O(log n) decodes."""
    stops = [s for s in (stops or []) if s]
    if not stops or not ids:
        return None
    has = lambda n: any(s in codec.decode(ids[:n]) for s in stops)
    if not has(len(ids)):
        return None
    lo, hi = 0, len(ids)          # has(lo) is False, has(hi) is True
    while hi - lo > 1:
        mid = (lo + hi) // 2
        lo, hi = (lo, mid) if has(mid) else (mid, hi)
    return hi

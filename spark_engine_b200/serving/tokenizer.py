"""Tokenizer access for the front end: a Hugging Face tokenizer + chat template when a tokenizer directory is
given, otherwise a byte-level fallback (ids 0..255 = bytes, 256 = BOS, 257 = EOS) so the whole serving path can run
without any checkpoint.  Incremental detokenisation holds back incomplete UTF-8 sequences."""
from __future__ import annotations

from typing import List, Optional


IMAGE_PLACEHOLDER = "<|image|>"


class ByteTokenizer:
    bos_token_id, eos_token_id, image_token_id = 256, 257, 258
    vocab_size = 259

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: List[int]) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, add_generation_prompt=True, tools=None) -> List[int]:
        parts = []
        if tools:
            import json
            parts.append("<|tools|>" + json.dumps(tools) + "\n")
        for m in messages:
            c = m.get("content") or ""
            if isinstance(c, list):
                c = "".join(p.get("text", "") for p in c if isinstance(p, dict))
            parts.append(f"<|{m['role']}|>{c}\n")
        if add_generation_prompt:
            parts.append("<|assistant|>")
        ids = [self.bos_token_id]
        for k, piece in enumerate("".join(parts).split(IMAGE_PLACEHOLDER)):      # media placeholders become one id each
            if k:
                ids.append(self.image_token_id)
            ids += self.encode(piece)
        return ids


class HfTokenizer:
    def __init__(self, path: str):
        from transformers import AutoTokenizer
        self.tk = AutoTokenizer.from_pretrained(path)
        self.eos_token_id = self.tk.eos_token_id
        self.vocab_size = len(self.tk)
        # the placeholder a multimodal checkpoint reserves for media rows, when it has one
        self.image_token_id = None
        for name in ("<|image_pad|>", "<image>", "<|image|>", "<|IMAGE|>"):
            t = self.tk.convert_tokens_to_ids(name)
            if isinstance(t, int) and t >= 0 and t != self.tk.unk_token_id:
                self.image_token_id, self.image_token = t, name
                break

    def encode(self, text):
        return self.tk.encode(text, add_special_tokens=False)

    def decode(self, ids):
        return self.tk.decode(ids, skip_special_tokens=True)

    def apply_chat_template(self, messages, add_generation_prompt=True, tools=None):
        return self.tk.apply_chat_template(messages, add_generation_prompt=add_generation_prompt, tools=tools, tokenize=True)


def load_tokenizer(path: Optional[str]):
    return HfTokenizer(path) if path else ByteTokenizer()


class IncrementalDetok:
    """Feeds token ids, returns the newly completed text (never splits a multi-byte character)."""

    def __init__(self, tok):
        self.tok, self.ids, self.emitted = tok, [], 0

    def feed(self, ids: List[int]) -> str:
        self.ids += ids
        text = self.tok.decode(self.ids)
        if text.endswith("�"):          # incomplete UTF-8 sequence at the end: wait for more tokens
            return ""
        new = text[self.emitted:]
        self.emitted = len(text)
        return new

"""Chat tokenizer: GLM chat template, stop ids and a byte-level fallback.

Template (reference ``crates/ferrite-http/src/tokenizer.rs:26-56``): every non-assistant
turn renders as ``<|user|>\\n{content}</s>\\n`` (system turns are rendered as user turns),
assistant turns as ``<|assistant|>\\n{content}</s>\\n``, and the generation prompt is
``<|assistant|>\\n``.  Stop ids are 154820 plus the ids of ``<|user|>``, ``<|endoftext|>``
and ``<|observation|>`` when the tokenizer knows them (``tokenizer.rs:95-101``).  The byte
tokenizer (ids = UTF-8 bytes, 256 = end of text) lets the whole HTTP path run without a model.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence

GLM_EOS = 154820
STOP_NAMES = ("<|user|>", "<|endoftext|>", "<|observation|>")


def render_chat_template(messages: Sequence[Dict[str, str]], add_generation_prompt: bool = True) -> str:
    out = []
    for m in messages:
        role = "assistant" if m.get("role") == "assistant" else "user"
        out.append(f"<|{role}|>\n{m.get('content', '')}</s>\n")
    if add_generation_prompt:
        out.append("<|assistant|>\n")
    return "".join(out)


class ByteTokenizer:
    """ids 0..255 are bytes; 256 is the end-of-text id."""

    EOS = 256
    vocab_size = 257

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))

    def decode_bytes(self, ids: Iterable[int]) -> bytes:
        return bytes(i for i in ids if 0 <= i < 256)

    def decode(self, ids: Iterable[int]) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")

    def stop_ids(self) -> List[int]:
        return [self.EOS]


class HFTokenizer:
    """A ``tokenizers``/``transformers`` tokenizer loaded from a model directory."""

    def __init__(self, model_dir: str):
        from transformers import AutoTokenizer
        self.tok = AutoTokenizer.from_pretrained(model_dir, local_files_only=True)
        self.vocab_size = len(self.tok)

    def encode(self, text: str) -> List[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def decode_bytes(self, ids: Iterable[int]) -> bytes:
        return self.decode(ids).encode("utf-8")

    def decode(self, ids: Iterable[int]) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=False)

    def stop_ids(self) -> List[int]:
        ids = [GLM_EOS]
        for name in STOP_NAMES:
            i = self.tok.convert_tokens_to_ids(name)
            if isinstance(i, int) and i >= 0 and i != getattr(self.tok, "unk_token_id", None):
                ids.append(i)
        return ids


class ChatTokenizer:
    def __init__(self, inner=None):
        self.inner = inner or ByteTokenizer()

    @staticmethod
    def load(model_dir: Optional[str]) -> "ChatTokenizer":
        if model_dir:
            try:
                return ChatTokenizer(HFTokenizer(model_dir))
            except Exception:
                pass
        return ChatTokenizer(ByteTokenizer())

    def encode_chat(self, messages: Sequence[Dict[str, str]]) -> List[int]:
        return self.inner.encode(render_chat_template(messages))

    def decode(self, ids: Iterable[int]) -> str:
        return self.inner.decode(ids)

    def decode_bytes(self, ids: Iterable[int]) -> bytes:
        return self.inner.decode_bytes(ids)

    def stop_ids(self) -> List[int]:
        return self.inner.stop_ids()

    @property
    def vocab_size(self) -> int:
        return self.inner.vocab_size


def utf8_holdback(data: bytes) -> int:
    """Number of trailing bytes that form an incomplete UTF-8 character (0..3); a stream
    frame must hold them back until the rest arrives (reference ``sse.rs:1-141``)."""
    n = len(data)
    for back in range(1, min(4, n) + 1):
        b = data[n - back]
        if b & 0xC0 == 0x80:
            continue  # continuation byte: keep looking for the lead byte
        if b & 0x80 == 0:
            return 0
        need = 2 if b & 0xE0 == 0xC0 else 3 if b & 0xF0 == 0xE0 else 4 if b & 0xF8 == 0xF0 else 1
        return back if back < need else 0
    return 0

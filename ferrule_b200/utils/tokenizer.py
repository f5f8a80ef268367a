"""Tokenizer handle, UTF-8-safe incremental detokenisation and chat templates.

`load_tokenizer(dir)` uses the HuggingFace `tokenizers` file (`tokenizer.json`) when present and
falls back to a byte-level tokenizer (ids 0..255 = bytes, 256 = BOS, 257 = EOS), which is what the
synthetic benchmarks and tests use.  `IncrementalDecodeState.push(token)` returns only text that
can no longer change: a multi-byte character split across tokens is held back until complete.

Counterpart of crates/ferrule-model/src/tokenizer.rs:8-60 and chat.rs:75-130 (ChatML, Llama3,
Qwen, DeepSeek, Plain templates).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from pathlib import Path
from typing import List, Sequence


class ByteTokenizer:
    """ids 0..255 are raw bytes; BOS = 256, EOS = 257."""
    bos_token_id, eos_token_id, vocab_size = 256, 257, 258

    def encode(self, text: str, add_bos: bool = False) -> List[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_bos else ids

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        return bytes(i for i in ids if 0 <= i < 256)


class HfTokenizer:
    def __init__(self, path):
        from tokenizers import Tokenizer as _T
        self._t = _T.from_file(str(path))
        self.vocab_size = self._t.get_vocab_size()
        self.bos_token_id = self._id_of(["<｜begin▁of▁sentence｜>", "<|begin_of_text|>", "<s>", "<|im_start|>"])
        self.eos_token_id = self._id_of(["<｜end▁of▁sentence｜>", "<|end_of_text|>", "</s>", "<|im_end|>", "<|endoftext|>"])

    def _id_of(self, names) -> int:
        for n in names:
            i = self._t.token_to_id(n)
            if i is not None:
                return i
        return -1

    def encode(self, text: str, add_bos: bool = False) -> List[int]:
        ids = self._t.encode(text, add_special_tokens=False).ids
        return ([self.bos_token_id] + ids) if (add_bos and self.bos_token_id >= 0) else ids

    def decode(self, ids: Sequence[int]) -> str:
        return self._t.decode(list(ids), skip_special_tokens=True)


def load_tokenizer(directory=None):
    if directory is not None:
        p = Path(directory) / "tokenizer.json"
        if p.exists():
            return HfTokenizer(p)
    return ByteTokenizer()


class IncrementalDecodeState:
    """Streams text deltas that are stable: never emits half of a multi-byte character, and costs a few token
    decodes per pushed token whatever the length of the output.

    Two offsets into the token list (the scheme of the common serving stacks): tokens before `prefix` are final
    text, tokens in [prefix, read) are the context that the next tokens may still merge with (byte-level BPE
    pieces, leading-space handling).  A push decodes [prefix, read) and [prefix, end): the new text is what the
    second has beyond the first - unless it ends inside a multi-byte character (replacement char), then nothing is
    emitted yet and the window grows."""

    def __init__(self, tokenizer=None, decode=None):
        self._decode = decode if decode is not None else tokenizer.decode
        self.ids: List[int] = []
        self.emitted = ""
        self.prefix = 0
        self.read = 0

    def push(self, token: int) -> str:
        self.ids.append(token)
        before = self._decode(self.ids[self.prefix:self.read]) if self.read > self.prefix else ""
        after = self._decode(self.ids[self.prefix:])
        if after.endswith("\ufffd") or not after.startswith(before):
            # inside a multi-byte character, or the new token changed how its predecessors read: wait for more
            if len(self.ids) - self.prefix > 64:
                # never settles (a tokenizer that rewrites earlier text): emit what there is and move on
                delta = after[len(before):] if after.startswith(before) else ""
                self._advance()
                self.emitted += delta
                return delta
            return ""
        delta = after[len(before):]
        self._advance()
        self.emitted += delta
        return delta

    def _advance(self) -> None:
        self.prefix, self.read = self.read, len(self.ids)
        # a context window that reads as nothing (special tokens, which the decoder skips) gives the next token no
        # left neighbour: a word-boundary decoder would take it for the first token of the text and drop its
        # leading space.  Reach back to a token that reads as something.
        steps = 0
        while 0 < self.prefix < self.read and steps < 8 and not self._decode(self.ids[self.prefix:self.read]):
            self.prefix -= 1
            steps += 1

    def finish(self) -> str:
        """Text still held back when the stream ends (an incomplete character is dropped)."""
        if self.read >= len(self.ids):
            return ""
        before = self._decode(self.ids[self.prefix:self.read]) if self.read > self.prefix else ""
        after = self._decode(self.ids[self.prefix:]).rstrip("\ufffd")
        delta = after[len(before):] if after.startswith(before) else ""
        self.prefix = self.read = len(self.ids)
        self.emitted += delta
        return delta


class ChatTemplate(Enum):
    CHATML = "chatml"
    LLAMA3 = "llama3"
    QWEN = "qwen"
    DEEPSEEK = "deepseek"
    PLAIN = "plain"


@dataclass
class ChatMessage:
    role: str
    content: str


def render_chat(messages: Sequence[ChatMessage], template: ChatTemplate = ChatTemplate.DEEPSEEK,
                add_generation_prompt: bool = True) -> str:
    if template in (ChatTemplate.CHATML, ChatTemplate.QWEN):
        out = ""
        if template == ChatTemplate.QWEN and not any(m.role == "system" for m in messages):
            out += "<|im_start|>system\nYou are a helpful assistant.<|im_end|>\n"
        for m in messages:
            out += f"<|im_start|>{m.role}\n{m.content}<|im_end|>\n"
        return out + ("<|im_start|>assistant\n" if add_generation_prompt else "")
    if template == ChatTemplate.LLAMA3:
        out = "<|begin_of_text|>"
        for m in messages:
            out += f"<|start_header_id|>{m.role}<|end_header_id|>\n\n{m.content}<|eot_id|>"
        return out + ("<|start_header_id|>assistant<|end_header_id|>\n\n" if add_generation_prompt else "")
    if template == ChatTemplate.DEEPSEEK:
        out = "<｜begin▁of▁sentence｜>"
        for m in messages:
            if m.role == "system":
                out += m.content
            elif m.role == "user":
                out += f"<｜User｜>{m.content}"
            else:
                out += f"<｜Assistant｜>{m.content}<｜end▁of▁sentence｜>"
        return out + ("<｜Assistant｜>" if add_generation_prompt else "")
    out = ""
    for m in messages:
        out += f"{m.role}: {m.content}\n"
    return out + ("assistant: " if add_generation_prompt else "")


def template_for_model(name: str) -> ChatTemplate:
    n = name.lower()
    if "deepseek" in n:
        return ChatTemplate.DEEPSEEK
    if "qwen" in n:
        return ChatTemplate.QWEN
    if "llama" in n:
        return ChatTemplate.LLAMA3
    return ChatTemplate.CHATML

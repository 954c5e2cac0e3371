"""Byte-level BPE tokenizer in the Qwen layout, with the ChatML template.

Reference behaviour covered (include/oil/qwen35_tokenizer.h:10-58, ``Qwen35Tokenizer``; include/oil/bpe_tokenizer.h
``ByteLevelBPE``): loads ``vocab.json`` + ``merges.txt`` (or a ``tokenizer.json`` holding both) from a model directory,
maps bytes to printable code points the GPT-2 way, splits text with the Qwen pre-tokenisation pattern (contractions,
letter runs, single digits, punctuation runs, whitespace), merges by rank, keeps special tokens (``<|im_start|>``,
``<|im_end|>``, ``<|endoftext|>`` ...) atomic, has no BOS token, ends turns with ``<|im_end|>``, and renders a message
list as ``<|im_start|>role\\ncontent<|im_end|>\\n`` with an optional ``<think>`` block for reasoning content.
``train`` builds a small vocabulary of the same kind from text (tests, toy models).
"""
from __future__ import annotations

import json
import os
from collections import Counter
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import regex

_PATTERN = regex.compile(r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")
DEFAULT_SPECIALS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>"]


def byte_map() -> Dict[int, str]:
    """Printable bytes map to themselves, the rest to code points from 256 upwards."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    out, n = {}, 0
    for b in range(256):
        if b in keep:
            out[b] = chr(b)
        else:
            out[b] = chr(256 + n)
            n += 1
    return out


@dataclass
class QwenMessage:
    role: str
    content: str
    reasoning_content: str = ""


class QwenTokenizer:
    def __init__(self, vocab: Dict[str, int], merges: Sequence[Tuple[str, str]], specials: Optional[Dict[str, int]] = None):
        self.token_to_id = dict(vocab)
        self.ranks = {tuple(m): i for i, m in enumerate(merges)}
        self.specials = dict(specials or {})
        self.id_to_token = {i: t for t, i in self.token_to_id.items()}
        self.id_to_token.update({i: t for t, i in self.specials.items()})
        self._b2u = byte_map()
        self._u2b = {u: b for b, u in self._b2u.items()}
        self._cache: Dict[str, List[int]] = {}
        self._special_re = regex.compile("(" + "|".join(regex.escape(s) for s in sorted(self.specials, key=len, reverse=True)) + ")") \
            if self.specials else None

    # -- loading -----------------------------------------------------------------------------------------------------
    @classmethod
    def load_from_dir(cls, model_dir: str) -> "QwenTokenizer":
        tj = os.path.join(model_dir, "tokenizer.json")
        specials: Dict[str, int] = {}
        if os.path.exists(os.path.join(model_dir, "vocab.json")):
            with open(os.path.join(model_dir, "vocab.json"), encoding="utf-8") as f:
                vocab = json.load(f)
            merges = []
            with open(os.path.join(model_dir, "merges.txt"), encoding="utf-8") as f:
                for line in f:
                    line = line.rstrip("\n")
                    if line and not line.startswith("#version"):
                        a, b = line.split(" ")
                        merges.append((a, b))
        elif os.path.exists(tj):
            with open(tj, encoding="utf-8") as f:
                j = json.load(f)
            vocab = j["model"]["vocab"]
            merges = [tuple(m.split(" ")) if isinstance(m, str) else tuple(m) for m in j["model"]["merges"]]
            specials = {t["content"]: t["id"] for t in j.get("added_tokens", [])}
        else:
            raise FileNotFoundError(f"{model_dir}: neither vocab.json + merges.txt nor tokenizer.json")
        cfg = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(cfg):
            with open(cfg, encoding="utf-8") as f:
                for i, t in json.load(f).get("added_tokens_decoder", {}).items():
                    specials[t["content"]] = int(i)
        if not specials:
            nxt = max(vocab.values()) + 1
            specials = {s: nxt + k for k, s in enumerate(DEFAULT_SPECIALS)}
        return cls(vocab, merges, specials)

    def save_to_dir(self, model_dir: str):
        os.makedirs(model_dir, exist_ok=True)
        with open(os.path.join(model_dir, "vocab.json"), "w", encoding="utf-8") as f:
            json.dump(self.token_to_id, f, ensure_ascii=False)
        with open(os.path.join(model_dir, "merges.txt"), "w", encoding="utf-8") as f:
            f.write("#version: 0.2\n")
            for (a, b), _ in sorted(self.ranks.items(), key=lambda kv: kv[1]):
                f.write(f"{a} {b}\n")
        with open(os.path.join(model_dir, "tokenizer_config.json"), "w", encoding="utf-8") as f:
            json.dump({"added_tokens_decoder": {str(i): {"content": s} for s, i in self.specials.items()}}, f)

    @classmethod
    def train(cls, texts: Sequence[str], vocab_size: int = 512, specials: Sequence[str] = DEFAULT_SPECIALS) -> "QwenTokenizer":
        b2u = byte_map()
        vocab = {b2u[b]: b for b in range(256)}
        words = Counter()
        for t in texts:
            for w in _PATTERN.findall(t):
                words[tuple(b2u[b] for b in w.encode("utf-8"))] += 1
        merges: List[Tuple[str, str]] = []
        while len(vocab) < vocab_size:
            pairs = Counter()
            for w, c in words.items():
                for a, b in zip(w, w[1:]):
                    pairs[(a, b)] += c
            if not pairs:
                break
            (a, b), cnt = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
            if cnt < 2:
                break
            merges.append((a, b))
            vocab[a + b] = len(vocab)
            new = Counter()
            for w, c in words.items():
                out, i = [], 0
                while i < len(w):
                    if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                        out.append(a + b)
                        i += 2
                    else:
                        out.append(w[i])
                        i += 1
                new[tuple(out)] += c
            words = new
        return cls(vocab, merges, {s: len(vocab) + k for k, s in enumerate(specials)})

    # -- encode / decode ---------------------------------------------------------------------------------------------
    @property
    def vocab_size(self) -> int:
        return max(self.id_to_token) + 1

    def bos_id(self) -> int:
        return -1                                   # the layout has no BOS token

    def im_start_id(self) -> int:
        return self.specials["<|im_start|>"]

    def im_end_id(self) -> int:
        return self.specials["<|im_end|>"]

    def eos_id(self) -> int:
        return self.im_end_id()

    def is_special(self, i: int) -> bool:
        return i in self.specials.values()

    def _bpe(self, word: str) -> List[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        parts = [self._b2u[b] for b in word.encode("utf-8")]
        while len(parts) > 1:
            best, at = None, -1
            for i, pr in enumerate(zip(parts, parts[1:])):
                r = self.ranks.get(pr)
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            parts[at:at + 2] = [parts[at] + parts[at + 1]]
        ids = [self.token_to_id[p] for p in parts]
        if len(self._cache) < 100000:
            self._cache[word] = ids
        return ids

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        chunks = self._special_re.split(text) if self._special_re is not None else [text]
        for ch in chunks:
            if not ch:
                continue
            if ch in self.specials:
                out.append(self.specials[ch])
            else:
                for w in _PATTERN.findall(ch):
                    out.extend(self._bpe(w))
        return out

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        buf, out = bytearray(), []
        for i in ids:
            i = int(i)
            tok = self.id_to_token.get(i)
            if tok is None:
                continue
            if self.is_special(i):
                if buf:
                    out.append(buf.decode("utf-8", "replace"))
                    buf = bytearray()
                if not skip_special:
                    out.append(tok)
            else:
                buf.extend(self._u2b[c] for c in tok)
        if buf:
            out.append(buf.decode("utf-8", "replace"))
        return "".join(out)

    # -- chat template -----------------------------------------------------------------------------------------------
    def render_chat(self, messages: Sequence[QwenMessage], add_generation_prompt: bool = True) -> str:
        s = ""
        for m in messages:
            body = m.content
            if m.role == "assistant" and m.reasoning_content:
                body = f"<think>\n{m.reasoning_content}\n</think>\n\n{m.content}"
            s += f"<|im_start|>{m.role}\n{body}<|im_end|>\n"
        if add_generation_prompt:
            s += "<|im_start|>assistant\n"
        return s

    def apply_chat_template(self, messages: Sequence[QwenMessage], add_generation_prompt: bool = True) -> List[int]:
        return self.encode(self.render_chat(messages, add_generation_prompt))


Qwen35Tokenizer = QwenTokenizer
Qwen35Message = QwenMessage
ByteLevelBPE = QwenTokenizer

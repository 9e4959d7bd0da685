"""Tokenizers and chat template of the reference, host side: text <-> token ids either side of the decode step.

`LlamaTokenizer` follows crates/slai/src/models/llama2/tokenizer.rs:72-183 (space -> U+2581, one token per character with
byte fallback at id byte+3, the literal strings `<s>` / `</s>` folded into the special ids, then repeated merging of the
adjacent pair whose concatenation has the highest vocabulary score); `Gpt2Tokenizer` follows
crates/slai/src/models/gpt2/tokenizer.rs:105-217 (byte-level BPE over the pieces of a split pattern, merge ranks from the
`tokenizer.ggml.merges` list, `<...>` spans looked up as whole special tokens); `ChatTemplate` follows
crates/slai-chat/src/chat_template.rs:11-39 (the model's Jinja template with `bos_token`, `eos_token` and
`add_generation_prompt = true`).  Vocabularies come from GGUF metadata (`gguf_io.GgufFile(...).metadata`) or from plain lists.
"""
from __future__ import annotations

import re
import unicodedata

SPACE_MARK = "\u2581"


class LlamaTokenizer:
    def __init__(self, tokens: list[str], scores: list[float], bos: int = 1, eos: int = 2, unk: int = 0):
        if len(tokens) != len(scores):
            raise ValueError("tokens and scores differ in length")
        self.vocab = list(tokens)
        self.scores = [float(s) for s in scores]
        self.bos, self.eos, self.unk = int(bos), int(eos), int(unk)
        self.index = {}
        for i, t in enumerate(self.vocab):  # a later duplicate replaces an earlier one, as a hash-map insert does
            self.index[t] = i

    @classmethod
    def from_gguf(cls, metadata: dict) -> "LlamaTokenizer":
        """Metadata keys of tokenizer.rs:24-36."""
        return cls(list(metadata["tokenizer.ggml.tokens"]), list(metadata["tokenizer.ggml.scores"]),
                   int(metadata["tokenizer.ggml.bos_token_id"]), int(metadata["tokenizer.ggml.eos_token_id"]),
                   int(metadata["tokenizer.ggml.unknown_token_id"]))

    def bos_str(self) -> str:
        return self.vocab[self.bos]

    def eos_str(self) -> str:
        return self.vocab[self.eos]

    def _fold(self, ids: list[int], literal: str, special: int) -> None:
        """Runs of single-character tokens that spell `literal` become the one id `special` (tokenizer.rs:99-140; the scan
        stops len(literal)-1 tokens before the end and, like the reference, moves on by one token after a replacement)."""
        n = len(literal)
        i = 0
        while i < max(len(ids) - (n - 1), 0):
            if "".join(self.vocab[t] for t in ids[i:i + n]) == literal:
                ids[i:i + n] = [special]
            i += 1

    def encode(self, text: str, bos: bool = True, eos: bool = False) -> list[int]:
        text = text.replace(" ", SPACE_MARK)
        ids = [self.bos] if bos else []
        for ch in text:
            tid = self.index.get(ch)
            if tid is not None:
                ids.append(tid)
            else:
                ids.extend(b + 3 for b in ch.encode("utf-8"))  # byte fallback: ids 3..258 are the single bytes
        self._fold(ids, "<s>", self.bos)
        self._fold(ids, "</s>", self.eos)
        while len(ids) >= 2:
            best, best_at, best_id = float("-inf"), -1, -1
            for i in range(len(ids) - 1):
                tid = self.index.get(self.vocab[ids[i]] + self.vocab[ids[i + 1]])
                if tid is not None and self.scores[tid] > best:
                    best, best_at, best_id = self.scores[tid], i, tid
            if best_at < 0:
                break
            ids[best_at:best_at + 2] = [best_id]
        if eos:
            ids.append(self.eos)
        return ids

    def decode(self, prev_token: int, token: int) -> str:
        """One token to text (tokenizer.rs:167-177): no leading blank right after BOS (id 1), `<0xNN>` pieces are bytes."""
        piece = self.vocab[token]
        if prev_token == 1:
            piece = piece.lstrip()
        if piece.startswith("<0x") and len(piece) >= 5:
            try:
                return chr(int(piece[3:5], 16))
            except ValueError:
                pass
        return piece.replace(SPACE_MARK, " ")

    def decode_all(self, ids: list[int]) -> str:
        out, prev = [], -1
        for t in ids:
            out.append(self.decode(prev, t))
            prev = t
        return "".join(out)


def bytes_to_unicode() -> dict[int, str]:
    """The byte -> printable character table of byte-level BPE (tokenizer.rs:22-36): printable Latin-1 bytes map to
    themselves, the others to code points from 256 up in byte order."""
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table = {b: chr(b) for b in keep}
    n = 0
    for b in range(256):
        if b not in table:
            table[b] = chr(256 + n)
            n += 1
    return table


def _is_letter(ch: str) -> bool:
    return unicodedata.category(ch).startswith("L")


def _is_number(ch: str) -> bool:
    return unicodedata.category(ch).startswith("N")


def split_pieces(text: str) -> list[str]:
    """The reference's split pattern (tokenizer.rs:74-75) as a scanner, alternatives tried in its order:
    `'s|'t|'re|'ve|'m|'ll|'d| ?\\p{L}+| ?\\p{N}+| ?[^\\s\\p{L}\\p{N}]+|\\s+` (Python's `re` has no \\p classes)."""
    out, i, n = [], 0, len(text)
    while i < n:
        for suf in ("'s", "'t", "'re", "'ve", "'m", "'ll", "'d"):
            if text.startswith(suf, i):
                out.append(suf)
                i += len(suf)
                break
        else:
            j = i + 1 if text[i] == " " and i + 1 < n else i
            if j < n and _is_letter(text[j]):
                k = j
                while k < n and _is_letter(text[k]):
                    k += 1
            elif j < n and _is_number(text[j]):
                k = j
                while k < n and _is_number(text[k]):
                    k += 1
            elif j < n and not text[j].isspace() and not _is_letter(text[j]) and not _is_number(text[j]):
                k = j
                while k < n and not text[k].isspace() and not _is_letter(text[k]) and not _is_number(text[k]):
                    k += 1
            elif text[i].isspace():
                k = i
                while k < n and text[k].isspace():
                    k += 1
            else:  # not reachable: every character is a letter, a number, a blank or "other"
                k = i + 1
            out.append(text[i:k])
            i = k
    return out


class Gpt2Tokenizer:
    def __init__(self, tokens: list[str], merges: list[str], bos: int, eos: int):
        self.bos, self.eos = int(bos), int(eos)
        self.encoder = {}
        for i, t in enumerate(tokens):
            self.encoder[t] = i
        self.decoder = {i: t for i, t in enumerate(tokens)}
        self.ranks = {}
        for i, line in enumerate(merges):
            a, b = line.split()[:2]
            self.ranks[(a, b)] = i
        self.byte_encoder = bytes_to_unicode()
        self.byte_decoder = {c: b for b, c in self.byte_encoder.items()}

    @classmethod
    def from_gguf(cls, metadata: dict) -> "Gpt2Tokenizer":
        """Metadata keys of tokenizer.rs:56-60."""
        return cls(list(metadata["tokenizer.ggml.tokens"]), list(metadata["tokenizer.ggml.merges"]),
                   int(metadata["tokenizer.ggml.bos_token_id"]), int(metadata["tokenizer.ggml.eos_token_id"]))

    def bos_str(self) -> str:
        return self.decoder[self.bos]

    def eos_str(self) -> str:
        return self.decoder[self.eos]

    def bpe(self, token: str) -> list[str]:
        """Merge loop of tokenizer.rs:169-215: while some adjacent pair has a rank, merge every occurrence of the
        lowest-ranked one."""
        word = list(token)
        while len(word) > 1:
            pairs = {(word[i], word[i + 1]) for i in range(len(word) - 1)}
            first, second = min(pairs, key=lambda p: self.ranks.get(p, float("inf")))
            if (first, second) not in self.ranks:
                break
            merged, i = [], 0
            while i < len(word):
                if i + 1 < len(word) and word[i] == first and word[i + 1] == second:
                    merged.append(first + second)
                    i += 2
                else:
                    merged.append(word[i])
                    i += 1
            word = merged
        return word

    def _encode_plain(self, text: str, out: list[int]) -> None:
        for piece in split_pieces(text):
            mapped = "".join(self.byte_encoder[b] for b in piece.encode("utf-8"))
            for part in self.bpe(mapped):
                tid = self.encoder.get(part)
                if tid is not None:  # parts missing from the vocabulary are dropped, as in the reference
                    out.append(tid)

    def encode(self, text: str) -> list[int]:
        """`<...>` spans are special tokens looked up whole (tokenizer.rs:127-144; an unknown one is a KeyError where the
        reference panics), the text between them goes through the byte-level BPE."""
        out, cursor = [], 0
        for m in re.finditer(r"<[^<>]*>", text):
            if cursor != m.start():
                self._encode_plain(text[cursor:m.start()], out)
            out.append(self.encoder[m.group(0)])
            cursor = m.end()
        if cursor < len(text):
            self._encode_plain(text[cursor:], out)
        return out

    def decode(self, ids: list[int]) -> str:
        """tokenizer.rs:154-167: pieces joined, mapped back to bytes, each byte read as one character (Latin-1), like the
        reference's `b as char`; use `decode_bytes` for the raw bytes."""
        return self.decode_bytes(ids).decode("latin-1")

    def decode_bytes(self, ids: list[int]) -> bytes:
        text = "".join(self.decoder[t] for t in ids if t in self.decoder)
        return bytes(self.byte_decoder[c] for c in text if c in self.byte_decoder)


# A Llama-2 chat layout in this project's own words (used when the file carries no `tokenizer.chat_template`): system text
# inside <<SYS>> markers at the head of the first user turn, user turns in [INST] ... [/INST], assistant turns closed by EOS.
DEFAULT_CHAT_TEMPLATE = (
    "{% set ns = namespace(sys='') %}"
    "{% for m in messages %}"
    "{% if m['role'] == 'system' %}{% set ns.sys = '<<SYS>>\\n' + m['content'] + '\\n<</SYS>>\\n\\n' %}"
    "{% elif m['role'] == 'user' %}{{ bos_token }}[INST] {{ ns.sys }}{{ m['content'] }} [/INST]{% set ns.sys = '' %}"
    "{% elif m['role'] == 'assistant' %} {{ m['content'] }} {{ eos_token }}"
    "{% endif %}{% endfor %}"
)


class ChatTemplate:
    """crates/slai-chat/src/chat_template.rs:11-39.  Needs `jinja2` (the reference uses minijinja)."""

    def __init__(self, template: str):
        # the two rewrites the reference applies for its template engine; harmless for jinja2, kept so that both see one text
        self.template = template.replace(".split(", "|split(").replace("[-1]", "|last")

    @classmethod
    def from_gguf(cls, metadata: dict) -> "ChatTemplate":
        return cls(str(metadata.get("tokenizer.chat_template", DEFAULT_CHAT_TEMPLATE)))

    def apply(self, messages: list[dict], bos: str, eos: str) -> str:
        """`messages`: [{"role": "system" | "user" | "assistant", "content": str}, ...] (Prompt::to_jinja_input,
        crates/slai-chat/src/prompt.rs:80-105)."""
        import jinja2
        env = jinja2.Environment(trim_blocks=True)
        env.filters.setdefault("split", lambda s, sep=None: str(s).split(sep))
        env.globals.update(bos_token=bos, eos_token=eos, add_generation_prompt=True)
        return env.from_string(self.template).render(messages=messages)

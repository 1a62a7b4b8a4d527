"""Tokenizers: HuggingFace ``tokenizers`` files, GGUF-embedded SentencePiece-style vocabularies, and a
small built-in word vocabulary for tests and weight-less models.

API parity with ``crates/runtime/src/tokenizer.rs:38-306, 636-683``: ``encode``,
``encode_with_special_tokens(add_bos, add_eos)``, ``decode``, ``decode_raw``, ``vocab_size``,
``bos/eos/pad/unk_token_id``, ``contains_token``, ``token_to_id``, ``id_to_token``; constructors
``new`` (basic), ``from_file``, ``from_model_dir``, ``from_pretrained`` (local caches only -- there is
no network), ``from_gguf`` / ``from_model_weights``; ``BatchTokenizer.encode_batch / decode_batch``.
Constants as in ``tokenizer.rs:12-15``: UNK 0, BOS 1, EOS 2, PAD 3.

The GGUF encoder follows the reference algorithm (prepend U+2581, spaces -> U+2581, greedy longest
match of at most 32 bytes, ``<0xNN>`` byte fallback, UNK) but looks candidates up in a trie instead
of re-slicing and re-validating UTF-8 for every length, and it honours token scores when two
matches of equal length exist.
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Dict, List, Optional, Sequence, Tuple

from .types import FileSystemError, InvalidInput, LoadingError

UNK_TOKEN_ID = 0
BOS_TOKEN_ID = 1
EOS_TOKEN_ID = 2
PAD_TOKEN_ID = 3

_BASIC_WORDS = (
    "the a an and or but in on at to for of with by is are was were be been have has had do does did "
    "will would could should can may might must I you he she it we they me him her us them "
    "this that these those here there where when why how what who which whose all some any no not yes "
    "hello world test example text model language AI quick brown fox dog cat house car tree book water"
).split() + list(".!?,;:'\"-_()[]{}") + list("0123456789") + list("abcdefghijklmnopqrstuvwxyz") + \
    list("ABCDEFGHIJKLMNOPQRSTUVWXYZ") + ["ing", "ed", "er", "ly", "tion", "ment", "ness", "ity", "ous", "ful",
                                           " ", "\n", "\t"]


class _Backend:
    bos_token_id = BOS_TOKEN_ID
    eos_token_id = EOS_TOKEN_ID
    pad_token_id = PAD_TOKEN_ID
    unk_token_id = UNK_TOKEN_ID

    def encode_raw(self, text: str) -> List[int]: raise NotImplementedError
    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str: raise NotImplementedError
    def vocab_size(self) -> int: raise NotImplementedError
    def token_to_id(self, tok: str) -> Optional[int]: raise NotImplementedError
    def id_to_token(self, i: int) -> Optional[str]: raise NotImplementedError


class _BasicBackend(_Backend):
    """About 200 words, punctuation, digits and letters; unknown words fall back to characters."""

    def __init__(self):
        self.vocab: Dict[str, int] = {"<unk>": UNK_TOKEN_ID, "<s>": BOS_TOKEN_ID, "</s>": EOS_TOKEN_ID,
                                      "<pad>": PAD_TOKEN_ID}
        for w in _BASIC_WORDS:
            if w not in self.vocab:
                self.vocab[w] = len(self.vocab)
        self.inv = {i: t for t, i in self.vocab.items()}

    def encode_raw(self, text: str) -> List[int]:
        out: List[int] = []
        for piece in re.findall(r"\w+|\s|[^\w\s]", text):
            if piece in self.vocab:
                out.append(self.vocab[piece])
            else:
                out.extend(self.vocab.get(ch, UNK_TOKEN_ID) for ch in piece)
        return out

    def decode(self, ids, skip_special=True):
        res: List[str] = []
        last_char = False
        for i in ids:
            if skip_special and i in (BOS_TOKEN_ID, EOS_TOKEN_ID, PAD_TOKEN_ID):
                continue
            tok = self.inv.get(int(i))
            if tok is None:
                continue
            single = len(tok) == 1 and tok.isalpha()
            space = tok.isspace()
            punct = all((not c.isalnum()) and (not c.isspace()) for c in tok)
            if res and not space and not punct and not res[-1].isspace():
                if not (last_char and single):
                    res.append(" ")
            res.append(tok)
            last_char = single
        return "".join(res)

    def vocab_size(self): return len(self.vocab)
    def token_to_id(self, tok): return self.vocab.get(tok)
    def id_to_token(self, i): return self.inv.get(int(i))


class _GGUFBackend(_Backend):
    """SentencePiece-style vocabulary stored in GGUF metadata (``tokenizer.ggml.*``)."""

    SP = "▁"

    def __init__(self, tokens: Sequence[str], scores: Optional[Sequence[float]] = None, bos: int = 1, eos: int = 2,
                 unk: int = 0, pad: Optional[int] = None, max_token_bytes: int = 32):
        self.tokens = list(tokens)
        self.scores = list(scores) if scores is not None else [0.0] * len(self.tokens)
        self.bos_token_id, self.eos_token_id, self.unk_token_id = bos, eos, unk
        self.pad_token_id = pad if pad is not None else PAD_TOKEN_ID
        self.max_token_bytes = max_token_bytes
        self.t2i: Dict[str, int] = {}
        for i, t in enumerate(self.tokens):
            if t not in self.t2i or self.scores[i] > self.scores[self.t2i[t]]:
                self.t2i[t] = i
        # byte trie over the UTF-8 encodings of all tokens
        self._trie: Dict = {}
        for t, i in self.t2i.items():
            b = t.encode("utf-8")
            if 0 < len(b) <= max_token_bytes:
                node = self._trie
                for ch in b:
                    node = node.setdefault(ch, {})
                node[-1] = i
        self._byte_tok = {b: self.t2i.get(f"<0x{b:02X}>") for b in range(256)}

    def encode_raw(self, text: str) -> List[int]:
        data = (self.SP + text.replace(" ", self.SP)).encode("utf-8")
        out: List[int] = []
        i, n = 0, len(data)
        while i < n:
            node, best, best_len = self._trie, None, 0
            j = i
            while j < n and j - i < self.max_token_bytes:
                node = node.get(data[j])
                if node is None:
                    break
                j += 1
                if -1 in node:
                    best, best_len = node[-1], j - i
            if best is not None:
                out.append(best)
                i += best_len
                continue
            bt = self._byte_tok.get(data[i])
            out.append(bt if bt is not None else self.unk_token_id)
            i += 1
        return out

    def decode(self, ids, skip_special=True):
        buf = bytearray()
        for i in ids:
            i = int(i)
            if skip_special and i in (self.bos_token_id, self.eos_token_id, self.pad_token_id):
                continue
            if 0 <= i < len(self.tokens):
                t = self.tokens[i]
                m = re.fullmatch(r"<0x([0-9A-Fa-f]{2})>", t)
                if m:
                    buf.append(int(m.group(1), 16))
                else:
                    buf.extend(t.encode("utf-8"))
        s = buf.decode("utf-8", errors="replace").replace(self.SP, " ")
        return s.lstrip(" ")

    def vocab_size(self): return len(self.tokens)
    def token_to_id(self, tok): return self.t2i.get(tok)
    def id_to_token(self, i): return self.tokens[i] if 0 <= int(i) < len(self.tokens) else None


class _HFBackend(_Backend):
    """A ``tokenizer.json`` handled by the HuggingFace ``tokenizers`` library."""

    def __init__(self, path: str):
        try:
            from tokenizers import Tokenizer as HFTok
        except Exception as e:  # pragma: no cover
            raise LoadingError(f"the 'tokenizers' package is not importable: {e}")
        self.tk = HFTok.from_file(path)
        for name, attr, default in (("<s>", "bos_token_id", BOS_TOKEN_ID), ("</s>", "eos_token_id", EOS_TOKEN_ID),
                                    ("<unk>", "unk_token_id", UNK_TOKEN_ID), ("<pad>", "pad_token_id", PAD_TOKEN_ID)):
            i = self.tk.token_to_id(name)
            setattr(self, attr, i if i is not None else default)
        for name, attr in (("<|begin_of_text|>", "bos_token_id"), ("<|end_of_text|>", "eos_token_id"),
                           ("<|endoftext|>", "eos_token_id")):
            i = self.tk.token_to_id(name)
            if i is not None:
                setattr(self, attr, i)

    def encode_raw(self, text): return list(self.tk.encode(text, add_special_tokens=False).ids)
    def decode(self, ids, skip_special=True): return self.tk.decode([int(i) for i in ids], skip_special_tokens=skip_special)
    def vocab_size(self): return self.tk.get_vocab_size()
    def token_to_id(self, tok): return self.tk.token_to_id(tok)
    def id_to_token(self, i): return self.tk.id_to_token(int(i))


class Tokenizer:
    def __init__(self, backend: _Backend, kind: str):
        self._b = backend
        self.kind = kind

    # ---- constructors ----
    @staticmethod
    def new() -> "Tokenizer":
        return Tokenizer(_BasicBackend(), "basic")

    @staticmethod
    def from_file(path: str) -> "Tokenizer":
        if not os.path.isfile(path):
            raise FileSystemError(f"tokenizer file not found: {path}")
        return Tokenizer(_HFBackend(path), "huggingface")

    @staticmethod
    def from_model_dir(model_dir: str) -> "Tokenizer":
        p = os.path.join(model_dir, "tokenizer.json")
        if os.path.isfile(p):
            return Tokenizer.from_file(p)
        raise FileSystemError(f"no tokenizer.json in {model_dir}")

    @staticmethod
    def from_pretrained(model_name: str) -> "Tokenizer":
        """Looks in the local HuggingFace cache only (``~/.cache/huggingface/hub/models--org--name``)."""
        root = os.environ.get("HF_HOME", os.path.join(os.path.expanduser("~"), ".cache", "huggingface"))
        pat = os.path.join(root, "hub", "models--" + model_name.replace("/", "--"), "snapshots", "*", "tokenizer.json")
        hits = sorted(glob.glob(pat))
        if not hits:
            raise FileSystemError(f"tokenizer for '{model_name}' not in the local cache ({pat})")
        return Tokenizer.from_file(hits[-1])

    @staticmethod
    def from_gguf(gguf_tokenizer) -> "Tokenizer":
        g = gguf_tokenizer
        return Tokenizer(_GGUFBackend(g.tokens, g.scores, g.bos_token_id, g.eos_token_id, g.unknown_token_id,
                                      g.padding_token_id), "gguf")

    @staticmethod
    def from_model_weights(weights) -> "Tokenizer":
        if getattr(weights, "gguf_tokenizer", None) is None:
            raise LoadingError("model weights carry no GGUF tokenizer")
        return Tokenizer.from_gguf(weights.gguf_tokenizer)

    @staticmethod
    def from_vocab(tokens: Sequence[str], scores: Optional[Sequence[float]] = None, **kw) -> "Tokenizer":
        return Tokenizer(_GGUFBackend(tokens, scores, **kw), "gguf")

    # ---- API ----
    def encode(self, text: str) -> List[int]:
        """Basic backend wraps BOS/EOS like the reference; others add BOS only."""
        if self.kind == "basic":
            return [self._b.bos_token_id] + self._b.encode_raw(text) + [self._b.eos_token_id]
        return self.encode_with_special_tokens(text, add_bos=True, add_eos=False)

    def encode_raw(self, text: str) -> List[int]:
        return self._b.encode_raw(text)

    def encode_with_special_tokens(self, text: str, add_bos: bool = True, add_eos: bool = False) -> List[int]:
        ids = self._b.encode_raw(text)
        if add_bos:
            ids = [self._b.bos_token_id] + ids
        if add_eos:
            ids = ids + [self._b.eos_token_id]
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        return self._b.decode(ids, skip_special=True)

    def decode_raw(self, ids: Sequence[int]) -> str:
        return self._b.decode(ids, skip_special=False)

    def vocab_size(self) -> int: return self._b.vocab_size()
    def bos_token_id(self) -> int: return self._b.bos_token_id
    def eos_token_id(self) -> int: return self._b.eos_token_id
    def pad_token_id(self) -> int: return self._b.pad_token_id
    def unk_token_id(self) -> int: return self._b.unk_token_id
    def contains_token(self, tok: str) -> bool: return self._b.token_to_id(tok) is not None
    def token_to_id(self, tok: str) -> Optional[int]: return self._b.token_to_id(tok)
    def id_to_token(self, i: int) -> Optional[str]: return self._b.id_to_token(i)


class BatchTokenizer:
    """Pads / truncates a batch to a common length (``tokenizer.rs:636-683``)."""

    def __init__(self, tokenizer: Tokenizer):
        self.tokenizer = tokenizer

    def encode_batch(self, texts: Sequence[str], max_length: Optional[int] = None) -> Tuple[List[List[int]], List[List[int]]]:
        enc = [self.tokenizer.encode(t) for t in texts]
        L = max_length if max_length is not None else max((len(e) for e in enc), default=0)
        pad = self.tokenizer.pad_token_id()
        ids, mask = [], []
        for e in enc:
            e = e[:L]
            mask.append([1] * len(e) + [0] * (L - len(e)))
            ids.append(e + [pad] * (L - len(e)))
        return ids, mask

    def decode_batch(self, batch: Sequence[Sequence[int]]) -> List[str]:
        return [self.tokenizer.decode(b) for b in batch]

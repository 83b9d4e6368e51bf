"""Tokenizers behind one small interface and the vocabulary padding rule.

Every tokenizer is a :class:`Tokenizer`: ``tokenize(text) -> ids``, ``detokenize(ids) -> text``, ``vocab_size``,
``eod`` (end-of-document id), optionally ``pad`` and ``tokenize_batch``.  A subclass only supplies the backend
calls (``_encode``, ``_decode``, ``_size``, optionally ``_get_vocab``); everything else is derived here.
``build_tokenizer`` picks the class from a registry keyed by ``tokenizer_type`` and stores the padded vocabulary
size in the arguments.  Types and padding rule as in megatron/tokenizer/tokenizer.py:30-404; the
``SyntheticTokenizer`` (ids are their own tokens) exists only here, for training on synthetic tokens.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Optional, Sequence, Union

import numpy as np

EOD_TEXT, PAD_TEXT = "<|endoftext|>", "<|padding|>"


def _vocab_size_with_padding(orig_vocab_size: int, args) -> int:
    """Vocabulary rounded up to a multiple of ``make_vocab_size_divisible_by * model_parallel_size``
    (50277 -> 50304 at MP 1, 50432 at MP 2), so every tensor-parallel rank holds an equal, aligned slice."""
    unit = args.make_vocab_size_divisible_by * args.model_parallel_size
    padded = -(-orig_vocab_size // unit) * unit
    if args.rank in (0, None):
        print(f" > padded vocab (size: {orig_vocab_size}) with {padded - orig_vocab_size} dummy tokens "
              f"(new size: {padded})", flush=True)
    return padded


class Tokenizer:
    """Interface + shared behaviour.  ``eod_id`` / ``pad_id`` are set by the subclass (None = not available)."""

    name = "tokenizer"
    eod_id: Optional[int] = None
    pad_id: Optional[int] = None

    # ---- backend hooks
    def _encode(self, text: str) -> List[int]:
        raise NotImplementedError

    def _decode(self, ids: List[int]) -> str:
        raise NotImplementedError(f"detokenizer is not implemented for {self.name} tokenizer")

    def _size(self) -> int:
        raise NotImplementedError

    def _get_vocab(self) -> Dict[str, int]:
        raise NotImplementedError(f"{self.name} does not implement vocabulary access.")

    # ---- public surface
    @property
    def vocab_size(self) -> int:
        return self._size()

    @property
    def vocab(self) -> Dict[str, int]:
        return self._get_vocab()

    @property
    def inv_vocab(self) -> Dict[int, str]:
        return {i: t for t, i in self._get_vocab().items()}

    def tokenize(self, text: str) -> List[int]:
        return self._encode(text)

    def tokenize_batch(self, texts: Union[str, Sequence[str]]):
        return [self._encode(t) for t in ([texts] if isinstance(texts, str) else texts)]

    def detokenize(self, token_ids: Iterable[int]) -> str:
        return self._decode([int(t) for t in token_ids])

    def _special(self, what: str, value: Optional[int]) -> int:
        if value is None:
            raise NotImplementedError(f"{what} is not provided for {self.name} tokenizer")
        return value

    eod = property(lambda self: self._special("EOD", self.eod_id))
    pad = property(lambda self: self._special("PAD", self.pad_id))
    cls = property(lambda self: self._special("CLS", None))
    sep = property(lambda self: self._special("SEP", None))
    mask = property(lambda self: self._special("MASK", None))


AbstractTokenizer = Tokenizer       # the name other code bases import


class SyntheticTokenizer(Tokenizer):
    """Fixed-size vocabulary without text: ids are their own tokens (synthetic-token training)."""

    name, eod_id, pad_id = "Synthetic", 0, 1

    def __init__(self, vocab_size: int):
        self._n = int(vocab_size)

    def _size(self):
        return self._n

    def _get_vocab(self):
        return {str(i): i for i in range(self._n)}

    def _encode(self, text):
        return [int(t) % self._n for t in str(text).split() if t.lstrip("-").isdigit()]

    def _decode(self, ids):
        return " ".join(str(i) for i in ids)


class _TokenizersBackend(Tokenizer):
    """Anything driven by a ``tokenizers.Tokenizer`` object in ``self.tokenizer``."""

    def _size(self):
        return self.tokenizer.get_vocab_size()

    def _get_vocab(self):
        return self.tokenizer.get_vocab()

    def _encode(self, text):
        return self.tokenizer.encode(text).ids

    def _decode(self, ids):
        return self.tokenizer.decode(ids)


class _GPT2BPETokenizer(_TokenizersBackend):
    """Byte-level BPE from ``vocab.json`` + ``merges.txt``."""

    name = "GPT2 BPE"

    def __init__(self, vocab_file: str, merge_file: str):
        from tokenizers import Tokenizer as _Tok, decoders, models, pre_tokenizers
        self.tokenizer = _Tok(models.BPE.from_file(vocab_file, merge_file))
        self.tokenizer.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
        self.tokenizer.decoder = decoders.ByteLevel()
        self.eod_id = self.tokenizer.token_to_id(EOD_TEXT)
        if self.eod_id is None:
            raise KeyError(f"{vocab_file} has no {EOD_TEXT} token")


class HFTokenizer(_TokenizersBackend):
    """A ``tokenizers`` JSON file (e.g. the 20B tokenizer)."""

    name = "HFTokenizer"

    def __init__(self, vocab_file: str):
        from tokenizers import Tokenizer as _Tok
        self.tokenizer = _Tok.from_file(vocab_file)
        self.eod_id = self.tokenizer.token_to_id(EOD_TEXT)
        self.pad_id = self.tokenizer.token_to_id(PAD_TEXT)

    def tokenize_batch(self, texts):
        return self.tokenizer.encode_batch(texts)       # Encoding objects, as the preprocessing tools expect


class SentencePieceTokenizer(Tokenizer):
    name = "SPM"

    def __init__(self, vocab_file: str):
        import sentencepiece as spm
        self.tokenizer = spm.SentencePieceProcessor(model_file=vocab_file)
        self.eod_id = self.tokenizer.piece_to_id(EOD_TEXT)

    def _size(self):
        return self.tokenizer.get_piece_size()

    def _get_vocab(self):
        return {self.tokenizer.id_to_piece(i): i for i in range(self._size())}

    def _encode(self, text):
        return self.tokenizer.encode(text)

    def _decode(self, ids):
        return self.tokenizer.decode(ids)


class HFGPT2Tokenizer(Tokenizer):
    """``transformers`` GPT-2 tokenizer (fast by default) from a local path or the hub name ``gpt2``."""

    def __init__(self, vocab_file: Optional[str] = None, fast: bool = True):
        from transformers import GPT2Tokenizer, GPT2TokenizerFast
        self.name = "HFGPT2TokenizerFast" if fast else "HFGPT2Tokenizer"
        self.tokenizer = (GPT2TokenizerFast if fast else GPT2Tokenizer).from_pretrained(vocab_file or "gpt2")
        self.tokenizer.add_special_tokens({"pad_token": PAD_TEXT})
        self.eod_id, self.pad_id = self.tokenizer.eos_token_id, self.tokenizer.pad_token_id

    def _size(self):
        return len(self.tokenizer)

    def _get_vocab(self):
        return self.tokenizer.get_vocab()

    def _encode(self, text):
        return self.tokenizer.encode(text)

    def _decode(self, ids):
        return self.tokenizer.decode(ids)


class CharLevelTokenizer(Tokenizer):
    """One token per UTF-8 byte; 0 = end of document, 1 = padding.  Decoding maps ids below 32 to a space-range
    character so that control bytes never reach a terminal."""

    name, eod_id, pad_id = "CharLevelTokenizer", 0, 1

    def __init__(self, vocab_size: int):
        self._n = vocab_size

    def _size(self):
        return self._n

    def clamp(self, n: int) -> int:
        return max(32, min(n, self._n))

    def decode_token(self, token: int) -> str:
        return chr(self.clamp(token))

    def _encode(self, text):
        return list(np.frombuffer(text.encode("utf-8", errors="replace"), dtype=np.uint8).astype(np.int64))

    def tokenize_batch(self, texts):
        return [self._encode(t) for t in texts] if isinstance(texts, list) else self._encode(texts)

    def _decode(self, ids):
        return "".join(self.decode_token(i) for i in ids)


class TiktokenTokenizer(Tokenizer):
    name = "TiktokenTokenizer"

    def __init__(self, vocab_file: str):
        import tiktoken
        self.tokenizer = tiktoken.get_encoding(vocab_file)
        self.eod_id = self.tokenizer.eot_token

    def _size(self):
        return self.tokenizer.n_vocab

    def _encode(self, text):
        return self.tokenizer.encode(text)

    def tokenize_batch(self, texts):
        return self.tokenizer.encode_batch(texts, allowed_special="all")

    def _decode(self, ids):
        return self.tokenizer.decode(tokens=ids, errors="strict")


def _need(args, *fields):
    for f in fields:
        if getattr(args, f) is None:
            raise AssertionError(f"tokenizer_type {args.tokenizer_type} needs `{f}`")


def _make_hf_gpt2(args):
    if args.vocab_file is None:
        print("WARNING: No vocab file found, loading Huggingface's pretrained GPT2Tokenizer")
    return HFGPT2Tokenizer(args.vocab_file)


# tokenizer_type (lower case) -> (required argument fields, constructor from the arguments)
_REGISTRY: Dict[str, tuple] = {
    "gpt2bpetokenizer": (("vocab_file", "merge_file"), lambda a: _GPT2BPETokenizer(a.vocab_file, a.merge_file)),
    "spmtokenizer": (("vocab_file",), lambda a: SentencePieceTokenizer(a.vocab_file)),
    "hftokenizer": (("vocab_file",), lambda a: HFTokenizer(a.vocab_file)),
    "hfgpt2tokenizer": ((), _make_hf_gpt2),
    "charleveltokenizer": ((), lambda a: CharLevelTokenizer(vocab_size=512)),
    "tiktokentokenizer": (("vocab_file",), lambda a: TiktokenTokenizer(a.vocab_file)),
}


def build_tokenizer(args):
    """Build the tokenizer named by ``args.tokenizer_type`` and set ``args.padded_vocab_size``."""
    if args.rank in (0, None):
        print(f"> building {args.tokenizer_type} tokenizer ...", flush=True)
    if getattr(args, "dataset_impl", None) == "synthetic" and args.vocab_file is None:
        tokenizer = SyntheticTokenizer(args.synthetic_vocab_size)
    else:
        entry = _REGISTRY.get(args.tokenizer_type.lower())
        if entry is None:
            raise NotImplementedError(f"{args.tokenizer_type} tokenizer is not implemented.")
        _need(args, *entry[0])
        tokenizer = entry[1](args)
    args.padded_vocab_size = _vocab_size_with_padding(tokenizer.vocab_size, args)
    return tokenizer

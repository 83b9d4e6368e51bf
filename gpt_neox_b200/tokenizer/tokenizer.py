"""Tokenizers behind one interface (``vocab_size``, ``tokenize``, ``detokenize``, ``eod``) and the
vocabulary padding rule (megatron/tokenizer/tokenizer.py:30-404): GPT-2 byte-level BPE from
vocab/merges files, HF ``tokenizers`` JSON, HF GPT2 fast tokenizer, SentencePiece, character level
and tiktoken.  A ``SyntheticTokenizer`` (new here) stands in when training on synthetic tokens."""
from __future__ import annotations

import json
from abc import ABC, abstractmethod
from functools import lru_cache
from typing import List, Union

import numpy as np


def build_tokenizer(args):
    """Build the tokenizer named by ``args.tokenizer_type`` and set ``args.padded_vocab_size``."""
    if args.rank in (0, None):
        print(f"> building {args.tokenizer_type} tokenizer ...", flush=True)
    t = args.tokenizer_type.lower()
    if getattr(args, "dataset_impl", None) == "synthetic" and args.vocab_file is None:
        tokenizer = SyntheticTokenizer(args.synthetic_vocab_size)
    elif t == "GPT2BPETokenizer".lower():
        assert args.vocab_file is not None
        assert args.merge_file is not None
        tokenizer = _GPT2BPETokenizer(args.vocab_file, args.merge_file)
    elif t == "SPMTokenizer".lower():
        assert args.vocab_file is not None
        tokenizer = SentencePieceTokenizer(args.vocab_file)
    elif t == "HFTokenizer".lower():
        assert args.vocab_file is not None
        tokenizer = HFTokenizer(args.vocab_file)
    elif t == "HFGPT2Tokenizer".lower():
        if args.vocab_file is None:
            print("WARNING: No vocab file found, loading Huggingface's pretrained GPT2Tokenizer")
        tokenizer = HFGPT2Tokenizer(args.vocab_file)
    elif t == "CharLevelTokenizer".lower():
        tokenizer = CharLevelTokenizer(vocab_size=512)
    elif t == "TiktokenTokenizer".lower():
        assert args.vocab_file is not None
        tokenizer = TiktokenTokenizer(args.vocab_file)
    else:
        raise NotImplementedError(f"{args.tokenizer_type} tokenizer is not implemented.")
    args.padded_vocab_size = _vocab_size_with_padding(tokenizer.vocab_size, args)
    return tokenizer


def _vocab_size_with_padding(orig_vocab_size, args):
    """Round the vocabulary up to a multiple of ``make_vocab_size_divisible_by * model_parallel_size``
    (50277 -> 50304 at MP 1, 50432 at MP 2)."""
    multiple = args.make_vocab_size_divisible_by * args.model_parallel_size
    after = orig_vocab_size
    while after % multiple != 0:
        after += 1
    if args.rank in (0, None):
        print(f" > padded vocab (size: {orig_vocab_size}) with {after - orig_vocab_size} dummy tokens "
              f"(new size: {after})", flush=True)
    return after


class AbstractTokenizer(ABC):
    def __init__(self, name):
        self.name = name

    @property
    @abstractmethod
    def vocab_size(self):
        ...

    @property
    @abstractmethod
    def vocab(self):
        ...

    @property
    @abstractmethod
    def inv_vocab(self):
        ...

    @abstractmethod
    def tokenize(self, text):
        ...

    def detokenize(self, token_ids):
        raise NotImplementedError(f"detokenizer is not implemented for {self.name} tokenizer")

    @property
    def cls(self):
        raise NotImplementedError(f"CLS is not provided for {self.name} tokenizer")

    @property
    def sep(self):
        raise NotImplementedError(f"SEP is not provided for {self.name} tokenizer")

    @property
    def pad(self):
        raise NotImplementedError(f"PAD is not provided for {self.name} tokenizer")

    @property
    def eod(self):
        raise NotImplementedError(f"EOD is not provided for {self.name} tokenizer")

    @property
    def mask(self):
        raise NotImplementedError(f"MASK is not provided for {self.name} tokenizer")


class SyntheticTokenizer(AbstractTokenizer):
    """Fixed-size vocabulary without text: ids are their own tokens (synthetic-token training)."""

    def __init__(self, vocab_size):
        super().__init__("Synthetic")
        self._n = int(vocab_size)
        self.eod_id = 0
        self.pad_id = 1

    @property
    def vocab_size(self):
        return self._n

    @property
    def vocab(self):
        return {str(i): i for i in range(self._n)}

    @property
    def inv_vocab(self):
        return {i: str(i) for i in range(self._n)}

    def tokenize(self, text):
        return [int(t) % self._n for t in str(text).split() if t.lstrip("-").isdigit()]

    def detokenize(self, token_ids):
        return " ".join(str(int(t)) for t in token_ids)

    @property
    def eod(self):
        return self.eod_id


@lru_cache()
def _bytes_to_unicode():
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(2 ** 8):
        if b not in bs:
            bs.append(b)
            cs.append(2 ** 8 + n)
            n += 1
    return dict(zip(bs, [chr(c) for c in cs]))


class _GPT2BPETokenizer(AbstractTokenizer):
    """Byte-level BPE from ``vocab.json`` + ``merges.txt``, executed by the ``tokenizers`` library."""

    def __init__(self, vocab_file, merge_file):
        super().__init__("GPT2 BPE")
        from tokenizers import Tokenizer, decoders, models, pre_tokenizers
        tok = Tokenizer(models.BPE.from_file(vocab_file, merge_file))
        tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
        tok.decoder = decoders.ByteLevel()
        self.tokenizer = tok
        self._vocab = tok.get_vocab()
        self._inv = {v: k for k, v in self._vocab.items()}
        self.eod_id = self._vocab["<|endoftext|>"]

    @property
    def vocab_size(self):
        return len(self._vocab)

    @property
    def vocab(self):
        return self._vocab

    @property
    def inv_vocab(self):
        return self._inv

    def tokenize(self, text):
        return self.tokenizer.encode(text).ids

    def detokenize(self, token_ids):
        return self.tokenizer.decode(list(map(int, token_ids)))

    @property
    def eod(self):
        return self.eod_id


class SentencePieceTokenizer(AbstractTokenizer):
    def __init__(self, vocab_file):
        super().__init__("SPM")
        import sentencepiece as spm
        self.tokenizer = spm.SentencePieceProcessor(model_file=vocab_file)
        self.eod_id = self.tokenizer.piece_to_id("<|endoftext|>")

    @property
    def vocab_size(self):
        return self.tokenizer.get_piece_size()

    @property
    def vocab(self):
        return {self.tokenizer.id_to_piece(i): i for i in range(self.tokenizer.get_piece_size())}

    @property
    def inv_vocab(self):
        return {i: self.tokenizer.id_to_piece(i) for i in range(self.tokenizer.get_piece_size())}

    def tokenize(self, text):
        return self.tokenizer.encode(text)

    def detokenize(self, token_ids):
        return self.tokenizer.decode(list(map(int, token_ids)))

    @property
    def eod(self):
        return self.eod_id


class HFTokenizer(AbstractTokenizer):
    """A ``tokenizers`` JSON file (e.g. the 20B tokenizer)."""

    def __init__(self, vocab_file):
        super().__init__("HFTokenizer")
        from tokenizers import Tokenizer
        self.tokenizer = Tokenizer.from_file(vocab_file)
        self.eod_id = self.tokenizer.token_to_id("<|endoftext|>")
        self.pad_id = self.tokenizer.token_to_id("<|padding|>")

    @property
    def vocab_size(self):
        return self.tokenizer.get_vocab_size()

    @property
    def vocab(self):
        return self.tokenizer.get_vocab()

    @property
    def inv_vocab(self):
        return {v: k for k, v in self.tokenizer.get_vocab().items()}

    def tokenize(self, text: str):
        return self.tokenizer.encode(text).ids

    def tokenize_batch(self, text_batch: Union[List[str], str]):
        return self.tokenizer.encode_batch(text_batch)

    def detokenize(self, token_ids):
        return self.tokenizer.decode(list(map(int, token_ids)))

    @property
    def eod(self):
        return self.eod_id


class HFGPT2Tokenizer(AbstractTokenizer):
    def __init__(self, vocab_file=None, fast=True):
        name = "HFGPT2TokenizerFast" if fast else "HFGPT2Tokenizer"
        super().__init__(name)
        if vocab_file is None:
            vocab_file = "gpt2"
        from transformers import GPT2Tokenizer, GPT2TokenizerFast
        self.tokenizer = (GPT2TokenizerFast if fast else GPT2Tokenizer).from_pretrained(vocab_file)
        self.tokenizer.add_special_tokens({"pad_token": "<|padding|>"})
        self.eod_id = self.tokenizer.eos_token_id
        self.pad_id = self.tokenizer.pad_token_id

    @property
    def vocab_size(self):
        return len(self.tokenizer)

    @property
    def vocab(self):
        return self.tokenizer.get_vocab()

    @property
    def inv_vocab(self):
        return {v: k for k, v in self.tokenizer.get_vocab().items()}

    def tokenize(self, text: str):
        return self.tokenizer.encode(text)

    def tokenize_batch(self, text_batch):
        return [self.tokenize(t) for t in ([text_batch] if isinstance(text_batch, str) else text_batch)]

    def detokenize(self, token_ids):
        return self.tokenizer.decode(list(map(int, token_ids)))

    @property
    def eod(self):
        return self.eod_id


class CharLevelTokenizer(AbstractTokenizer):
    """One token per byte; 0 = end of document, 1 = padding."""

    def __init__(self, vocab_size):
        super().__init__("CharLevelTokenizer")
        self._vocab_size = vocab_size
        self.eod_id = 0
        self.pad_id = 1

    def clamp(self, n):
        return max(32, min(n, self.vocab_size))

    @property
    def vocab_size(self):
        return self._vocab_size

    @property
    def vocab(self):
        raise NotImplementedError

    @property
    def inv_vocab(self):
        raise NotImplementedError

    def decode_token(self, token: int):
        return str(chr(self.clamp(token)))

    def tokenize(self, text: str):
        return list(np.frombuffer(text.encode("utf-8", errors="replace"), dtype=np.uint8).astype(np.int64))

    def tokenize_batch(self, text_batch):
        if isinstance(text_batch, list):
            return [self.tokenize(s) for s in text_batch]
        return self.tokenize(text_batch)

    def detokenize(self, token_ids):
        return "".join(map(self.decode_token, token_ids))

    @property
    def eod(self):
        return self.eod_id


class TiktokenTokenizer(AbstractTokenizer):
    def __init__(self, vocab_file):
        super().__init__("TiktokenTokenizer")
        import tiktoken
        self.tokenizer = tiktoken.get_encoding(vocab_file)
        self.eod_id = self.tokenizer.eot_token
        self.pad_id = None

    @property
    def vocab_size(self):
        return self.tokenizer.n_vocab

    @property
    def vocab(self):
        raise NotImplementedError("TiktokenTokenizer does not implement vocabulary access.")

    @property
    def inv_vocab(self):
        raise NotImplementedError("TiktokenTokenizer does not implement vocabulary access.")

    def tokenize(self, text: str):
        return self.tokenizer.encode(text)

    def tokenize_batch(self, text_batch: List[str]):
        return self.tokenizer.encode_batch(text_batch, allowed_special="all")

    def detokenize(self, token_ids):
        return self.tokenizer.decode(tokens=list(map(int, token_ids)), errors="strict")

    @property
    def eod(self):
        return self.eod_id

    @property
    def pad(self):
        raise NotImplementedError

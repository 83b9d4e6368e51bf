"""Train a byte-level BPE tokenizer on jsonl corpora and write a ``tokenizer.json`` for ``HFTokenizer``.

Counterpart of megatron/tokenizer/train_tokenizer.py:49-84 (BPE model, byte-level pre-tokeniser with prefix
space, NFKC normaliser, the special tokens ``<|endoftext|>`` and ``<|padding|>``).  Documents are streamed
from the files line by line, so a corpus never has to fit in memory; ``.jsonl``, ``.json`` and their
``.gz`` forms are read.

    python -m gpt_neox_b200.tokenizer.train_tokenizer --json_input_dir data/ --tokenizer_output_path tok.json -v 52000
"""
from __future__ import annotations

import argparse
import glob
import gzip
import json
import os
from typing import Iterator, Sequence

SPECIAL_TOKENS = ("<|endoftext|>", "<|padding|>")


def corpus_files(input_dir: str) -> list:
    pats = ("*.jsonl", "*.json", "*.jsonl.gz", "*.json.gz")
    return sorted(f for p in pats for f in glob.glob(os.path.join(input_dir, p)))


def iter_documents(input_dir: str, text_key: str = "text") -> Iterator[str]:
    """Yield the ``text_key`` field of every record of every corpus file (one JSON object per line)."""
    for path in corpus_files(input_dir):
        opener = gzip.open if path.endswith(".gz") else open
        with opener(path, "rt", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                rec = json.loads(line)
                if text_key in rec and rec[text_key]:
                    yield rec[text_key]


def train_tokenizer(input_dir: str, save_path: str = None, tokenizer_type: str = "BPE", vocab_size: int = 52000,
                    text_key: str = "text", special_tokens: Sequence[str] = SPECIAL_TOKENS, min_frequency: int = 2):
    """Returns the trained ``tokenizers.Tokenizer``; saved (pretty-printed) when ``save_path`` is given."""
    if tokenizer_type != "BPE":
        raise NotImplementedError(f"Tokenizer type {tokenizer_type} not implemented")
    if not corpus_files(input_dir):
        raise FileNotFoundError(f"no .jsonl / .json files in {input_dir}")
    from tokenizers import Tokenizer, decoders, models, normalizers, pre_tokenizers, processors, trainers
    tok = Tokenizer(models.BPE())
    tok.normalizer = normalizers.NFKC()
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=True)
    tok.post_processor = processors.ByteLevel(trim_offsets=True)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=int(vocab_size), special_tokens=list(special_tokens),
                                  min_frequency=int(min_frequency), show_progress=False,
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(iter_documents(input_dir, text_key), trainer)
    if save_path:
        os.makedirs(os.path.dirname(os.path.abspath(save_path)), exist_ok=True)
        tok.save(save_path, pretty=True)
        print(f"Tokenizer saved at {save_path}")
    return tok


def parse_args(input_args=None):
    p = argparse.ArgumentParser(description="Train a byte-level BPE tokenizer on jsonl files")
    p.add_argument("--json_input_dir", type=str, required=True, help="folder with the training data (jsonl)")
    p.add_argument("--tokenizer_output_path", type=str, required=True, help="where to write the tokenizer (.json)")
    p.add_argument("--tokenizer_type", type=str, choices=["BPE"], default="BPE")
    p.add_argument("-v", "--vocab_size", type=int, default=52000)
    p.add_argument("--text_key", type=str, default="text")
    p.add_argument("--min_frequency", type=int, default=2)
    return p.parse_args(input_args)


def main(args=None):
    a = parse_args(args) if not isinstance(args, argparse.Namespace) else args
    train_tokenizer(a.json_input_dir, save_path=a.tokenizer_output_path, tokenizer_type=a.tokenizer_type,
                    vocab_size=a.vocab_size, text_key=getattr(a, "text_key", "text"),
                    min_frequency=getattr(a, "min_frequency", 2))


if __name__ == "__main__":
    main()

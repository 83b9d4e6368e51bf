"""Tokenise raw text into the indexed binary datasets the training loader reads.

One pipeline (reader -> worker pool -> one indexed-dataset builder per output stream), three front ends:

* ``python -m gpt_neox_b200.data.preprocess_data``                      plain documents
  (tools/datasets/preprocess_data.py:43-268)
* ``python -m gpt_neox_b200.data.preprocess_data --mask-before-token``   also writes a ``_label`` stream
  whose tokens up to and including the first occurrence of the pattern are -100
  (tools/datasets/preprocess_data_with_mask.py)
* ``python -m gpt_neox_b200.data.preprocess_data --chat-template``       conversations rendered with the
  tokenizer's chat template, with per-role loss masks and optional reward streams
  (tools/datasets/preprocess_data_with_chat_template.py:78-383)

Inputs: ``.jsonl`` (optionally ``.gz`` / ``.zst``), or ``.txt`` with one document per line; several files as a
comma-separated list.  Outputs: ``<prefix>_<key>_document.{bin,idx}`` (+ ``_label`` / ``_reward``).
"""
from __future__ import annotations

import argparse
import os
import gzip
import io
import json
import multiprocessing
import sys
import time
from types import SimpleNamespace
from typing import Dict, Iterable, List, Tuple

import numpy as np

from . import indexed_dataset

TOKENIZER_CHOICES = ["HFGPT2Tokenizer", "HFTokenizer", "GPT2BPETokenizer", "CharLevelTokenizer", "TiktokenTokenizer",
                     "SPMTokenizer"]


# ----------------------------------------------------------------------------------------- reading
def _open_text(path):
    if path.endswith(".gz"):
        return io.TextIOWrapper(gzip.open(path, "rb"), encoding="utf-8")
    if path.endswith(".zst"):
        try:
            import zstandard
        except ImportError as e:
            raise RuntimeError("reading .zst input needs the `zstandard` package") from e
        return io.TextIOWrapper(zstandard.ZstdDecompressor().stream_reader(open(path, "rb")), encoding="utf-8")
    return open(path, "r", encoding="utf-8")


def yield_from_files(paths: Iterable[str], keys: List[str], raw_json: bool = False):
    """Documents of every input file, in order.  jsonl rows give ``row[keys[0]]`` (or the whole row when
    ``raw_json``); other files give one document per non-empty line."""
    for path in paths:
        is_json = ".jsonl" in path or path.endswith(".json")
        with _open_text(path) as f:
            for line in f:
                line = line.rstrip("\n")
                if not line.strip():
                    continue
                if is_json:
                    row = json.loads(line)
                    yield row if raw_json else row[keys[0]] if isinstance(row, dict) else row
                else:
                    yield line


# ----------------------------------------------------------------------------------------- masking helpers
def find_subsequence(seq, pattern) -> int:
    """Index of the first occurrence of ``pattern`` in ``seq`` (-1 if absent); linear time via the
    prefix-function of ``pattern + [sentinel] + seq``."""
    m = len(pattern)
    if m == 0:
        return 0
    fail = [0] * m
    k = 0
    for i in range(1, m):
        while k and pattern[i] != pattern[k]:
            k = fail[k - 1]
        if pattern[i] == pattern[k]:
            k += 1
        fail[i] = k
    k = 0
    for i, tok in enumerate(seq):
        while k and tok != pattern[k]:
            k = fail[k - 1]
        if tok == pattern[k]:
            k += 1
        if k == m:
            return i - m + 1
    return -1


def mask_before(tokens: List[int], pattern: List[int]) -> List[int]:
    """Label stream: -100 up to and including the first occurrence of ``pattern`` (everything if absent)."""
    at = find_subsequence(tokens, pattern)
    cut = len(tokens) if at < 0 else at + len(pattern)
    return [-100] * cut + list(tokens[cut:])


def build_chat(chat, generation_role: str, apply_mask: bool, tokenizer, only_last_turn: bool = False,
               for_rm: bool = False) -> Tuple[List[int], List[int]]:
    """Render ``[{role, content}, ...]`` with the tokenizer's chat template.  Returns (tokens, labels) where
    labels are -100 on every token the model is not trained to produce: turns of other roles (``apply_mask``),
    every turn but the last (``only_last_turn``), or everything but a final EOS (``for_rm``)."""
    if not apply_mask:
        toks = list(tokenizer.apply_chat_template(chat))
        return toks, list(toks)
    eos = tokenizer.eos_token_id
    if for_rm:
        if eos is None:
            raise ValueError("Tokenizer does not have an EOS token, unable to determine good mask, please edit "
                             "and make your own.")
        toks = list(tokenizer.apply_chat_template(chat))
        # labels are read shifted by one (input[:-1], label[1:]): two EOS so that exactly the last one is scored
        return toks + [eos, eos], [-100] * (len(toks) + 1) + [eos]
    toks: List[int] = []
    labels: List[int] = []
    for i, turn in enumerate(chat):
        nxt_is_gen = i + 1 < len(chat) and chat[i + 1]["role"] == generation_role
        piece = list(tokenizer.apply_chat_template(chat[: i + 1], add_generation_prompt=nxt_is_gen))[len(toks):]
        toks.extend(piece)
        hide = (only_last_turn and i != len(chat) - 1) or turn["role"] != generation_role
        labels.extend([-100] * len(piece) if hide else piece)
    if eos is not None:
        labels.append(eos if labels and labels[-1] != -100 else -100)
        toks.append(eos)
    return toks, labels


# ----------------------------------------------------------------------------------------- worker
class Encoder:
    """Runs in the pool workers: ``initializer`` builds the tokenizer once per process."""
    tokenizer = None

    def __init__(self, args):
        self.args = args

    def initializer(self):
        if self.args.chat_template:
            from transformers import AutoTokenizer
            Encoder.tokenizer = AutoTokenizer.from_pretrained(self.args.tokenizer_path)
        else:
            from ..tokenizer import build_tokenizer
            Encoder.tokenizer = build_tokenizer(self.args)

    def encode(self, doc) -> Tuple[Dict[str, List[List[int]]], int]:
        a = self.args
        out: Dict[str, List[List[int]]] = {}
        if a.chat_template:
            for key in a.jsonl_keys:
                toks, labels = build_chat(doc[key], a.generation_role, not a.no_mask, Encoder.tokenizer,
                                          a.only_last, a.for_rm)
                out[key] = [toks]
                out[key + "_label"] = [labels]
                if a.reward_key is not None:
                    r = doc[a.reward_key]
                    out[key + "_reward"] = [[float(r)] if not a.binary_reward else [1.0 if r else 0.0]]
            return out, len(json.dumps(doc))
        text = doc["text"] if isinstance(doc, dict) else doc
        if a.ftfy:
            import ftfy
            text = ftfy.fix_text(text)
        ids = Encoder.tokenizer.tokenize(text)
        for key in a.jsonl_keys:
            sents = [list(ids)] if ids else []
            if a.append_eod:
                if not sents:
                    sents = [[]]
                sents[-1].append(Encoder.tokenizer.eod)
            out[key] = sents
            if a.mask_before_token is not None:
                out[key + "_label"] = [mask_before(s, a.mask_before_token) for s in sents]
        return out, len(text)


# ----------------------------------------------------------------------------------------- driver
def process_share_from_env(env=None):
    """(rank, world size) of this process among the preprocessing workers of a multi-node job: ``RANK`` /
    ``WORLD_SIZE`` first, then SLURM's, then Open MPI's variables (tools/datasets/multinode_prepare_data.sh:15-16);
    (0, 1) when none is set."""
    env = os.environ if env is None else env
    for r, w in (("RANK", "WORLD_SIZE"), ("SLURM_PROCID", "SLURM_NTASKS"),
                 ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE")):
        if r in env and w in env:
            return int(env[r]), int(env[w])
    return 0, 1


def share_of(items, rank: int, world: int):
    """Contiguous, balanced share of ``items`` for ``rank``: the first ``len % world`` ranks get one more."""
    n, rem = divmod(len(items), world)
    lo = rank * n + min(rank, rem)
    return list(items[lo:lo + n + (1 if rank < rem else 0)])


def get_args(input_args=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    g = p.add_argument_group("input data")
    g.add_argument("--input", type=str, default=None, help="comma-separated input files")
    g.add_argument("--input-list", type=str, default=None,
                   help="text file with one input path per line; with several processes (RANK / WORLD_SIZE, or the "
                        "SLURM / Open MPI equivalents) each takes a contiguous share of the lines and appends its "
                        "rank to --output-prefix (merge the parts with data/dataset_tools.py merge)")
    g.add_argument("--jsonl-keys", nargs="+", default=None, help="keys to extract (default: text / conversation)")
    g.add_argument("--num-docs", type=int, default=None, help="number of documents, for the progress report")
    g.add_argument("--mask-before-token", type=str, default=None,
                   help="comma-separated token ids; labels are masked up to and including their first occurrence")
    g = p.add_argument_group("chat template")
    g.add_argument("--chat-template", action="store_true", help="rows hold conversations; use the HF chat template")
    g.add_argument("--tokenizer-path", type=str, default=None, help="HF tokenizer directory (chat template mode)")
    g.add_argument("--no-mask", action="store_true")
    g.add_argument("--for-rm", action="store_true")
    g.add_argument("--generation-role", type=str, default="assistant")
    g.add_argument("--only-last", action="store_true")
    g.add_argument("--reward-key", type=str, default=None)
    g.add_argument("--binary-reward", action="store_true")
    g = p.add_argument_group("tokenizer")
    g.add_argument("--tokenizer-type", type=str, default=None, choices=TOKENIZER_CHOICES)
    g.add_argument("--vocab-file", type=str, default=None)
    g.add_argument("--merge-file", type=str, default=None)
    g.add_argument("--append-eod", action="store_true")
    g.add_argument("--ftfy", action="store_true")
    g = p.add_argument_group("output data")
    g.add_argument("--output-prefix", type=str, required=True)
    g.add_argument("--dataset-impl", type=str, default="mmap", choices=["lazy", "cached", "mmap"])
    g = p.add_argument_group("runtime")
    g.add_argument("--workers", type=int, default=1)
    g.add_argument("--log-interval", type=int, default=100)
    a = p.parse_args(input_args)
    if (a.input is None) == (a.input_list is None):
        p.error("give exactly one of --input and --input-list")
    if a.input_list is not None:
        rank, world = process_share_from_env()
        with open(a.input_list) as f:
            paths = [ln.strip() for ln in f if ln.strip()]
        mine = share_of(paths, rank, world)
        if not mine:
            p.error(f"rank {rank} of {world}: no input files in its share of {a.input_list}")
        a.input = ",".join(mine)
        if world > 1:
            a.output_prefix = f"{a.output_prefix}{rank}"
        print(f"rank {rank} of {world}: {len(mine)} of {len(paths)} input files -> {a.output_prefix}")
    if a.chat_template:
        if a.tokenizer_path is None:
            p.error("--chat-template needs --tokenizer-path")
        a.jsonl_keys = a.jsonl_keys or ["conversation"]
    else:
        if a.tokenizer_type is None:
            p.error("--tokenizer-type is required")
        a.jsonl_keys = a.jsonl_keys or ["text"]
    if a.mask_before_token is not None:
        a.mask_before_token = [int(t) for t in a.mask_before_token.split(",") if t.strip()]
    # the tokenizer builder reads these
    a.rank, a.model_parallel_size, a.make_vocab_size_divisible_by, a.keep_last = 0, 1, 128, True
    return a


def _vocab_size(args):
    if args.chat_template:
        from transformers import AutoTokenizer
        return len(AutoTokenizer.from_pretrained(args.tokenizer_path))
    from ..tokenizer import build_tokenizer
    t = build_tokenizer(SimpleNamespace(**vars(args)))
    return getattr(t, "vocab_size", None) or args.padded_vocab_size


def _set_dtype(builder, dt):
    if hasattr(builder, "_dtype"):
        builder._dtype = dt
    else:
        builder.dtype = dt
        builder.element_size = builder.element_sizes[dt]


def main(input_args=None):
    args = get_args(input_args)
    enc = Encoder(args)
    vocab = _vocab_size(args)
    print(f"Vocab size: {vocab}")
    print(f"Output prefix: {args.output_prefix}")
    docs = yield_from_files(args.input.split(","), args.jsonl_keys, raw_json=args.chat_template)
    if args.workers > 1:
        pool = multiprocessing.Pool(args.workers, initializer=enc.initializer)
        encoded = pool.imap(enc.encode, docs, chunksize=25)
    else:
        pool = None
        enc.initializer()
        encoded = (enc.encode(d) for d in docs)
    streams = list(args.jsonl_keys)
    if args.chat_template or args.mask_before_token is not None:
        streams += [k + "_label" for k in args.jsonl_keys]
    if args.chat_template and args.reward_key is not None:
        streams += [k + "_reward" for k in args.jsonl_keys]
    builders, bins, idxs = {}, {}, {}
    for s in streams:
        bins[s] = f"{args.output_prefix}_{s}_document.bin"
        idxs[s] = f"{args.output_prefix}_{s}_document.idx"
        builders[s] = indexed_dataset.make_builder(bins[s], impl=args.dataset_impl, vocab_size=vocab)
        if s.endswith("_label"):
            _set_dtype(builders[s], np.int32)        # labels hold -100
        elif s.endswith("_reward"):
            _set_dtype(builders[s], np.float32)
    t0 = time.time()
    nbytes = 0
    n = 0
    for n, (doc, size) in enumerate(encoded, start=1):
        nbytes += size
        for key, sents in doc.items():
            for sent in sents:
                builders[key].add_item(np.array(sent, dtype=builders[key].dtype))
            builders[key].end_document()
        if n % args.log_interval == 0:
            dt = time.time() - t0
            total = f"/{args.num_docs}" if args.num_docs else ""
            print(f"Processed {n}{total} documents ({n / dt:.2f} docs/s, {nbytes / dt / 1048576:.2f} MB/s).",
                  file=sys.stderr)
    if pool is not None:
        pool.close()
        pool.join()
    for s in streams:
        builders[s].finalize(idxs[s])
    print(f"Wrote {n} documents to {len(streams)} stream(s) in {time.time() - t0:.1f}s")
    return {s: bins[s][:-4] for s in streams}


if __name__ == "__main__":
    main()

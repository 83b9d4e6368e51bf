"""Turn a preference dataset into the JSONL files the SFT / DPO / RM / KTO recipes tokenise.

Input records carry two chat transcripts, ``chosen`` and ``rejected`` (lists of ``{"role", "content"}``), as in
HuggingFaceH4/ultrafeedback_binarized; the reference's data scripts do the same split (post-training/llama_data.py:1-49,
post-training/dpo_data.py).  Source: a local JSONL file (``--input``), or a Hugging Face dataset name when the
``datasets`` package and network are available (``--hf-dataset``, ``--hf-split``).

    python post-training/prepare_preference_data.py --input prefs_train.jsonl --split train --out data
    python prepare_data.py ...   # or: python -m gpt_neox_b200.data.preprocess_data --chat-template ... per recipe

Outputs under ``<out>``:
    pairwise/<name>_dpo_<split>.jsonl   {"chosen": [...], "rejected": [...]}                  (DPO, reward model)
    sft/<name>_sft_<split>.jsonl        {"messages": chosen}                                   (SFT)
    kto/<name>_kto_<split>.jsonl        {"messages": chosen, "reward": 1} / {rejected, -1}     (KTO)
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Iterable, Iterator


def read_records(path: str) -> Iterator[dict]:
    with open(path) as f:
        for line in f:
            if line.strip():
                yield json.loads(line)


def hf_records(name: str, split: str) -> Iterator[dict]:
    from datasets import load_dataset            # optional dependency
    yield from load_dataset(name, split=split)


def valid_pair(rec: dict) -> bool:
    c, r = rec.get("chosen"), rec.get("rejected")
    return bool(c) and bool(r) and c != r and c[-1].get("role") == "assistant" and r[-1].get("role") == "assistant"


def write_recipes(records: Iterable[dict], out: str, name: str, split: str, keep_invalid: bool = False) -> dict:
    paths = {k: os.path.join(out, d, f"{name}_{k}_{split}.jsonl") for k, d in
             (("dpo", "pairwise"), ("sft", "sft"), ("kto", "kto"))}
    for p in paths.values():
        os.makedirs(os.path.dirname(p), exist_ok=True)
    counts = {"pairs": 0, "dropped": 0}
    with open(paths["dpo"], "w") as fd, open(paths["sft"], "w") as fs, open(paths["kto"], "w") as fk:
        for rec in records:
            if not keep_invalid and not valid_pair(rec):
                counts["dropped"] += 1
                continue
            counts["pairs"] += 1
            fd.write(json.dumps({"chosen": rec["chosen"], "rejected": rec["rejected"]}) + "\n")
            fs.write(json.dumps({"messages": rec["chosen"]}) + "\n")
            fk.write(json.dumps({"messages": rec["chosen"], "reward": 1}) + "\n")
            fk.write(json.dumps({"messages": rec["rejected"], "reward": -1}) + "\n")
    counts["paths"] = paths
    return counts


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--input", type=str, help="JSONL with `chosen` / `rejected` transcripts")
    src.add_argument("--hf-dataset", type=str, help="Hugging Face dataset name (needs `datasets` + network)")
    ap.add_argument("--hf-split", type=str, default="train_prefs")
    ap.add_argument("--split", type=str, default="train")
    ap.add_argument("--name", type=str, default="prefs")
    ap.add_argument("--out", type=str, default="data")
    ap.add_argument("--keep-invalid", action="store_true", help="keep pairs without two distinct assistant endings")
    a = ap.parse_args(argv)
    recs = read_records(a.input) if a.input else hf_records(a.hf_dataset, a.hf_split)
    c = write_recipes(recs, a.out, a.name, a.split, a.keep_invalid)
    print(json.dumps(c))


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Download and tokenise a registered corpus (reference: prepare_data.py:29-77)."""
import argparse

from gpt_neox_b200.data.corpora import DATA_DOWNLOADERS, prepare_dataset
from gpt_neox_b200.data.preprocess_data import TOKENIZER_CHOICES

DATASET_CHOICES = [i for i in DATA_DOWNLOADERS if i != "pass"]


def get_args(argv=None):
    p = argparse.ArgumentParser(description="Download & preprocess neox datasets")
    p.add_argument("dataset", nargs="?", default="enwik8", choices=DATASET_CHOICES, help="name of dataset to download.")
    p.add_argument("-t", "--tokenizer", default="GPT2BPETokenizer", choices=TOKENIZER_CHOICES)
    p.add_argument("-d", "--data-dir", default=None, help="defaults to ./data")
    p.add_argument("-v", "--vocab-file", default=None)
    p.add_argument("-m", "--merge-file", default=None)
    p.add_argument("-f", "--force-redownload", dest="force_redownload", default=False, action="store_true")
    return p.parse_args(argv)


if __name__ == "__main__":
    a = get_args()
    prepare_dataset(dataset_name=a.dataset, tokenizer_type=a.tokenizer, data_dir=a.data_dir, vocab_file=a.vocab_file,
                    merge_file=a.merge_file, force_redownload=a.force_redownload)

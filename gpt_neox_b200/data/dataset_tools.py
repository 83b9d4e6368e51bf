"""Small dataset utilities: count tokens of indexed datasets, merge datasets
(tools/datasets/dataset_token_count.py, tools/datasets/merge_datasets.py).

    python -m gpt_neox_b200.data.dataset_tools count  <prefix> [<prefix> ...]
    python -m gpt_neox_b200.data.dataset_tools merge  --input <dir> --output-prefix <prefix>
"""
from __future__ import annotations

import argparse
import os

import numpy as np

from . import indexed_dataset


def token_count(prefix: str, skip_warmup=True) -> int:
    ds = indexed_dataset.make_dataset(prefix, impl=indexed_dataset.infer_dataset_impl(prefix) or "mmap",
                                      skip_warmup=skip_warmup)
    return int(np.sum(ds.sizes))


def merge(input_dir: str, output_prefix: str):
    """Concatenate every ``<name>.{bin,idx}`` pair of ``input_dir`` (sorted by name) into one dataset."""
    prefixes = sorted({os.path.join(input_dir, f[:-4]) for f in os.listdir(input_dir)
                       if f.endswith(".bin") and os.path.isfile(os.path.join(input_dir, f[:-4] + ".idx"))})
    if not prefixes:
        raise FileNotFoundError(f"no .bin/.idx pairs in {input_dir}")
    builder = None
    for pfx in prefixes:
        if builder is None:
            first = indexed_dataset.make_dataset(pfx, "mmap", skip_warmup=True)
            builder = indexed_dataset.MMapIndexedDatasetBuilder(indexed_dataset.data_file_path(output_prefix),
                                                                dtype=first.dtype)
            del first
        builder.merge_file_(pfx)
    builder.finalize(indexed_dataset.index_file_path(output_prefix))
    return output_prefix


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = p.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("count")
    c.add_argument("prefixes", nargs="+")
    m = sub.add_parser("merge")
    m.add_argument("--input", required=True)
    m.add_argument("--output-prefix", required=True)
    a = p.parse_args(argv)
    if a.cmd == "count":
        for pfx in a.prefixes:
            print(f"{pfx}: {token_count(pfx)} tokens")
    else:
        print("merged into", merge(a.input, a.output_prefix))


if __name__ == "__main__":
    main()

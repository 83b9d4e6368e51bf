#!/usr/bin/env python
"""Merge indexed datasets into one.

Forwards its command line to ``python -m gpt_neox_b200.data.dataset_tools merge`` (reference script: tools/datasets/merge_datasets.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.data.dataset_tools import main  # noqa: E402

if __name__ == "__main__":
    main(["merge"] + sys.argv[1:])

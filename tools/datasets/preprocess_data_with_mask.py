#!/usr/bin/env python
"""Tokenise jsonl documents and write a label mask (--mask-before-token).

Forwards its command line to ``python -m gpt_neox_b200.data.preprocess_data`` (reference script: tools/datasets/preprocess_data_with_mask.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.data.preprocess_data import main  # noqa: E402

if __name__ == "__main__":
    main(sys.argv[1:])

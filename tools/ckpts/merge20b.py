#!/usr/bin/env python
"""Merge the tensor-parallel shards of a checkpoint into one model-parallel rank.

Forwards its command line to ``python -m gpt_neox_b200.ckpt.convert merge`` (reference script: tools/ckpts/merge20b.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.ckpt.convert import main  # noqa: E402

if __name__ == "__main__":
    main(["merge"] + sys.argv[1:])

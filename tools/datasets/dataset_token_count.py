#!/usr/bin/env python
"""Count the tokens of indexed datasets.

Forwards its command line to ``python -m gpt_neox_b200.data.dataset_tools count`` (reference script: tools/datasets/dataset_token_count.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.data.dataset_tools import main  # noqa: E402

if __name__ == "__main__":
    main(["count"] + sys.argv[1:])

#!/usr/bin/env python
"""Print (or --diff two) checkpoint files.

Forwards its command line to ``python -m gpt_neox_b200.ckpt.convert inspect`` (reference script: tools/ckpts/inspect_checkpoints.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.ckpt.convert import main  # noqa: E402

if __name__ == "__main__":
    main(["inspect"] + sys.argv[1:])

#!/usr/bin/env python
"""Upload a converted Hugging Face directory to the hub.

Forwards its command line to ``python -m gpt_neox_b200.ckpt.convert upload`` (reference script: tools/ckpts/upload.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.ckpt.convert import main  # noqa: E402

if __name__ == "__main__":
    main(["upload"] + sys.argv[1:])

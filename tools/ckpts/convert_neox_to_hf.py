#!/usr/bin/env python
"""NeoX checkpoint -> Hugging Face (GPT-NeoX / Llama / Mistral).

Forwards its command line to ``python -m gpt_neox_b200.ckpt.convert neox-to-hf`` (reference script: tools/ckpts/convert_neox_to_hf.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.ckpt.convert import main  # noqa: E402

if __name__ == "__main__":
    main(["neox-to-hf"] + sys.argv[1:])

#!/usr/bin/env python
"""Hugging Face Llama / Mistral model -> NeoX checkpoint files.

Forwards its command line to ``python -m gpt_neox_b200.ckpt.convert hf-to-neox`` (reference script: tools/ckpts/convert_hf_llama_to_neox.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.ckpt.convert import main  # noqa: E402

if __name__ == "__main__":
    main(["hf-to-neox"] + sys.argv[1:])

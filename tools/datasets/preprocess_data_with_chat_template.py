#!/usr/bin/env python
"""Tokenise conversations with a Hugging Face chat template.

Forwards its command line to ``python -m gpt_neox_b200.data.preprocess_data --chat-template`` (reference script: tools/datasets/preprocess_data_with_chat_template.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.data.preprocess_data import main  # noqa: E402

if __name__ == "__main__":
    argv = sys.argv[1:]
    main(argv if "--chat-template" in argv else ["--chat-template"] + argv)

#!/usr/bin/env python
"""NeoX Mamba checkpoint -> mamba_ssm parameter names.

Forwards its command line to ``python -m gpt_neox_b200.ckpt.convert neox-to-mamba-ssm`` (reference script: tools/ckpts/convert_neox_to_mamba_ssm.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.ckpt.convert import main  # noqa: E402

if __name__ == "__main__":
    main(["neox-to-mamba-ssm"] + sys.argv[1:])

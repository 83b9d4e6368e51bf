#!/usr/bin/env python
"""Registry of downloadable corpora (import ``DATA_DOWNLOADERS`` / ``prepare_dataset`` from here).

Forwards its command line to ``python -m gpt_neox_b200.data.corpora`` (reference script: tools/datasets/corpora.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.data.corpora import *  # noqa: E402,F401,F403
from gpt_neox_b200.data.corpora import DATA_DOWNLOADERS, prepare_dataset  # noqa: E402,F401

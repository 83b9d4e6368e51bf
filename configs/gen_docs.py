#!/usr/bin/env python
"""Write ``configs/neox_arguments.md`` from the argument schema (``--check``: fail if the file is stale)."""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


def main(argv=None):
    from gpt_neox_b200.config import gen_docs
    argv = sys.argv[1:] if argv is None else argv
    path = os.path.join(HERE, "neox_arguments.md")
    text = gen_docs()
    if "--check" in argv:
        current = open(path).read() if os.path.exists(path) else ""
        if current != text:
            print("configs/neox_arguments.md is stale: run `python configs/gen_docs.py`", file=sys.stderr)
            return 1
        return 0
    with open(path, "w") as f:
        f.write(text)
    print(f"wrote {path}")
    return 0


if __name__ == "__main__":
    sys.exit(main())

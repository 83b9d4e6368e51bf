#!/usr/bin/env python
"""``python deepy.py train.py [-d conf_dir] a.yml b.yml ...``: parse the YAML configs, then start one
process per GPU running the given script (reference: deepy.py:22-37, which delegates to the DeepSpeed
runner; here the launcher is gpt_neox_b200/launcher.py)."""
import logging
import os
import sys


def main(input_args=None):
    logging.basicConfig(level=os.environ.get("LOGLEVEL", "INFO"))
    from gpt_neox_b200 import launcher
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.utils.common import get_wandb_api_key

    neox_args = NeoXArgs.consume_deepy_args(input_args)
    main_args = neox_args.get_deepspeed_main_args()
    token = get_wandb_api_key(neox_args=neox_args)
    if token is not None:
        os.environ["WANDB_API_KEY"] = token
    return launcher.main(main_args)


if __name__ == "__main__":
    sys.exit(main())

#!/usr/bin/env python
"""Per-rank training entry (reference: train.py:23-31)."""
from gpt_neox_b200.config import NeoXArgs
from gpt_neox_b200.training import pretrain


def main(input_args=None, overwrite_values=None):
    neox_args = NeoXArgs.consume_neox_args(input_args=input_args, overwrite_values=overwrite_values)
    neox_args.configure_distributed_args()
    neox_args.build_tokenizer()
    neox_args.initialize_tensorboard_writer()
    neox_args.initialize_comet()
    pretrain(neox_args=neox_args)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Per-rank text-generation entry (reference: generate.py:30-93): ``text_gen_type`` selects
unconditional / input-file / interactive / precompute."""
from gpt_neox_b200.text_generation_utils import (generate_samples_input_from_file, generate_samples_interactive,
                                                 generate_samples_unconditional, precompute_logits)
from gpt_neox_b200.utils.common import print_rank_0, setup_for_inference_or_eval


def main(input_args=None, overwrite_values=None):
    model, neox_args = setup_for_inference_or_eval(use_cache=True, input_args=input_args,
                                                   overwrite_values=overwrite_values)
    if neox_args.recompute:
        model.module.inference_mode(use_cache=False)
    kw = dict(neox_args=neox_args, model=model, recompute=neox_args.recompute, temperature=neox_args.temperature,
              top_k=neox_args.top_k, top_p=neox_args.top_p)
    if neox_args.text_gen_type == "unconditional":
        print_rank_0(f"Generating samples unconditionally and saving results to {neox_args.sample_output_file}")
        generate_samples_unconditional(number_of_samples=neox_args.num_samples,
                                       output_file=neox_args.sample_output_file,
                                       maximum_tokens=neox_args.maximum_tokens, **kw)
    elif neox_args.text_gen_type == "input-file":
        print_rank_0(f"Generating samples from input file {neox_args.sample_input_file}")
        assert neox_args.sample_input_file is not None
        generate_samples_input_from_file(input_file=neox_args.sample_input_file,
                                         output_file=neox_args.sample_output_file,
                                         maximum_tokens=neox_args.maximum_tokens,
                                         prompt_end=neox_args.prompt_end, **kw)
    elif neox_args.text_gen_type == "interactive":
        generate_samples_interactive(maximum_tokens=neox_args.maximum_tokens, prompt_end=neox_args.prompt_end, **kw)
    elif neox_args.text_gen_type == "precompute":
        precompute_logits(neox_args=neox_args, model=model)
    else:
        raise ValueError(f"`text_gen_type` either not specified or not recognised: {neox_args.text_gen_type}")


if __name__ == "__main__":
    main()

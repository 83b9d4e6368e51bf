#!/usr/bin/env python
"""Per-rank evaluation entry (reference: eval.py:34-75): runs the evaluation-harness tasks named by
``eval_tasks`` and writes the results as JSON."""
import json
import os
from datetime import datetime

from gpt_neox_b200.eval_tasks import run_eval_harness
from gpt_neox_b200.training import forward_step
from gpt_neox_b200.utils.common import init_wandb, print_rank_0, setup_for_inference_or_eval


def main(input_args=None, overwrite_values=None):
    model, neox_args = setup_for_inference_or_eval(use_cache=False, input_args=input_args,
                                                   overwrite_values=overwrite_values)
    results = run_eval_harness(model, forward_step, neox_args, eval_tasks=neox_args.eval_tasks,
                               bootstrap_iters=10000)
    if neox_args.rank == 0:
        init_wandb(neox_args=neox_args)
        print_rank_0(json.dumps(results.get("results", results), indent=4, default=str))
        path = neox_args.eval_results_prefix or ""
        if os.path.isdir(path):
            path = os.path.join(path, "eval_results")
        path = f"{path or 'eval_results'}_eval_results_{datetime.now().strftime('%m-%d-%Y-%H-%M-%S')}.json"
        with open(path, "w") as f:
            json.dump(results, f, indent=4, default=str)


if __name__ == "__main__":
    main()

from .eval_adapter import EvalHarnessAdapter, run_eval_harness

__all__ = ["EvalHarnessAdapter", "run_eval_harness"]

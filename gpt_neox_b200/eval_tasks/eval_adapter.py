"""Adapter between a trained model and the LM Evaluation Harness request types
(eval_tasks/eval_adapter.py:36-560): ``loglikelihood``, ``loglikelihood_rolling`` and ``generate_until``.

The scoring core has no dependency on the harness package: requests are plain ``(context, continuation)``
pairs (or objects with ``.args``), so it is usable (and tested) stand-alone; ``run_eval`` hands the adapter
to ``lm_eval.evaluator`` when that package is importable.

Data parallelism: a batch of requests is padded to a multiple of the data-parallel size, each rank scores
its slice, and the per-request results (two numbers each) are all-gathered — not the ``[b, s, vocab]``
logits the reference gathers (eval_adapter.py:349-359).
"""
from __future__ import annotations

import copy
from functools import partial
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

from .. import parallel as mpu
from ..text_generation_utils import forward_model, generate_samples_from_prompt


def _args_of(req):
    return req.args if hasattr(req, "args") else req


def _chunks(seq, n):
    for i in range(0, len(seq), n):
        yield seq[i:i + n]


class EvalHarnessAdapter:
    def __init__(self, model, forward_step_fn, neox_args, batch_size=None):
        self._model = model
        self.neox_args = neox_args
        self.tokenizer = neox_args.tokenizer
        self._device = torch.device("cuda", neox_args.local_rank or 0) if torch.cuda.is_available() \
            else torch.device("cpu")
        self._eot_token_id = getattr(neox_args.tokenizer, "eod_id", None) or neox_args.tokenizer.eod
        self._max_length = neox_args.max_position_embeddings
        self._max_gen_toks = 128
        self._vocab_size = neox_args.padded_vocab_size
        self.is_main = (neox_args.rank or 0) == 0
        self.is_pipe_parallel = bool(neox_args.is_pipe_parallel)
        self.is_last_stage = True if not self.is_pipe_parallel else model.is_last_stage()
        self.dp_world_size = mpu.get_data_parallel_world_size()
        self.dp_rank = mpu.get_data_parallel_rank()
        self.dp_group = mpu.get_data_parallel_group()
        self.is_data_parallel = self.dp_world_size > 1
        self.is_mp_rank_0 = mpu.get_model_parallel_rank() == 0
        self._batch_size = batch_size or (neox_args.batch_size or 1) * self.dp_world_size
        if not hasattr(self.tokenizer, "encode"):
            self.tokenizer.encode = self.tokenizer.tokenize
        if not hasattr(self.tokenizer, "decode"):
            self.tokenizer.decode = self.tokenizer.detokenize
        self._forward_step_fn = partial(forward_step_fn, neox_args=neox_args, timers=None, return_logits=True) \
            if forward_step_fn is not None else None
        self.generate = partial(generate_samples_from_prompt, neox_args=neox_args, model=model)
        self.cache_hook = None

    # ------------------------------------------------------------------ harness properties
    vocab_size = property(lambda self: self._vocab_size)
    eot_token_id = property(lambda self: self._eot_token_id)
    max_length = property(lambda self: self._max_length)
    max_gen_toks = property(lambda self: self._max_gen_toks)
    batch_size = property(lambda self: self._batch_size)
    device = property(lambda self: self._device)
    model = property(lambda self: self._model)
    rank = property(lambda self: 0)
    world_size = property(lambda self: 1)

    def tok_encode(self, string: str, **kwargs):
        return self.tokenizer.encode(string)

    def tok_decode(self, tokens, **kwargs):
        return self.tokenizer.decode(tokens)

    def _module(self):
        return self._model.module if hasattr(self._model, "module") else self._model

    # ------------------------------------------------------------------ request front ends
    def loglikelihood(self, requests) -> List[Tuple[float, bool]]:
        enc = []
        for req in requests:
            context, continuation = _args_of(req)[:2]
            ctx = [self.eot_token_id] if context == "" else self.tok_encode(context)
            enc.append(((context, continuation), ctx, self.tok_encode(continuation)))
        return self._loglikelihood_tokens(enc)

    def loglikelihood_rolling(self, requests) -> List[float]:
        """Full-document log-likelihood with non-overlapping windows of ``max_length`` tokens; every window
        is conditioned on the EOT token or on the last token of the previous window."""
        out = []
        for req in requests:
            (text,) = _args_of(req)[:1]
            toks = self.tok_encode(text)
            windows, prev = [], self.eot_token_id
            for lo in range(0, len(toks), self.max_length):
                piece = toks[lo:lo + self.max_length]
                windows.append((None, [prev], piece))
                prev = piece[-1]
            out.append(sum(ll for ll, _ in self._loglikelihood_tokens(windows, disable_tqdm=True)))
        return out

    def generate_until(self, requests) -> List[str]:
        self._module().inference_mode(use_cache=True)
        order = sorted(range(len(requests)), key=lambda i: len(self.tok_encode(_args_of(requests[i])[0])))
        res = [None] * len(requests)
        for i in order:
            context, gen_kwargs = _args_of(requests[i])[:2]
            if not isinstance(gen_kwargs, dict):
                raise ValueError(f"Expected `kwargs` to be of type `dict` but got {gen_kwargs}")
            kwargs = copy.deepcopy(gen_kwargs)
            until = kwargs.pop("until", None)
            if isinstance(until, str):
                until = [until]
            elif until is not None and not isinstance(until, list):
                raise ValueError(f"Expected `kwargs['until']` to be of type Union[str,list] but got {until}")
            if not until:
                until = [self.tok_decode([self.eot_token_id])]
            max_gen = kwargs.pop("max_gen_toks", self.max_gen_toks)
            kwargs.pop("do_sample", None)
            self._module().clear_cache()
            cont = self.generate(text=context, stop_tokens=[self.tok_encode(u) for u in until],
                                 recompute=self.neox_args.recompute, maximum_tokens=max_gen,
                                 **{k: v for k, v in kwargs.items() if k in ("temperature", "top_k", "top_p")})
            s = (cont[0]["text"] or "") if cont else ""
            for term in until:
                s = s.split(term)[0]
            res[i] = s
        self._module().train_mode()
        return res

    # ------------------------------------------------------------------ scoring core
    def _loglikelihood_tokens(self, requests, disable_tqdm=False):
        """requests: (cache_key, context tokens, continuation tokens) -> [(sum log p, greedy-match)]."""
        self._module().inference_mode(use_cache=False)
        order = sorted(range(len(requests)), key=lambda i: -(len(requests[i][1]) + len(requests[i][2])))
        res = [None] * len(requests)
        with torch.no_grad():
            for chunk in _chunks(order, self.batch_size):
                rows, inplens = [], []
                for i in chunk:
                    _, ctx, cont = requests[i]
                    inp = (list(ctx) + list(cont))[-(self.max_length + 1):][:-1]
                    rows.append(inp)
                    inplens.append(len(inp))
                width = max(inplens)
                batch = torch.zeros(len(rows), width, dtype=torch.long)
                for r, inp in enumerate(rows):
                    batch[r, :len(inp)] = torch.tensor(inp, dtype=torch.long)
                conts = [requests[i][2] for i in chunk]
                scores = self._score_batch(batch.to(self.device), inplens, conts)
                for i, sc in zip(chunk, scores):
                    res[i] = sc
        self._module().train_mode()
        return res

    def _score_batch(self, batch, inplens, conts):
        """Each data-parallel rank scores a slice of the batch; the (log-likelihood, match) pairs are gathered."""
        n = batch.shape[0]
        local, pad = self._dp_scatter(batch)
        lo = self.dp_rank * local.shape[0]
        logits = self._model_call(local)
        out = torch.zeros(local.shape[0], 2, dtype=torch.float32, device=self.device)
        if logits is not None:
            lp = F.log_softmax(logits.float(), dim=-1)
            for r in range(local.shape[0]):
                g = lo + r
                if g >= n:
                    continue
                cont = torch.tensor(conts[g][-inplens[g]:], dtype=torch.long, device=lp.device)
                sl = lp[r, inplens[g] - len(cont): inplens[g]]
                out[r, 0] = sl.gather(1, cont[:, None]).sum()
                out[r, 1] = float(bool((sl.argmax(-1) == cont).all()))
        if self.is_pipe_parallel and torch.distributed.is_initialized():
            src = self._model.grid.stage_to_global(self._model.num_stages - 1)
            torch.distributed.broadcast(out, src, group=mpu.get_pipe_parallel_group())
        out = self._dp_gather(out)[:n]
        return [(float(a), bool(b > 0.5)) for a, b in out.cpu().tolist()]

    def _dp_scatter(self, inps):
        """Pad the batch to a multiple of the data-parallel size and return this rank's rows."""
        n = inps.shape[0]
        per = -(-n // self.dp_world_size)
        pad = per * self.dp_world_size - n
        if pad:
            inps = torch.cat([inps, inps.new_zeros(pad, inps.shape[1])], dim=0)
        return inps[self.dp_rank * per:(self.dp_rank + 1) * per].contiguous(), pad

    def _dp_gather(self, x):
        if not self.is_data_parallel:
            return x
        parts = [torch.empty_like(x) for _ in range(self.dp_world_size)]
        torch.distributed.all_gather(parts, x.contiguous(), group=self.dp_group)
        return torch.cat(parts, dim=0)

    def _model_call(self, inps) -> Optional[torch.Tensor]:
        """tokens [b, s] -> logits [b, s, vocab] (None off the last pipeline stage)."""
        b, s = inps.shape
        pos = torch.arange(s, device=inps.device)[None].expand(b, -1)
        from ..utils.common import get_attn_mask
        needs_mask = any(t not in ("flash",) for t in (self.neox_args.attention_config or ["global"]))
        mask = get_attn_mask(s, inps.device, self.neox_args.sliding_window_width) if needs_mask else None
        return forward_model(self._model, (inps, pos, mask), self.is_pipe_parallel,
                             full_vocab=self.neox_args.padded_vocab_size)

    # ------------------------------------------------------------------ harness driver
    def run_eval(self, eval_tasks=None, num_fewshot=0, bootstrap_iters=2, use_cache=False, name="neox", limit=None):
        """Tasks that name local ``.jsonl`` files (eval_tasks/local_tasks.py) are evaluated in-tree, with no further
        package and no network; every other task goes to ``lm_eval.evaluator`` as in the reference."""
        from . import local_tasks
        eval_tasks = eval_tasks or ["lambada_openai", "piqa", "hellaswag", "winogrande", "mathqa", "pubmedqa",
                                    "triviaqa"]
        local = [t for t in eval_tasks if local_tasks.resolve(t) is not None]
        remote = [t for t in eval_tasks if t not in local]
        if remote:
            try:
                from lm_eval import evaluator, tasks        # noqa: F401
            except ImportError as e:
                raise ImportError(f"tasks {remote} need the `lm_eval` package (LM Evaluation Harness); tasks stored as "
                                  "local .jsonl files (NEOX_EVAL_TASK_DIR) run without it") from e
        was_training = self._module().training
        self._module().eval()
        results = {"results": {}, "versions": {}, "config": {}}
        try:
            if remote:
                results = evaluator.simple_evaluate(model=self, tasks=remote, num_fewshot=num_fewshot, limit=limit,
                                                    bootstrap_iters=bootstrap_iters)
            if local:
                mine = local_tasks.evaluate(self, local, num_fewshot=num_fewshot, limit=limit)
                results["results"].update(mine["results"])
                results.setdefault("versions", {}).update(mine["versions"])
                results.setdefault("config", {}).update(mine["config"])
        finally:
            if was_training:
                self._module().train()
        return results


def run_eval_harness(model, forward_step_fn, neox_args, batch_size=None, eval_tasks=None, num_fewshot=0,
                     bootstrap_iters=2):
    print("Running evaluation harness...", flush=True)
    adapter = EvalHarnessAdapter(model, forward_step_fn, neox_args, batch_size)
    return adapter.run_eval(eval_tasks=eval_tasks, num_fewshot=num_fewshot, bootstrap_iters=bootstrap_iters)

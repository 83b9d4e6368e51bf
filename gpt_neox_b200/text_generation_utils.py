"""Autoregressive generation: greedy / temperature / top-k / top-p sampling with a KV cache, batched
prompts of unequal length, stop sequences, and the file / unconditional / interactive drivers
(megatron/text_generation_utils.py:38-980).

The decode loop keeps every per-step decision on the device (sampling, "has this row started / finished",
token substitution); the host only reads one flag per step to know when all rows are done.
"""
from __future__ import annotations

import copy
import json
import os
import time
from typing import List, Optional, Union

import torch
import torch.nn.functional as F

from . import parallel as mpu
from .utils.common import get_ltor_masks_and_position_ids, is_mp_rank_0, print_rank_0


def _device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def get_batch(neox_args, context_tokens: torch.Tensor):
    """tokens [b, s] -> (tokens, attention_mask, position_ids)."""
    tokens = context_tokens.contiguous().to(_device())
    attention_mask, _, position_ids = get_ltor_masks_and_position_ids(
        data=tokens, eod_token=neox_args.tokenizer.eod, eod_mask_loss=neox_args.eod_mask_loss)
    return tokens, attention_mask, position_ids


def pad_batch(context_tokens: List[List[int]], pad_id: int, pad_len: int, truncate: bool = False):
    """Right-pad every prompt to ``pad_len`` (in place); returns (padded prompts, original lengths).
    Prompts longer than ``pad_len`` are an error unless ``truncate`` keeps their last ``pad_len`` tokens."""
    lengths = []
    for i, toks in enumerate(context_tokens):
        n = len(toks)
        if n > pad_len:
            if not truncate:
                raise ValueError("context_length is bigger than to be padded length")
            toks = context_tokens[i] = toks[-pad_len:]
            n = pad_len
        toks.extend([pad_id] * (pad_len - n))
        lengths.append(n)
    return context_tokens, lengths


def filter_logits(logits, top_k=0, top_p=0.0, filter_value=-float("Inf")):
    """Top-k then nucleus filtering of ``[batch, vocab]`` logits (in place, vectorised over the batch)."""
    if top_k > 0:
        kth = torch.topk(logits, top_k)[0][..., -1, None]
        logits.masked_fill_(logits < kth, filter_value)
    if top_p > 0.0:
        sorted_logits, sorted_idx = torch.sort(logits, descending=True, dim=-1)
        cum = torch.cumsum(F.softmax(sorted_logits, dim=-1), dim=-1)
        drop_sorted = cum > top_p
        drop_sorted[..., 1:] = drop_sorted[..., :-1].clone()      # keep the first token crossing the threshold
        drop_sorted[..., 0] = False
        drop = torch.zeros_like(drop_sorted).scatter_(-1, sorted_idx, drop_sorted)
        logits.masked_fill_(drop, filter_value)
    return logits


def switch(val1, val2, boolean):
    """Elements of ``val2`` where ``boolean`` else ``val1``."""
    return torch.where(boolean.bool(), val2.type_as(val1), val1)


def forward_model(model, model_inputs, is_pipe_parallel=False, pipe_parallel_size=0,
                  full_vocab: Optional[int] = None) -> Optional[torch.Tensor]:
    """Logits ``[b, s, vocab]`` gathered over the tensor-parallel group; with pipeline parallelism only the
    last stage returns them (None elsewhere)."""
    if is_pipe_parallel and hasattr(model, "eval_batch"):
        tokens = model_inputs[0]
        # the pipeline engine wants (inputs, labels); labels are unused when logits are returned
        it = iter([{"text": F.pad(tokens, pad=(0, 1))}])
        micro_batches_before = model.micro_batches
        model.micro_batches = 1
        try:
            _, logits = model.eval_batch(it, return_logits=True)
        finally:
            model.micro_batches = micro_batches_before
    else:
        logits = model(model_inputs)
    if logits is None:
        return None
    ws = mpu.get_model_parallel_world_size()
    if ws > 1 and full_vocab is not None and logits.shape[-1] * ws == full_vocab:
        logits = mpu.gather_from_model_parallel_region(logits)       # vocab-parallel head: assemble the rows
    return logits


def broadcast_terminate_signal(terminate_runs: int):
    """Rank 0 of the tensor-parallel group tells the others whether to stop."""
    t = torch.tensor([terminate_runs], dtype=torch.long, device=_device())
    if torch.distributed.is_initialized() and mpu.get_model_parallel_world_size() > 1:
        torch.distributed.broadcast(t, mpu.get_model_parallel_src_rank(), group=mpu.get_model_parallel_group())
    return int(t[0].item())


def stop_tokens_in_completion(stop_tokens, context_tokens, batch_index, current_index):
    """True when the tokens ending at ``current_index`` of row ``batch_index`` equal one stop sequence."""
    if stop_tokens is None:
        return False
    row = context_tokens[batch_index]
    for seq in stop_tokens:
        n = len(seq)
        if n and current_index + 1 >= n and bool((row[current_index + 1 - n: current_index + 1] == seq).all()):
            return True
    return False


def _sample(logits, temperature, top_k, top_p):
    if temperature == 0.0 and top_k == 0 and top_p == 0.0:
        return torch.argmax(logits, dim=-1).view(-1), logits
    logits = logits.float()
    if temperature > 0.0:
        logits = logits / temperature
    logits = filter_logits(logits, top_k=top_k, top_p=top_p)
    return torch.multinomial(F.softmax(logits, dim=-1), num_samples=1).view(-1), logits


def stream_tokens(neox_args, model, context_tokens: List[List[int]], eos_token_id: int = None,
                  maximum_tokens: int = None, recompute: bool = False, temperature: float = 0.0, top_k: int = 0,
                  top_p: float = 0.0, stop_tokens=None):
    """Generator over decode steps.  Yields ``(tokens [b, seq], start_index [b], end_index [b], logits,
    is_done [b])`` after every generated position; rows whose prompt is longer than the current position
    keep their prompt token there (generation starts at the shortest prompt's end)."""
    model.eval()
    dev = _device()
    ctx, lengths = pad_batch(copy.deepcopy(context_tokens), pad_id=neox_args.tokenizer.eod,
                             pad_len=neox_args.seq_length)
    tokens = torch.tensor(ctx, dtype=torch.long, device=dev)
    start_index = torch.tensor(lengths, dtype=torch.long, device=dev)
    if stop_tokens:
        if not isinstance(stop_tokens[0], (list, tuple)):
            stop_tokens = [stop_tokens]
        stop_tokens = [torch.tensor(s, dtype=torch.long, device=dev) for s in stop_tokens]
    if torch.distributed.is_initialized() and mpu.get_model_parallel_world_size() > 1:
        src, grp = mpu.get_model_parallel_src_rank(), mpu.get_model_parallel_group()
        torch.distributed.broadcast(tokens, src, group=grp)
        torch.distributed.broadcast(start_index, src, group=grp)
    tokens, attention_mask, position_ids = get_batch(neox_args, tokens)
    eos_token_id = eos_token_id or neox_args.tokenizer.eod
    maximum_tokens = maximum_tokens or (neox_args.seq_length - int(start_index.max().item()) - 1)
    bsz = tokens.size(0)
    pos = first = int(start_index.min().item())
    last = min(neox_args.seq_length - 1, pos + maximum_tokens - 1)
    pipe = bool(neox_args.is_pipe_parallel)
    if any(k in ("mamba", "rwkv") for k in (neox_args.attention_config or [])):
        # the recurrent blocks keep no state between calls: every step runs the whole prefix
        recompute = True
    if pipe and mpu.get_pipe_parallel_world_size() > 1:
        # the pipeline engine derives positions and masks from the tokens it is given and fixes the shape of the
        # activations between stages on first use: a one-token cached step does not fit, so the prefix is re-run
        recompute = True
    if recompute:
        # whoever switched the layers to cached decoding (generate.py does, by default) must not make a
        # recomputing loop append the whole prefix to the cache at every step
        net = getattr(model, "module", model)
        if hasattr(net, "inference_mode"):
            net.inference_mode(use_cache=False)
        if hasattr(net, "clear_cache"):
            net.clear_cache()
    with torch.no_grad():
        done = torch.zeros(bsz, dtype=torch.bool, device=dev)
        end_index = torch.full((bsz,), -1, dtype=torch.long, device=dev)
        gen_logits = torch.empty(maximum_tokens, neox_args.padded_vocab_size, dtype=torch.float32, device=dev) \
            if neox_args.return_logits else None
        while pos <= last:
            if recompute:
                logits = forward_model(model, (tokens, position_ids, attention_mask), pipe,
                                       full_vocab=neox_args.padded_vocab_size)
                step_logits = logits[:, pos - 1, :] if logits is not None else None
            else:
                sl = slice(0, pos) if pos == first else slice(pos - 1, pos)
                logits = forward_model(model, (tokens[:, sl].contiguous(), position_ids[:, sl].contiguous(),
                                               attention_mask), pipe, full_vocab=neox_args.padded_vocab_size)
                step_logits = logits[:, -1].reshape(bsz, -1) if logits is not None else None
            if step_logits is not None:
                new, used = _sample(step_logits, temperature, top_k, top_p)
                if gen_logits is not None:
                    gen_logits[pos - first] = used[0]
            else:
                new = torch.zeros(bsz, dtype=torch.long, device=dev)
            if pipe and torch.distributed.is_initialized() and mpu.get_pipe_parallel_world_size() > 1:
                torch.distributed.broadcast(new, model.grid.stage_to_global(model.num_stages - 1),
                                            group=mpu.get_pipe_parallel_group())
            started = start_index <= pos
            tokens[:, pos] = switch(tokens[:, pos], new, started)
            hit_eos = (new == eos_token_id) & started
            done = done | hit_eos
            if stop_tokens:
                hits = [stop_tokens_in_completion(stop_tokens, tokens, b, pos) for b in range(bsz)]
                done = done | torch.tensor(hits, dtype=torch.bool, device=dev)
            end_index[started & ~done] = pos
            pos += 1
            yield tokens, start_index, end_index, gen_logits, done
            if bool(done.all()):
                break


def generate_samples_from_prompt(neox_args, model, text: Union[List[str], str], eos_token_id: int = None,
                                 maximum_tokens: int = 64, prompt_end: str = "\n", recompute: bool = False,
                                 temperature: float = 0.0, top_k: int = 0, top_p: float = 0.0, stop_tokens=None):
    """One completion per prompt; returns a list of dicts with ``context, text, length, finished, message,
    duration_seconds`` (and ``logits`` when ``return_logits``)."""
    eos_token_id = eos_token_id or neox_args.tokenizer.eod
    prompts = [text] if isinstance(text, str) else list(text)
    results = []
    todo = iter(prompts)
    while True:
        t0 = time.time()
        raw = next(todo, None)
        terminate = 1 if raw is None else 0
        if raw is not None:
            ctx = [eos_token_id] if raw == "" else neox_args.tokenizer.tokenize(raw)
            if len(ctx) >= neox_args.seq_length // 2:
                print_rank_0("\nWarning! Context length", len(ctx),
                             "\nPlease give smaller context (e.g. half of the max sequence length)!")
        if not is_mp_rank_0():
            ctx = neox_args.tokenizer.tokenize("EMPTY TEXT")
            terminate = 0
        if broadcast_terminate_signal(terminate) == 1:
            return results
        state = None
        for state in stream_tokens(neox_args=neox_args, model=model, context_tokens=[ctx],
                                   eos_token_id=eos_token_id, maximum_tokens=maximum_tokens, recompute=recompute,
                                   temperature=temperature, top_k=top_k, top_p=top_p, stop_tokens=stop_tokens):
            pass
        toks, starts, ends, logits, dones = state
        for row, s, e, d in zip(toks.cpu().tolist(), starts.cpu().tolist(), ends.cpu().tolist(),
                                dones.cpu().tolist()):
            message, out_text, gen = None, None, []
            if e >= s:
                gen = row[s:e + 1]
                try:
                    out_text = neox_args.tokenizer.detokenize(gen)
                except KeyError:
                    message = "WARNING: generated token which doesn't exist."
            else:
                message = "WARNING: text generation did not start; try different batching or adjust parameters"
            if is_mp_rank_0():
                rec = {"context": raw, "text": out_text, "length": len(gen), "finished": d, "message": message,
                       "duration_seconds": float(time.time() - t0)}
                if neox_args.return_logits and logits is not None:
                    rec["logits"] = logits.cpu().numpy().tolist()
                results.append(rec)
    return results


def generate_samples_input_from_file(neox_args, model, input_file, output_file=None, eos_token_id: int = None,
                                     maximum_tokens: int = 64, prompt_end: str = "\n", recompute: bool = False,
                                     temperature: float = 0.0, top_k: int = 0, top_p: float = 0.0):
    """Prompts separated by ``prompt_end`` in ``input_file``; completions written as JSON lines."""
    print_rank_0(f"generate_samples_input_from_file() loading input from {input_file}")
    with open(input_file, "r", encoding="utf-8") as f:
        prompts = [p.strip() for p in f.read().split(prompt_end)]
    prompts = [p for p in prompts if p]
    print_rank_0(f"generate_samples_input_from_file() prompts loaded: {len(prompts)}")
    if is_mp_rank_0() and output_file is None:
        output_file = str(input_file) + ".output.jsonl"
        print_rank_0(f"generate_samples_input_from_file() setting default output file to {output_file}")
    print_rank_0("generate_samples_input_from_file() generating...")
    out = generate_samples_from_prompt(neox_args=neox_args, model=model, text=prompts, eos_token_id=eos_token_id,
                                       maximum_tokens=maximum_tokens, prompt_end=prompt_end, recompute=recompute,
                                       temperature=temperature, top_k=top_k, top_p=top_p)
    if is_mp_rank_0():
        with open(output_file, "w") as f:
            for item in out:
                f.write(json.dumps(item) + "\n")
    print_rank_0("generate_samples_input_from_file() done")
    return out


def generate_samples_unconditional(neox_args, model, number_of_samples: int = 10, output_file=None,
                                   eos_token_id: int = None, maximum_tokens: int = 64, recompute: bool = False,
                                   temperature: float = 0.0, top_k: int = 0, top_p: float = 0.0):
    """``number_of_samples`` completions of the empty prompt."""
    print_rank_0("generate_samples_unconditional() generating...")
    assert number_of_samples > 0, "number_of_samples must be > 0"
    out = generate_samples_from_prompt(neox_args=neox_args, model=model, text=[""] * number_of_samples,
                                       eos_token_id=eos_token_id, maximum_tokens=maximum_tokens,
                                       recompute=recompute, temperature=temperature, top_k=top_k, top_p=top_p)
    if is_mp_rank_0() and output_file is not None:
        with open(output_file, "w") as f:
            for item in out:
                f.write(json.dumps(item) + "\n")
    print_rank_0("generate_samples_unconditional() done")
    return out


def generate_samples_interactive(neox_args, model, maximum_tokens: int = 64, prompt_end: str = "\n",
                                 eos_token_id: int = None, recompute: bool = False, temperature: float = 0.0,
                                 top_k: int = 0, top_p: float = 0.0):
    """Prompt on stdin (rank 0), stream the completion to stdout; an empty answer to 'continue' exits."""
    while True:
        model.module.clear_cache() if hasattr(model, "module") else None
        terminate = 0
        if torch.distributed.is_initialized() and torch.distributed.get_rank() != 0:
            ctx = neox_args.tokenizer.tokenize("EMPTY TEXT")
            raw = ""
        else:
            os.system("clear")
            raw, line = "", input("Context prompt >>> ")
            while not line.endswith(prompt_end.strip()) and prompt_end.strip():
                raw += line + "\n"
                line = input()
                if line == "":
                    break
            raw += line
            ctx = neox_args.tokenizer.tokenize(raw) if raw else [neox_args.tokenizer.eod]
            if len(ctx) >= neox_args.seq_length // 2:
                print_rank_0("\nWarning! Context length", len(ctx), "\nPlease give smaller context!")
        if broadcast_terminate_signal(terminate) == 1:
            return
        shown = ""
        for toks, starts, ends, _logits, _done in stream_tokens(
                neox_args=neox_args, model=model, context_tokens=[ctx], eos_token_id=eos_token_id,
                maximum_tokens=maximum_tokens, recompute=recompute, temperature=temperature, top_k=top_k,
                top_p=top_p):
            if mpu.get_model_parallel_rank() == 0:
                gen = toks[0].cpu().tolist()[int(starts[0]): int(ends[0]) + 1]
                text = neox_args.tokenizer.detokenize(gen)
                print_rank_0(text[len(shown):], end="", flush=True)
                shown = text
        print_rank_0()
        if torch.distributed.is_initialized():
            torch.distributed.barrier(group=mpu.get_model_parallel_group())
        if not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0:
            if input("Generation finished. Continue? (y / anything else to stop) ").strip().lower() != "y":
                terminate = 1
        if broadcast_terminate_signal(terminate) == 1:
            return


def get_logp(logits, labels, force_fp32=False):
    """Per-token log-probability of ``labels`` under (possibly vocab-parallel) ``logits``."""
    if force_fp32:
        logits = logits.float()
    return -mpu.vocab_parallel_cross_entropy(logits.contiguous(), labels)


def precompute_logits(neox_args, model):
    """Walk the training set once with the frozen model and store, per sample, the reference log-probs (or
    top-k logits) the preference-learning losses need (DPO / KTO reference pass)."""
    import numpy as np
    from .training import get_batch as train_get_batch
    from .data.data_utils import build_train_valid_test_data_loaders
    if neox_args.precompute_model_name is None:
        mdl = str(neox_args.load).rstrip("/").split("/")[-1]
    else:
        mdl = neox_args.precompute_model_name
    print_rank_0("precompute_logits() generating...")
    model.eval()
    loader, _, _ = build_train_valid_test_data_loaders(neox_args)
    it = iter(loader) if loader is not None else None
    out_dir = neox_args.save or "."
    os.makedirs(out_dir, exist_ok=True)
    rows = []
    with torch.no_grad():
        for _ in range(neox_args.train_iters or 0):
            tokens, labels, _mask, attention_mask, position_ids = train_get_batch(neox_args, it)
            logits = forward_model(model, (tokens, position_ids, attention_mask), neox_args.is_pipe_parallel)
            if logits is None:
                continue
            lp = torch.log_softmax(logits.float(), dim=-1)
            rows.append(torch.gather(lp, 2, labels.unsqueeze(-1)).squeeze(-1).cpu().numpy())
    if is_mp_rank_0() and rows:
        np.save(os.path.join(out_dir, f"{mdl}_ref_logp_rank{mpu.get_data_parallel_rank()}.npy"),
                np.concatenate(rows, axis=0))
    print_rank_0("precompute_logits() done")

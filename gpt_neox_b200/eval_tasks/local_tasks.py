"""Offline evaluation tasks for the harness adapter.

The reference evaluates through the ``lm_eval`` package, which downloads its task data
(eval_tasks/eval_adapter.py:388-520).  On a machine without that package or without network the same three
request types still have to run end to end, so this module evaluates tasks stored as local ``.jsonl`` files
through the adapter's ``loglikelihood`` / ``loglikelihood_rolling`` and returns a result dictionary of the
harness's shape (``{"results": {task: {metric: value}}, "versions": ..., "config": ...}``).

One JSON object per line; the task type is taken from the keys of the first record:

* ``{"query": ..., "choices": [...], "gold": i}``  multiple choice (PIQA / HellaSwag / ARC style):
  ``acc`` picks the continuation with the highest log-likelihood, ``acc_norm`` the highest log-likelihood per byte;
* ``{"text": ...}``  LAMBADA style: the last word is the continuation; ``ppl`` and ``acc`` (greedy match);
* ``{"document": ...}``  rolling perplexity (WikiText style): ``word_perplexity``, ``byte_perplexity``, ``bits_per_byte``.

A task is named by its file path, or by a bare name resolved to ``<dir>/<name>.jsonl`` with ``dir`` taken from the
``NEOX_EVAL_TASK_DIR`` environment variable.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional


def resolve(task: str) -> Optional[str]:
    """Path of the local file behind a task name, or None."""
    if os.path.isfile(task):
        return task
    root = os.environ.get("NEOX_EVAL_TASK_DIR")
    if root:
        for cand in (os.path.join(root, task), os.path.join(root, task + ".jsonl")):
            if os.path.isfile(cand):
                return cand
    return None


def _read(path: str, limit: Optional[int]) -> List[dict]:
    rows = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                rows.append(json.loads(line))
            if limit is not None and len(rows) >= limit:
                break
    if not rows:
        raise ValueError(f"evaluation task file {path} is empty")
    return rows


def _fewshot_prefix(rows: List[dict], n: int) -> str:
    """The first ``n`` records as solved examples (multiple-choice tasks only)."""
    shots = []
    for r in rows[:n]:
        shots.append(r["query"] + r["choices"][int(r["gold"])])
    return "\n\n".join(shots) + ("\n\n" if shots else "")


def _multiple_choice(lm, rows, num_fewshot):
    prefix = _fewshot_prefix(rows, num_fewshot)
    rows = rows[num_fewshot:] if num_fewshot else rows
    reqs, spans = [], []
    for r in rows:
        spans.append((len(reqs), len(r["choices"])))
        reqs += [(prefix + r["query"], c) for c in r["choices"]]
    scores = lm.loglikelihood(reqs)
    acc = acc_norm = 0
    for r, (s0, n) in zip(rows, spans):
        ll = [scores[s0 + i][0] for i in range(n)]
        per_byte = [l / max(1, len(c.encode("utf-8"))) for l, c in zip(ll, r["choices"])]
        gold = int(r["gold"])
        acc += int(max(range(n), key=ll.__getitem__) == gold)
        acc_norm += int(max(range(n), key=per_byte.__getitem__) == gold)
    k = max(1, len(rows))
    return {"acc": acc / k, "acc_norm": acc_norm / k}


def _last_word(lm, rows):
    reqs = []
    for r in rows:
        text = r["text"].rstrip()
        cut = text.rfind(" ")
        reqs.append((text[:cut], text[cut:]) if cut > 0 else ("", text))
    scores = lm.loglikelihood(reqs)
    lls = [s[0] for s in scores]
    return {"ppl": math.exp(-sum(lls) / max(1, len(lls))), "acc": sum(int(s[1]) for s in scores) / max(1, len(scores))}


def _rolling(lm, rows):
    docs = [r["document"] for r in rows]
    lls = lm.loglikelihood_rolling([(d,) for d in docs])
    words = sum(len(d.split()) for d in docs)
    nbytes = sum(len(d.encode("utf-8")) for d in docs)
    total = sum(lls)
    return {"word_perplexity": math.exp(-total / max(1, words)), "byte_perplexity": math.exp(-total / max(1, nbytes)),
            "bits_per_byte": -total / max(1, nbytes) / math.log(2)}


def evaluate(lm, tasks: List[str], num_fewshot: int = 0, limit: Optional[int] = None) -> Dict:
    """Evaluate ``lm`` (an ``EvalHarnessAdapter``) on local task files; raises ``FileNotFoundError`` for a task
    that has no local file."""
    results, versions = {}, {}
    for task in tasks:
        path = resolve(task)
        if path is None:
            raise FileNotFoundError(f"evaluation task {task!r}: no local task file (set NEOX_EVAL_TASK_DIR or pass a path)")
        rows = _read(path, limit)
        name = os.path.splitext(os.path.basename(path))[0]
        first = rows[0]
        if "choices" in first:
            results[name] = _multiple_choice(lm, rows, num_fewshot)
        elif "document" in first:
            results[name] = _rolling(lm, rows)
        elif "text" in first:
            results[name] = _last_word(lm, rows)
        else:
            raise ValueError(f"{path}: records need 'query' + 'choices' + 'gold', 'text' or 'document'")
        versions[name] = 0
    return {"results": results, "versions": versions,
            "config": {"model": "neox", "num_fewshot": num_fewshot, "limit": limit, "task_source": "local files"}}

"""Sampling server for online post-training (REINFORCE-style): feeds `OnlineDataset`
(gpt_neox_b200/data/online_dataset.py) with freshly sampled completions and their rewards.

Counterpart of the reference's example (post-training/online_data_example_llama3.py:1-177), restructured as
a small reusable server:

* one listener per data-parallel rank on ``base_port + dp_rank``; per refill the trainer connects, sends the
  split name, and receives ONE pickled list of ``{"prefix": [ids], "completions": [[ids], ...],
  "rewards": [floats]}`` before the server closes the connection;
* a *prompt source* (JSONL file with a ``text`` / ``prompt`` field, or a built-in toy list), a *sampler*
  (an OpenAI-compatible ``/v1/completions`` endpoint such as a vLLM server, or a toy sampler for dry runs)
  and a *reward function* (a ``transformers`` text-classification pipeline, or completion length for dry
  runs) are plugged in from the command line.

    python post-training/online_data_server.py --dp-size 2 --batch-per-rank 64 --num-completions 4 \\
        --tokenizer meta-llama/Meta-Llama-3-8B-Instruct --endpoint http://localhost:{port}/v1/completions \\
        --endpoint-base-port 8000 --model meta-llama/Meta-Llama-3-8B-Instruct \\
        --prompts data/imdb_prompts.jsonl --reward-pipeline lvwerra/distilbert-imdb --reward-label POSITIVE

    python post-training/online_data_server.py --demo          # no network, no model: toy prompts / sampler / reward

The payload is pickled: run the server only on hosts you control, next to the trainer.
"""
from __future__ import annotations

import argparse
import json
import pickle
import socket
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Callable, Dict, List, Sequence


# ------------------------------------------------------------------------------------------ pluggable parts
class ByteTokenizer:
    """Dry-run tokenizer: UTF-8 bytes (ids 0..255)."""

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))


def load_prompts(path: str | None) -> Dict[str, List[str]]:
    """``{"train": [...], "valid": [...]}`` from a JSONL file (fields ``text`` or ``prompt``, optional ``split``)."""
    if path is None:
        toy = ["The film opens with", "I went in expecting", "Nobody warned me that", "Halfway through the movie",
               "The lead actor", "For a sequel this", "The soundtrack alone", "It is rare that"]
        return {"train": toy, "valid": toy[:4], "test": toy[4:]}
    out: Dict[str, List[str]] = {"train": [], "valid": [], "test": []}
    with open(path) as f:
        for line in f:
            if not line.strip():
                continue
            rec = json.loads(line)
            out.setdefault(rec.get("split", "train"), []).append(rec.get("prompt", rec.get("text", "")))
    for k in ("valid", "test"):
        if not out[k]:
            out[k] = out["train"]
    return out


def http_sampler(url: str, model: str, temperature: float = 1.0, stop: str | None = None, retries: int = 10,
                 wait_s: float = 5.0) -> Callable[[str, int, int], List[str]]:
    """Sampler over an OpenAI-compatible completions endpoint: (prompt, n, max_tokens) -> n completions."""
    import requests

    def sample(prompt: str, n: int, max_tokens: int) -> List[str]:
        body = {"model": model, "prompt": prompt, "n": n, "max_tokens": max_tokens, "temperature": temperature,
                "stream": False}
        if stop:
            body["stop"] = stop
        last = None
        for _ in range(retries):
            try:
                r = requests.post(url, json=body, headers={"User-Agent": "neox-online-data-server"}, timeout=600)
                return [c["text"].strip() for c in r.json()["choices"]]
            except Exception as e:  # noqa: BLE001 - the sampling server may still be starting
                last = e
                time.sleep(wait_s)
        raise RuntimeError(f"sampling endpoint {url} unreachable: {last}")
    return sample


def toy_sampler(prompt: str, n: int, max_tokens: int) -> List[str]:
    """Deterministic dry-run completions of different lengths."""
    words = ["fine", "dull", "bright", "slow", "sharp", "long", "odd", "warm"]
    return [" ".join(words[(len(prompt) + i + j) % len(words)] for j in range(1 + (i % 4)))[:max_tokens] for i in range(n)]


def pipeline_reward(model_name: str, label: str) -> Callable[[Sequence[str]], List[float]]:
    """Reward = probability a ``transformers`` text-classification pipeline assigns to ``label``."""
    from transformers import pipeline
    clf = pipeline("text-classification", model_name, top_k=None, truncation=True, device="cpu")

    def reward(texts: Sequence[str]) -> List[float]:
        return [next(s["score"] for s in scores if s["label"] == label) for scores in clf(list(texts))]
    return reward


def length_reward(texts: Sequence[str]) -> List[float]:
    return [float(len(t.split())) for t in texts]


# ------------------------------------------------------------------------------------------ server
class OnlineDataServer:
    """Serves one data-parallel rank: every accepted connection gets one batch of sampled groups."""

    def __init__(self, dp_rank: int, dp_size: int, prompts: Dict[str, List[str]], tokenizer, sampler, reward_fn,
                 batch_per_rank: int = 64, num_completions: int = 4, max_completion_len: int = 256,
                 prompt_template: str = "{prompt}", eos_text: str = "", host: str = "localhost",
                 base_port: int = 10000, workers: int = 16):
        self.dp_rank, self.dp_size = dp_rank, dp_size
        self.prompts, self.tok, self.sampler, self.reward_fn = prompts, tokenizer, sampler, reward_fn
        self.batch, self.n, self.max_len = batch_per_rank, num_completions, max_completion_len
        self.template, self.eos_text = prompt_template, eos_text
        self.cursor = {k: dp_rank for k in prompts}          # ranks walk disjoint strides of every split
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.sock.bind((host, base_port + dp_rank))
        self.sock.listen(4)
        self.port = self.sock.getsockname()[1]
        self.pool = ThreadPoolExecutor(max_workers=workers)
        self._stop = threading.Event()

    def one_group(self, prompt: str) -> dict:
        text = self.template.format(prompt=prompt)
        prefix_ids = self.tok.encode(text)
        completions = self.sampler(text, self.n, max(1, self.max_len - len(prefix_ids)))
        rewards = self.reward_fn([prompt + " " + c for c in completions])
        return {"prefix": prefix_ids, "completions": [self.tok.encode(c + self.eos_text) for c in completions],
                "rewards": [float(r) for r in rewards]}

    def make_batch(self, split: str) -> List[dict]:
        split = {"valid": "valid", "validation": "valid"}.get(split, split)
        pool = self.prompts.get(split) or self.prompts["train"]
        picks = []
        for _ in range(self.batch):
            picks.append(pool[self.cursor.get(split, self.dp_rank) % len(pool)])
            self.cursor[split] = self.cursor.get(split, self.dp_rank) + self.dp_size
        return list(self.pool.map(self.one_group, picks))

    def serve_once(self):
        conn, _addr = self.sock.accept()
        with conn:
            split = conn.recv(4096).decode() or "train"
            conn.sendall(pickle.dumps(self.make_batch(split)))

    def serve_forever(self):
        self.sock.settimeout(1.0)
        while not self._stop.is_set():
            try:
                self.serve_once()
            except socket.timeout:
                continue

    def close(self):
        self._stop.set()
        self.sock.close()
        self.pool.shutdown(wait=False)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--demo", action="store_true", help="toy prompts / sampler / reward, byte tokenizer")
    ap.add_argument("--dp-size", type=int, default=1)
    ap.add_argument("--base-port", type=int, default=10000)
    ap.add_argument("--batch-per-rank", type=int, default=64)
    ap.add_argument("--num-completions", type=int, default=4)
    ap.add_argument("--max-completion-len", type=int, default=256)
    ap.add_argument("--prompts", type=str, default=None)
    ap.add_argument("--prompt-template", type=str, default="{prompt}")
    ap.add_argument("--eos-text", type=str, default="")
    ap.add_argument("--tokenizer", type=str, default=None, help="Hugging Face tokenizer name or path")
    ap.add_argument("--endpoint", type=str, default=None, help="completions URL; {port} = endpoint-base-port + rank")
    ap.add_argument("--endpoint-base-port", type=int, default=8000)
    ap.add_argument("--model", type=str, default="")
    ap.add_argument("--stop", type=str, default=None)
    ap.add_argument("--reward-pipeline", type=str, default=None)
    ap.add_argument("--reward-label", type=str, default="POSITIVE")
    a = ap.parse_args(argv)
    if a.demo or a.tokenizer is None:
        tok = ByteTokenizer()
    else:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.tokenizer)
    reward = pipeline_reward(a.reward_pipeline, a.reward_label) if a.reward_pipeline else length_reward
    prompts = load_prompts(a.prompts)
    threads = []
    for r in range(a.dp_size):
        sampler = toy_sampler if (a.demo or not a.endpoint) else http_sampler(
            a.endpoint.format(port=a.endpoint_base_port + r), a.model, stop=a.stop)
        srv = OnlineDataServer(r, a.dp_size, prompts, tok, sampler, reward, a.batch_per_rank, a.num_completions,
                               a.max_completion_len, a.prompt_template, a.eos_text, base_port=a.base_port)
        print(f"online data server for dp rank {r} on port {srv.port}", flush=True)
        t = threading.Thread(target=srv.serve_forever, daemon=True)
        t.start()
        threads.append(t)
    for t in threads:
        t.join()


if __name__ == "__main__":
    main()

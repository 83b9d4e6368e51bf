"""Checkpoint conversion between this framework's on-disk layout and Hugging Face / raw-LLaMA / mamba_ssm
state dicts, in both directions, including tensor-parallel merge and split.

    python -m gpt_neox_b200.ckpt.convert neox-to-hf   --input_dir <ckpt/global_stepN> --config_file cfg.yml --output_dir out [--architecture neox|llama|mistral]
    python -m gpt_neox_b200.ckpt.convert hf-to-neox   --hf_dir <dir> --config_file cfg.yml --output_dir out [--tp N]
    python -m gpt_neox_b200.ckpt.convert raw-llama-to-neox --input_dir <dir with consolidated.*.pth> --config_file cfg.yml --output_dir out [--tp N]
    python -m gpt_neox_b200.ckpt.convert merge        --input_dir <ckpt> --output_dir out      (TP shards -> one shard)
    python -m gpt_neox_b200.ckpt.convert neox-to-mamba-ssm --input_dir <ckpt> --config_file cfg.yml --output_dir out
    python -m gpt_neox_b200.ckpt.convert inspect      <file-or-dir>
    python -m gpt_neox_b200.ckpt.convert upload       --hf_dir out --repo_id user/name

Reference tools covered: tools/ckpts/convert_neox_to_hf.py, convert_hf_to_sequential.py,
convert_hf_llama_to_neox.py, convert_raw_llama_weights_to_neox.py, convert_neox_to_mamba_ssm.py, merge20b.py,
inspect_checkpoints.py, upload.py.

Layout facts the rules below encode (per tensor-parallel rank, sequential module numbering: 0 = embedding,
2 .. L+1 = layers, L+3 = final norm, L+4 = LM head):
  * ``attention.query_key_value``: MHA rows are grouped per head ``[q_h; k_h; v_h]``; GQA rows are
    ``[all q heads; all k heads; all v heads]`` of the rank.  Column-parallel: concatenate ranks on dim 0.
  * ``attention.dense.weight`` / ``mlp.linear2.weight``: row-parallel, concatenate on dim 1; their biases are
    replicated parameters that every rank adds before the reduction, so the merged bias is the *sum* over ranks
    and a split divides by the number of ranks.
  * ``mlp.linear1`` of a gated MLP: rows ``[up_rank; gate_rank]`` (first half is the value, second the gate).
  * embeddings / LM head: vocab-parallel, concatenate on dim 0 (padding rows are kept).
"""
from __future__ import annotations

import argparse
import json
import os
import re
from collections import OrderedDict
from typing import Dict, List

import torch
import yaml

# ----------------------------------------------------------------------------------------- merge / split rules
CAT0 = ("attention.query_key_value.weight", "attention.query_key_value.bias", "mlp.linear1.weight",
        "mlp.linear1.bias", "word_embeddings.weight", "final_linear.weight", "mlp.w1", "mlp.w2", "mlp.w3",
        "mixer.in_proj.weight", "mixer.in_proj.bias", "mixer.conv1d.weight", "mixer.conv1d.bias",
        "mixer.dt_proj.weight", "mixer.dt_proj.bias", "mixer.A_log", "mixer.D")
CAT1 = ("attention.dense.weight", "mlp.linear2.weight", "mixer.out_proj.weight", "mixer.x_proj.weight")
SUMMED = ("attention.dense.bias", "mlp.linear2.bias", "mixer.out_proj.bias")


def _rule(name: str) -> str:
    for pat in CAT0:
        if name.endswith(pat):
            return "cat0"
    for pat in CAT1:
        if name.endswith(pat):
            return "cat1"
    for pat in SUMMED:
        if name.endswith(pat):
            return "sum"
    return "same"


def merge_tp(shards: List[Dict[str, torch.Tensor]], gated_mlp: bool = False) -> Dict[str, torch.Tensor]:
    """Per-rank state dicts -> one full state dict."""
    if len(shards) == 1:
        return OrderedDict(shards[0])
    out = OrderedDict()
    for name in shards[0]:
        parts = [s[name] for s in shards]
        rule = _rule(name)
        if rule == "cat0":
            if gated_mlp and name.endswith(("mlp.linear1.weight", "mlp.linear1.bias")):
                ups = [p[: p.shape[0] // 2] for p in parts]
                gates = [p[p.shape[0] // 2:] for p in parts]
                out[name] = torch.cat(ups + gates, dim=0)
            else:
                out[name] = torch.cat(parts, dim=0)
        elif rule == "cat1":
            out[name] = torch.cat(parts, dim=1)
        elif rule == "sum":
            out[name] = torch.stack([p.float() for p in parts]).sum(0).to(parts[0].dtype)
        else:
            out[name] = parts[0]
    return out


def split_tp(full: Dict[str, torch.Tensor], tp: int, gated_mlp: bool = False, gqa_sizes=None):
    """Full state dict -> ``tp`` per-rank state dicts.  ``gqa_sizes = (q_rows, k_rows, v_rows)`` of the fused
    QKV when it is laid out ``[all q; all k; all v]``: each section is split on its own."""
    if tp == 1:
        return [OrderedDict(full)]
    outs = [OrderedDict() for _ in range(tp)]
    for name, t in full.items():
        rule = _rule(name)
        if rule == "cat0":
            if gqa_sizes is not None and "query_key_value" in name:
                secs = torch.split(t, list(gqa_sizes), dim=0)
                chunks = [torch.cat([torch.chunk(s, tp, dim=0)[r] for s in secs], dim=0) for r in range(tp)]
            elif gated_mlp and name.endswith(("mlp.linear1.weight", "mlp.linear1.bias")):
                up, gate = t[: t.shape[0] // 2], t[t.shape[0] // 2:]
                chunks = [torch.cat([torch.chunk(up, tp, 0)[r], torch.chunk(gate, tp, 0)[r]], 0) for r in range(tp)]
            else:
                chunks = torch.chunk(t, tp, dim=0)
        elif rule == "cat1":
            chunks = torch.chunk(t, tp, dim=1)
        elif rule == "sum":
            chunks = [t / tp] * tp
        else:
            chunks = [t] * tp
        for r in range(tp):
            outs[r][name] = chunks[r].clone()
    return outs


# ----------------------------------------------------------------------------------------- reading / writing neox layout
def load_neox_shards(ckpt_dir: str) -> List[Dict[str, torch.Tensor]]:
    """Per-TP-rank state dicts keyed ``sequential.<idx>.<param>``, from either the sequential files
    (``mp_rank_XX_model_states.pt``) or the per-layer pipeline files (``layer_XX-model_YY-model_states.pt``)."""
    files = sorted(os.listdir(ckpt_dir))
    layer_re = re.compile(r"layer_(\d+)-model_(\d+)-model_states\.pt$")
    layer_files = [(int(m.group(1)), int(m.group(2)), f) for f in files if (m := layer_re.match(f))]
    if layer_files:
        tp = max(r for _, r, _ in layer_files) + 1
        shards = [OrderedDict() for _ in range(tp)]
        for idx, r, f in sorted(layer_files):
            sd = torch.load(os.path.join(ckpt_dir, f), map_location="cpu", weights_only=False)
            for k, v in sd.items():
                shards[r][f"sequential.{idx}.{k}"] = v
        return shards
    ms = [f for f in files if re.match(r"mp_rank_\d+_model_states\.pt$", f)]
    if not ms:
        raise FileNotFoundError(f"no model state files in {ckpt_dir}")
    shards = []
    for f in ms:
        sd = torch.load(os.path.join(ckpt_dir, f), map_location="cpu", weights_only=False)
        shards.append(OrderedDict(sd["module"] if "module" in sd and sd["module"] is not None else sd))
    return shards


def save_neox_shards(shards, out_dir: str, tag: str = "global_step0", extra=None):
    d = os.path.join(out_dir, tag)
    os.makedirs(d, exist_ok=True)
    for r, sd in enumerate(shards):
        state = {"module": sd, "optimizer": None, "lr_scheduler": None, "dp_world_size": 1,
                 "mp_world_size": len(shards), "global_steps": 0, "global_samples": 0, "skipped_steps": 0,
                 "iteration": 0}
        state.update(extra or {})
        torch.save(state, os.path.join(d, f"mp_rank_{r:02d}_model_states.pt"))
    with open(os.path.join(out_dir, "latest"), "w") as f:
        f.write(tag)
    return d


def _load_config(path) -> dict:
    cfg = {}
    for p in ([path] if isinstance(path, str) else path):
        with open(p) as f:
            cfg.update(yaml.safe_load(f))
    return {k.replace("-", "_"): v for k, v in cfg.items()}


def _layer_indices(sd):
    return sorted({int(k.split(".")[1]) for k in sd if k.startswith("sequential.")})


def _group_layers(sd):
    """-> (embedding idx, [transformer layer idx...], final norm idx, head idx or None)."""
    idxs = _layer_indices(sd)
    layers = [i for i in idxs if any(k.startswith(f"sequential.{i}.") and (".attention." in k or ".mixer." in k
                                                                           or ".mlp." in k) for k in sd)]
    emb = idxs[0]
    rest = [i for i in idxs if i > (layers[-1] if layers else emb)]
    norm = rest[0] if rest else None
    head = rest[1] if len(rest) > 1 else None
    return emb, layers, norm, head


# ----------------------------------------------------------------------------------------- QKV layout helpers
def qkv_neox_to_separate(w, heads, kv_heads, head_dim):
    """Fused full (all ranks merged rank-major) QKV -> (q, k, v) with rows ordered by head."""
    if kv_heads == heads:
        x = w.view(heads, 3, head_dim, *w.shape[1:])
        return tuple(x[:, i].reshape(heads * head_dim, *w.shape[1:]) for i in range(3))
    q, k, v = torch.split(w, [heads * head_dim, kv_heads * head_dim, kv_heads * head_dim], dim=0)
    return q, k, v


def qkv_separate_to_neox(q, k, v, heads, kv_heads, head_dim):
    if kv_heads == heads:
        tail = q.shape[1:]
        x = torch.stack([t.view(heads, head_dim, *tail) for t in (q, k, v)], dim=1)
        return x.reshape(3 * heads * head_dim, *tail)
    return torch.cat([q, k, v], dim=0)


def _merged_gqa_fix(shards, full, heads, kv_heads, head_dim):
    """With GQA each rank holds [q_r; k_r; v_r]; a plain dim-0 concat interleaves ranks.  Rebuild
    [all q; all k; all v]."""
    tp = len(shards)
    if tp == 1 or kv_heads == heads:
        return full
    qs, ks = heads * head_dim // tp, kv_heads * head_dim // tp
    for name in list(full):
        if "query_key_value" in name:
            parts = [torch.split(s[name], [qs, ks, ks], dim=0) for s in shards]
            full[name] = torch.cat([p[0] for p in parts] + [p[1] for p in parts] + [p[2] for p in parts], dim=0)
    return full


# ----------------------------------------------------------------------------------------- neox -> HF
def hf_config_from_neox(cfg: dict, architecture: str, vocab_size: int) -> dict:
    h, L, nh = cfg["hidden_size"], cfg["num_layers"], cfg["num_attention_heads"]
    kv = cfg.get("num_kv_heads") or nh
    common = {"hidden_size": h, "num_hidden_layers": L, "num_attention_heads": nh, "vocab_size": vocab_size,
              "max_position_embeddings": cfg.get("max_position_embeddings", 2048),
              "tie_word_embeddings": not cfg.get("no_weight_tying", False),
              "torch_dtype": {"fp16": "float16", "bfloat16": "bfloat16"}.get(cfg.get("precision"), "float32")}
    if architecture == "neox":
        act = cfg.get("activation", "gelu")
        common.update(architectures=["GPTNeoXForCausalLM"], model_type="gpt_neox",
                      intermediate_size=cfg.get("intermediate_size") or 4 * h,
                      hidden_act="gelu_fast" if cfg.get("bias_gelu_fusion") else act,
                      rotary_pct=cfg.get("rotary_pct", 1.0), rotary_emb_base=cfg.get("rotary_emb_base", 10000),
                      layer_norm_eps=cfg.get("layernorm_epsilon", 1e-5),
                      use_parallel_residual=bool(cfg.get("gpt_j_residual", False)),
                      attention_bias=cfg.get("use_bias_in_attn_linear", True), use_cache=True)
    else:
        inter = cfg.get("intermediate_size")
        if inter is None:
            inter = int(4 * h * 2 / 3)
            m = cfg.get("mlp_multiple_of", 256) or 1
            inter = m * ((inter + m - 1) // m)
        common.update(architectures=["LlamaForCausalLM" if architecture == "llama" else "MistralForCausalLM"],
                      model_type=architecture, intermediate_size=inter, hidden_act="silu", num_key_value_heads=kv,
                      rms_norm_eps=cfg.get("rms_norm_epsilon", 1e-8), rope_theta=cfg.get("rotary_emb_base", 10000),
                      attention_bias=False, mlp_bias=False, head_dim=h // nh, use_cache=True)
        if architecture == "mistral":
            common["sliding_window"] = cfg.get("sliding_window_width")
    return common


def neox_to_hf_state(full: Dict[str, torch.Tensor], cfg: dict, architecture: str = "neox"):
    emb, layers, norm, head = _group_layers(full)
    nh = cfg["num_attention_heads"]
    kv = cfg.get("num_kv_heads") or nh
    hd = cfg["hidden_size"] // nh
    out = OrderedDict()
    g = lambda i, n: full[f"sequential.{i}.{n}"]
    has = lambda i, n: f"sequential.{i}.{n}" in full
    nw = lambda i, n: g(i, n + ".scale") if has(i, n + ".scale") else g(i, n + ".weight")   # RMSNorm names it scale
    if architecture == "neox":
        out["gpt_neox.embed_in.weight"] = g(emb, "word_embeddings.weight")
        for li, i in enumerate(layers):
            p = f"gpt_neox.layers.{li}."
            for n in ("input_layernorm", "post_attention_layernorm"):
                for s in ("weight", "bias"):
                    if has(i, f"{n}.{s}"):
                        out[p + f"{n}.{s}"] = g(i, f"{n}.{s}")
            for src, dst in (("attention.query_key_value", "attention.query_key_value"),
                             ("attention.dense", "attention.dense"), ("mlp.linear1", "mlp.dense_h_to_4h"),
                             ("mlp.linear2", "mlp.dense_4h_to_h")):
                for s in ("weight", "bias"):
                    if has(i, f"{src}.{s}"):
                        out[p + f"{dst}.{s}"] = g(i, f"{src}.{s}")
        for s in ("weight", "bias"):
            if has(norm, f"norm.{s}"):
                out[f"gpt_neox.final_layer_norm.{s}"] = g(norm, f"norm.{s}")
        out["embed_out.weight"] = g(head, "final_linear.weight") if head is not None else g(emb, "word_embeddings.weight")
        return out
    out["model.embed_tokens.weight"] = g(emb, "word_embeddings.weight")
    for li, i in enumerate(layers):
        p = f"model.layers.{li}."
        q, k, v = qkv_neox_to_separate(g(i, "attention.query_key_value.weight"), nh, kv, hd)
        out[p + "self_attn.q_proj.weight"], out[p + "self_attn.k_proj.weight"] = q, k
        out[p + "self_attn.v_proj.weight"] = v
        out[p + "self_attn.o_proj.weight"] = g(i, "attention.dense.weight")
        w1 = g(i, "mlp.linear1.weight")
        out[p + "mlp.up_proj.weight"], out[p + "mlp.gate_proj.weight"] = w1[: w1.shape[0] // 2], w1[w1.shape[0] // 2:]
        out[p + "mlp.down_proj.weight"] = g(i, "mlp.linear2.weight")
        out[p + "input_layernorm.weight"] = nw(i, "input_layernorm")
        out[p + "post_attention_layernorm.weight"] = nw(i, "post_attention_layernorm")
    out["model.norm.weight"] = nw(norm, "norm")
    out["lm_head.weight"] = g(head, "final_linear.weight") if head is not None else g(emb, "word_embeddings.weight")
    return out


def hf_to_neox_state(hf: Dict[str, torch.Tensor], cfg: dict, architecture: str = "neox"):
    L, nh = cfg["num_layers"], cfg["num_attention_heads"]
    kv = cfg.get("num_kv_heads") or nh
    hd = cfg["hidden_size"] // nh
    out = OrderedDict()
    if architecture == "neox":
        out["sequential.0.word_embeddings.weight"] = hf["gpt_neox.embed_in.weight"]
        for li in range(L):
            p, q = f"gpt_neox.layers.{li}.", f"sequential.{li + 2}."
            for n in ("input_layernorm", "post_attention_layernorm"):
                for s in ("weight", "bias"):
                    if p + f"{n}.{s}" in hf:
                        out[q + f"{n}.{s}"] = hf[p + f"{n}.{s}"]
            for dst, src in (("attention.query_key_value", "attention.query_key_value"),
                             ("attention.dense", "attention.dense"), ("mlp.linear1", "mlp.dense_h_to_4h"),
                             ("mlp.linear2", "mlp.dense_4h_to_h")):
                for s in ("weight", "bias"):
                    if p + f"{src}.{s}" in hf:
                        out[q + f"{dst}.{s}"] = hf[p + f"{src}.{s}"]
        for s in ("weight", "bias"):
            if f"gpt_neox.final_layer_norm.{s}" in hf:
                out[f"sequential.{L + 3}.norm.{s}"] = hf[f"gpt_neox.final_layer_norm.{s}"]
        if cfg.get("no_weight_tying", False):
            out[f"sequential.{L + 4}.final_linear.weight"] = hf["embed_out.weight"]
        return out
    out["sequential.0.word_embeddings.weight"] = hf["model.embed_tokens.weight"]
    for li in range(L):
        p, q = f"model.layers.{li}.", f"sequential.{li + 2}."
        out[q + "attention.query_key_value.weight"] = qkv_separate_to_neox(
            hf[p + "self_attn.q_proj.weight"], hf[p + "self_attn.k_proj.weight"], hf[p + "self_attn.v_proj.weight"],
            nh, kv, hd)
        out[q + "attention.dense.weight"] = hf[p + "self_attn.o_proj.weight"]
        out[q + "mlp.linear1.weight"] = torch.cat([hf[p + "mlp.up_proj.weight"], hf[p + "mlp.gate_proj.weight"]], 0)
        out[q + "mlp.linear2.weight"] = hf[p + "mlp.down_proj.weight"]
        out[q + "input_layernorm.scale"] = hf[p + "input_layernorm.weight"]
        out[q + "post_attention_layernorm.scale"] = hf[p + "post_attention_layernorm.weight"]
    out[f"sequential.{L + 3}.norm.scale"] = hf["model.norm.weight"]
    if cfg.get("no_weight_tying", True):
        out[f"sequential.{L + 4}.final_linear.weight"] = hf.get("lm_head.weight", hf["model.embed_tokens.weight"])
    return out


def raw_llama_to_hf_names(raw_shards: List[Dict[str, torch.Tensor]], cfg: dict):
    """Meta's ``consolidated.NN.pth`` shards -> HF-named full tensors.  The raw format stores q/k with
    interleaved rotary pairs; the rotate-half convention used here needs them de-interleaved per head."""
    nh = cfg["num_attention_heads"]
    kv = cfg.get("num_kv_heads") or nh
    hd = cfg["hidden_size"] // nh
    cat0 = ("wq", "wk", "wv", "w1", "w3", "output", )
    cat1 = ("wo", "w2", "tok_embeddings")
    full = {}
    for name in raw_shards[0]:
        parts = [s[name] for s in raw_shards]
        leaf = name.split(".")[-2] if name.endswith(".weight") else name
        if len(parts) == 1 or parts[0].dim() == 1 or "norm" in name or "rope" in name:
            full[name] = parts[0]
        elif leaf in cat0:
            full[name] = torch.cat(parts, dim=0)
        elif leaf in cat1:
            full[name] = torch.cat(parts, dim=1)
        else:
            full[name] = parts[0]

    def unpermute(w, n):
        return w.view(n, hd // 2, 2, w.shape[1]).transpose(1, 2).reshape(n * hd, w.shape[1])

    hf = OrderedDict()
    hf["model.embed_tokens.weight"] = full["tok_embeddings.weight"]
    hf["model.norm.weight"] = full["norm.weight"]
    hf["lm_head.weight"] = full["output.weight"]
    for li in range(cfg["num_layers"]):
        p, q = f"layers.{li}.", f"model.layers.{li}."
        hf[q + "self_attn.q_proj.weight"] = unpermute(full[p + "attention.wq.weight"], nh)
        hf[q + "self_attn.k_proj.weight"] = unpermute(full[p + "attention.wk.weight"], kv)
        hf[q + "self_attn.v_proj.weight"] = full[p + "attention.wv.weight"]
        hf[q + "self_attn.o_proj.weight"] = full[p + "attention.wo.weight"]
        hf[q + "mlp.gate_proj.weight"] = full[p + "feed_forward.w1.weight"]
        hf[q + "mlp.down_proj.weight"] = full[p + "feed_forward.w2.weight"]
        hf[q + "mlp.up_proj.weight"] = full[p + "feed_forward.w3.weight"]
        hf[q + "input_layernorm.weight"] = full[p + "attention_norm.weight"]
        hf[q + "post_attention_layernorm.weight"] = full[p + "ffn_norm.weight"]
    return hf


def neox_to_mamba_ssm_state(full: Dict[str, torch.Tensor]):
    emb, layers, norm, head = _group_layers(full)
    out = OrderedDict()
    out["backbone.embedding.weight"] = full[f"sequential.{emb}.word_embeddings.weight"]
    for li, i in enumerate(layers):
        for k, v in full.items():
            pre = f"sequential.{i}."
            if k.startswith(pre):
                out[f"backbone.layers.{li}." + k[len(pre):]] = v
    out["backbone.norm_f.weight"] = full.get(f"sequential.{norm}.norm.scale", full.get(f"sequential.{norm}.norm.weight"))
    out["lm_head.weight"] = full[f"sequential.{head}.final_linear.weight"] if head is not None \
        else out["backbone.embedding.weight"]
    return out


# ----------------------------------------------------------------------------------------- drivers
def _gated(cfg):
    return cfg.get("activation", "gelu") in ("swiglu", "geglu", "reglu", "bilinear", "glu")


_PRECISIONS = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32, "auto": None, None: None}


def convert_neox_to_hf(input_dir, config_file, output_dir, architecture="neox", vocab_size=None, precision=None,
                       pad_token_id=None, save_tokenizer=True):
    """``precision``: cast the floating-point weights (``auto`` / None keeps the checkpoint's dtype);
    ``pad_token_id``: written into ``config.json``; ``save_tokenizer``: copy the ``vocab_file`` of an
    ``HFTokenizer`` config beside the weights as ``tokenizer.json``."""
    cfg = _load_config(config_file)
    shards = load_neox_shards(input_dir)
    full = merge_tp(shards, gated_mlp=_gated(cfg))
    nh = cfg["num_attention_heads"]
    full = _merged_gqa_fix(shards, full, nh, cfg.get("num_kv_heads") or nh, cfg["hidden_size"] // nh)
    hf = neox_to_hf_state(full, cfg, architecture)
    emb_key = "gpt_neox.embed_in.weight" if architecture == "neox" else "model.embed_tokens.weight"
    vocab = vocab_size or hf[emb_key].shape[0]
    if vocab < hf[emb_key].shape[0]:                       # drop padding rows
        for k in (emb_key, "embed_out.weight", "lm_head.weight"):
            if k in hf:
                hf[k] = hf[k][:vocab].clone()
    dtype = _PRECISIONS[precision]
    if dtype is not None:
        hf = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in hf.items()}
    os.makedirs(output_dir, exist_ok=True)
    hf_cfg = hf_config_from_neox(cfg, architecture, vocab)
    if dtype is not None:
        hf_cfg["torch_dtype"] = str(dtype).replace("torch.", "")
    if pad_token_id is not None:
        hf_cfg["pad_token_id"] = int(pad_token_id)
    with open(os.path.join(output_dir, "config.json"), "w") as f:
        json.dump(hf_cfg, f, indent=2)
    torch.save({k: v.contiguous() for k, v in hf.items()}, os.path.join(output_dir, "pytorch_model.bin"))
    vocab_file = cfg.get("vocab_file")
    if save_tokenizer and cfg.get("tokenizer_type", "") == "HFTokenizer" and vocab_file and os.path.exists(vocab_file):
        import shutil
        shutil.copyfile(vocab_file, os.path.join(output_dir, "tokenizer.json"))
    return hf


def convert_hf_to_neox(hf_dir, config_file, output_dir, tp=1, architecture=None):
    cfg = _load_config(config_file)
    if architecture is None:
        with open(os.path.join(hf_dir, "config.json")) as f:
            architecture = {"gpt_neox": "neox"}.get(json.load(f).get("model_type", "gpt_neox"), "llama")
    path = os.path.join(hf_dir, "pytorch_model.bin")
    if os.path.exists(path):
        hf = torch.load(path, map_location="cpu", weights_only=False)
    else:
        from safetensors.torch import load_file
        hf = {}
        for f in sorted(os.listdir(hf_dir)):
            if f.endswith(".safetensors"):
                hf.update(load_file(os.path.join(hf_dir, f)))
    full = hf_to_neox_state(hf, cfg, architecture)
    full = _pad_vocab(full, cfg, tp)
    nh = cfg["num_attention_heads"]
    kvh = cfg.get("num_kv_heads") or nh
    hd = cfg["hidden_size"] // nh
    gqa = (nh * hd, kvh * hd, kvh * hd) if kvh != nh else None
    return save_neox_shards(split_tp(full, tp, gated_mlp=_gated(cfg), gqa_sizes=gqa), output_dir)


def _pad_vocab(full, cfg, tp):
    mult = cfg.get("make_vocab_size_divisible_by", 128) * tp
    for k in list(full):
        if k.endswith(("word_embeddings.weight", "final_linear.weight")):
            v = full[k]
            pad = (-v.shape[0]) % mult
            if pad:
                full[k] = torch.cat([v, v.new_zeros(pad, v.shape[1])], dim=0)
    return full


def convert_raw_llama_to_neox(input_dir, config_file, output_dir, tp=1):
    cfg = _load_config(config_file)
    files = sorted(f for f in os.listdir(input_dir) if re.match(r"consolidated\.\d+\.pth$", f))
    raw = [torch.load(os.path.join(input_dir, f), map_location="cpu", weights_only=False) for f in files]
    hf = raw_llama_to_hf_names(raw, cfg)
    full = _pad_vocab(hf_to_neox_state(hf, dict(cfg, no_weight_tying=True), "llama"), cfg, tp)
    nh = cfg["num_attention_heads"]
    kvh = cfg.get("num_kv_heads") or nh
    hd = cfg["hidden_size"] // nh
    gqa = (nh * hd, kvh * hd, kvh * hd) if kvh != nh else None
    return save_neox_shards(split_tp(full, tp, gated_mlp=True, gqa_sizes=gqa), output_dir)


def inspect(path, out=print):
    """Print the tree of keys, shapes and dtypes of a checkpoint file or of every ``.pt`` in a directory."""
    files = [path] if os.path.isfile(path) else sorted(os.path.join(path, f) for f in os.listdir(path)
                                                       if f.endswith((".pt", ".pth", ".bin")))

    def walk(obj, indent):
        if isinstance(obj, dict):
            for k, v in obj.items():
                if torch.is_tensor(v):
                    out(f"{' ' * indent}{k}: {tuple(v.shape)} {str(v.dtype).replace('torch.', '')}")
                elif isinstance(v, (dict, list, tuple)):
                    out(f"{' ' * indent}{k}:")
                    walk(v, indent + 2)
                else:
                    s = repr(v)
                    out(f"{' ' * indent}{k}: {s if len(s) < 80 else s[:77] + '...'}")
        elif isinstance(obj, (list, tuple)):
            for i, v in enumerate(obj[:50]):
                walk({f"[{i}]": v}, indent)
    for f in files:
        out(f"== {f}")
        walk(torch.load(f, map_location="cpu", weights_only=False), 2)


def _flatten(obj, prefix=""):
    out = {}
    if isinstance(obj, dict):
        for k, v in obj.items():
            out.update(_flatten(v, f"{prefix}{k}." if not torch.is_tensor(v) else f"{prefix}{k}"))
    elif isinstance(obj, (list, tuple)):
        for i, v in enumerate(obj):
            out.update(_flatten(v, f"{prefix}{i}." if not torch.is_tensor(v) else f"{prefix}{i}"))
    else:
        out[prefix.rstrip(".") if not torch.is_tensor(obj) else prefix] = obj
    return out


def diff(path_a, path_b, attributes=(), out=print):
    """Compare two checkpoint files key by key: entries present on one side only, tensors whose shape or dtype
    differ, and the largest absolute difference of those that match in shape.  ``attributes`` names extra
    tensor reductions to print for differing tensors (``mean``, ``std``, ``norm``, ``min``, ``max``).
    Returns the number of differing entries."""
    a = _flatten(torch.load(path_a, map_location="cpu", weights_only=False))
    b = _flatten(torch.load(path_b, map_location="cpu", weights_only=False))
    n = 0
    for k in sorted(set(a) | set(b)):
        if k not in a or k not in b:
            out(f"{'<' if k in a else '>'} {k}: only in {path_a if k in a else path_b}")
            n += 1
            continue
        va, vb = a[k], b[k]
        if torch.is_tensor(va) and torch.is_tensor(vb):
            if va.shape != vb.shape or va.dtype != vb.dtype:
                out(f"! {k}: {tuple(va.shape)} {va.dtype} vs {tuple(vb.shape)} {vb.dtype}")
                n += 1
            elif not torch.equal(va, vb):
                d = (va.double() - vb.double()).abs().max().item()
                extra = "".join(f" {at}: {getattr(va.double(), at)().item():.6g} vs {getattr(vb.double(), at)().item():.6g}"
                                for at in attributes)
                out(f"~ {k}: max |a - b| = {d:.6g}{extra}")
                n += 1
        elif torch.is_tensor(va) != torch.is_tensor(vb) or va != vb:
            out(f"~ {k}: {va!r} vs {vb!r}")
            n += 1
    out(f"{n} differing entries")
    return n


def upload(hf_dir, repo_id, private=False):
    try:
        from huggingface_hub import HfApi
    except ImportError as e:
        raise RuntimeError("upload needs the `huggingface_hub` package and network access") from e
    api = HfApi()
    api.create_repo(repo_id, private=private, exist_ok=True)
    api.upload_folder(folder_path=hf_dir, repo_id=repo_id)


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = p.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("neox-to-hf")
    a.add_argument("--input_dir", required=True); a.add_argument("--config_file", required=True, nargs="+")
    a.add_argument("--output_dir", required=True); a.add_argument("--architecture", default="neox",
                                                                   choices=["neox", "llama", "mistral"])
    a.add_argument("--vocab_size", type=int, default=None)
    a.add_argument("--precision", default="auto", choices=["auto", "fp16", "bf16", "fp32"])
    a.add_argument("--pad-token-id", "--pad_token_id", dest="pad_token_id", type=int, default=None)
    a.add_argument("--no_save_tokenizer", action="store_true")
    a = sub.add_parser("hf-to-neox")
    # the second spelling of each flag is the one the reference's convert_hf_to_sequential.py takes
    a.add_argument("--hf_dir", "--hf-model-name", dest="hf_dir", required=True)
    a.add_argument("--config_file", "--config", dest="config_file", required=True, nargs="+")
    a.add_argument("--output_dir", "--output-dir", dest="output_dir", required=True)
    a.add_argument("--tp", type=int, default=1)
    a.add_argument("--pp", type=int, default=0, help="accepted for parity: the per-layer files written here load "
                                                     "under any pipeline-parallel size")
    a = sub.add_parser("raw-llama-to-neox")
    a.add_argument("--input_dir", required=True); a.add_argument("--config_file", required=True, nargs="+")
    a.add_argument("--output_dir", required=True); a.add_argument("--tp", type=int, default=1)
    a = sub.add_parser("merge")
    a.add_argument("--input_dir", required=True); a.add_argument("--output_dir", required=True)
    a.add_argument("--config_file", nargs="+", default=None)
    a = sub.add_parser("neox-to-mamba-ssm")
    a.add_argument("--input_dir", required=True); a.add_argument("--output_dir", required=True)
    a = sub.add_parser("inspect")
    a.add_argument("path", nargs="?")
    a.add_argument("--diff", "--compare", dest="diff", nargs=2, metavar=("A", "B"), default=None)
    a.add_argument("--attributes", nargs="*", default=[])
    a = sub.add_parser("upload")
    a.add_argument("--hf_dir", required=True); a.add_argument("--repo_id", required=True)
    a.add_argument("--private", action="store_true")
    args = p.parse_args(argv)
    if args.cmd == "neox-to-hf":
        convert_neox_to_hf(args.input_dir, args.config_file, args.output_dir, args.architecture, args.vocab_size,
                           precision=args.precision, pad_token_id=args.pad_token_id,
                           save_tokenizer=not args.no_save_tokenizer)
    elif args.cmd == "hf-to-neox":
        convert_hf_to_neox(args.hf_dir, args.config_file, args.output_dir, args.tp)
    elif args.cmd == "raw-llama-to-neox":
        convert_raw_llama_to_neox(args.input_dir, args.config_file, args.output_dir, args.tp)
    elif args.cmd == "merge":
        cfg = _load_config(args.config_file) if args.config_file else {}
        save_neox_shards([merge_tp(load_neox_shards(args.input_dir), gated_mlp=_gated(cfg))], args.output_dir)
    elif args.cmd == "neox-to-mamba-ssm":
        os.makedirs(args.output_dir, exist_ok=True)
        torch.save(neox_to_mamba_ssm_state(merge_tp(load_neox_shards(args.input_dir))),
                   os.path.join(args.output_dir, "pytorch_model.bin"))
    elif args.cmd == "inspect":
        if args.diff:
            diff(args.diff[0], args.diff[1], args.attributes)
        else:
            inspect(args.path)
    elif args.cmd == "upload":
        upload(args.hf_dir, args.repo_id, args.private)


if __name__ == "__main__":
    main()

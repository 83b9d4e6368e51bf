"""Checkpoint conversion: logits parity with the independent Hugging Face implementations, TP split/merge
round trips, raw-LLaMA q/k de-interleave."""
import os

import pytest
import torch

from common import tiny_config


def _build(**over):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.initialize import initialize_megatron
    cfg = tiny_config(use_cpu_initialization=True, attention_config=[[["global"], 2]], **over)
    a = NeoXArgs.from_dict(cfg)
    a.configure_distributed_args()
    a.build_tokenizer()
    mpu.destroy_model_parallel()
    initialize_megatron(a)
    torch.manual_seed(3)
    m = training.get_model(a)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.02)                      # exercise the bias mappings
    return cfg, a, m.eval()


def _logits(m, tokens):
    from gpt_neox_b200.utils.common import get_attn_mask
    s = tokens.shape[1]
    pos = torch.arange(s)[None].expand(tokens.shape[0], -1)
    with torch.no_grad():
        return m((tokens, pos, get_attn_mask(s, "cpu", None))).float()


@pytest.mark.parametrize("arch,over", [
    ("neox", dict()),
    ("neox", dict(gpt_j_residual=False, rotary_pct=1.0)),
    ("llama", dict(norm="rmsnorm", activation="swiglu", use_bias_in_mlp=False, use_bias_in_attn_linear=False,
                   gpt_j_residual=False, rotary_pct=1.0, mlp_multiple_of=32, rms_norm_epsilon=1e-6)),
    ("llama", dict(norm="rmsnorm", activation="swiglu", use_bias_in_mlp=False, use_bias_in_attn_linear=False,
                   gpt_j_residual=False, rotary_pct=1.0, mlp_multiple_of=32, rms_norm_epsilon=1e-6,
                   num_kv_heads=2)),
])
def test_logits_match_huggingface(arch, over):
    import transformers
    from gpt_neox_b200.ckpt import convert
    cfg, a, m = _build(**over)
    full = {k: v.detach().clone() for k, v in m.state_dict().items()}
    hf_sd = convert.neox_to_hf_state(full, cfg, arch)
    hc = convert.hf_config_from_neox(cfg, arch, a.padded_vocab_size)
    if arch == "llama":
        hc["intermediate_size"] = full["sequential.2.mlp.linear2.weight"].shape[1]
    hc.pop("architectures"), hc.pop("torch_dtype")
    mt = hc.pop("model_type")
    conf = (transformers.GPTNeoXConfig if mt == "gpt_neox" else transformers.LlamaConfig)(**hc)
    conf._attn_implementation = "eager"
    hf = (transformers.GPTNeoXForCausalLM if mt == "gpt_neox" else transformers.LlamaForCausalLM)(conf).eval()
    missing, unexpected = hf.load_state_dict(hf_sd, strict=False)
    assert not unexpected, unexpected
    assert all("rotary" in k or "inv_freq" in k or "masked_bias" in k or k.endswith(".attention.bias")
               for k in missing), missing
    tokens = torch.randint(0, 100, (2, 24))
    ours = _logits(m, tokens)
    with torch.no_grad():
        theirs = hf(tokens).logits.float()
    torch.testing.assert_close(ours, theirs, rtol=2e-4, atol=2e-4)
    # and back
    back = convert.hf_to_neox_state(hf_sd, dict(cfg, no_weight_tying=True), arch)
    for k, v in back.items():
        torch.testing.assert_close(v, full[k])


@pytest.mark.parametrize("gated,kv", [(False, None), (True, 2)])
def test_tp_split_merge_roundtrip(gated, kv):
    from gpt_neox_b200.ckpt import convert
    over = dict(num_kv_heads=kv) if kv else {}
    if gated:
        over.update(activation="swiglu", mlp_multiple_of=32)
    cfg, a, m = _build(**over)
    full = {k: v.detach().clone() for k, v in m.state_dict().items()}
    nh, hd = cfg["num_attention_heads"], cfg["hidden_size"] // cfg["num_attention_heads"]
    gqa = (nh * hd, kv * hd, kv * hd) if kv else None
    shards = convert.split_tp(full, 2, gated_mlp=gated, gqa_sizes=gqa)
    assert shards[0]["sequential.2.attention.dense.weight"].shape[1] == cfg["hidden_size"] // 2
    merged = convert.merge_tp(shards, gated_mlp=gated)
    merged = convert._merged_gqa_fix(shards, merged, nh, kv or nh, hd)
    for k, v in full.items():
        torch.testing.assert_close(merged[k], v, msg=k)


def test_cli_neox_to_hf_and_inspect(tmp_path):
    import yaml
    from gpt_neox_b200.ckpt import convert
    cfg, a, m = _build()
    d = convert.save_neox_shards(convert.split_tp({k: v.detach() for k, v in m.state_dict().items()}, 2),
                                 str(tmp_path / "ckpt"))
    cf = tmp_path / "cfg.yml"
    cf.write_text(yaml.safe_dump({k: v for k, v in cfg.items()}))
    convert.main(["neox-to-hf", "--input_dir", d, "--config_file", str(cf), "--output_dir", str(tmp_path / "hf")])
    assert os.path.exists(tmp_path / "hf" / "config.json") and os.path.exists(tmp_path / "hf" / "pytorch_model.bin")
    lines = []
    convert.inspect(d, out=lines.append)
    assert any("query_key_value.weight" in l for l in lines)
    out = convert.convert_hf_to_neox(str(tmp_path / "hf"), str(cf), str(tmp_path / "back"), tp=2)
    back = convert.merge_tp(convert.load_neox_shards(out))
    torch.testing.assert_close(back["sequential.2.mlp.linear1.weight"], m.state_dict()["sequential.2.mlp.linear1.weight"])


def test_raw_llama_unpermute_is_inverse_of_interleave():
    from gpt_neox_b200.ckpt import convert
    cfg = dict(num_attention_heads=2, hidden_size=8, num_layers=1)
    hd = 4
    w_hf = torch.arange(8 * 8, dtype=torch.float32).view(8, 8)
    # HF (rotate-half) -> raw (interleaved pairs): the permutation Meta-format loaders apply
    w_raw = w_hf.view(2, 2, hd // 2, 8).transpose(1, 2).reshape(8, 8)
    raw = {"tok_embeddings.weight": torch.zeros(4, 8), "norm.weight": torch.ones(8), "output.weight": torch.zeros(4, 8),
           "layers.0.attention.wq.weight": w_raw, "layers.0.attention.wk.weight": w_raw,
           "layers.0.attention.wv.weight": w_hf, "layers.0.attention.wo.weight": w_hf,
           "layers.0.feed_forward.w1.weight": torch.zeros(6, 8), "layers.0.feed_forward.w2.weight": torch.zeros(8, 6),
           "layers.0.feed_forward.w3.weight": torch.zeros(6, 8), "layers.0.attention_norm.weight": torch.ones(8),
           "layers.0.ffn_norm.weight": torch.ones(8)}
    hf = convert.raw_llama_to_hf_names([raw], cfg)
    torch.testing.assert_close(hf["model.layers.0.self_attn.q_proj.weight"], w_hf)

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


_LLAMA = dict(norm="rmsnorm", activation="swiglu", use_bias_in_mlp=False, use_bias_in_attn_linear=False,
              gpt_j_residual=False, rotary_pct=1.0, mlp_multiple_of=32, rms_norm_epsilon=1e-6, no_weight_tying=True)


def _rank_logits(rank, world, cfg, tokens, train_iters):
    """Train (``train_iters`` > 0, saving at the end) or load, then return the full-vocabulary logits of ``tokens``."""
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.utils.common import get_attn_mask
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world, train_iters=max(train_iters, 1)))
    a.configure_distributed_args()
    a.build_tokenizer()
    if train_iters > 0:
        model = training.pretrain(a)
    else:
        initialize_megatron(a)
        model, _, _, _ = training.setup_model_and_optimizer(neox_args=a, use_cache=False)
    net = getattr(model, "module", model)
    net.eval()
    t = torch.tensor(tokens)
    pos = torch.arange(t.shape[1])[None].expand(t.shape[0], -1)
    with torch.no_grad():
        out = net((t, pos, get_attn_mask(t.shape[1], "cpu", None))).float()
        if world > 1:
            out = mpu.gather_from_model_parallel_region(out)
    return out.tolist()


def test_tp2_checkpoint_files_round_trip_through_huggingface(tmp_path):
    """Real files, tensor parallel 2, grouped-query attention: (a) train, save, merge + convert to a Hugging Face
    Llama folder: same logits; (b) split that folder back into a TP-2 NeoX checkpoint, load it: same logits."""
    import transformers
    import yaml
    from common import run_distributed
    from gpt_neox_b200.ckpt import convert
    tokens = torch.randint(0, 100, (2, 24), generator=torch.Generator().manual_seed(0)).tolist()
    base = tiny_config(use_cpu_initialization=True, attention_config=[[["global"], 2]], make_vocab_size_divisible_by=64,
                       model_parallel_size=2, num_kv_heads=2, **_LLAMA)
    cfg = dict(base, save=str(tmp_path / "ck"), checkpoint_factor=2)
    ours = torch.tensor(run_distributed(_rank_logits, 2, cfg, tokens, 2)[0])
    with open(tmp_path / "cfg.yml", "w") as f:
        yaml.safe_dump(cfg, f)
    convert.convert_neox_to_hf(str(tmp_path / "ck" / "global_step2"), str(tmp_path / "cfg.yml"), str(tmp_path / "hf"),
                               architecture="llama")
    hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "hf"), attn_implementation="eager").eval().float()
    with torch.no_grad():
        theirs = hf(torch.tensor(tokens)).logits.float()
    torch.testing.assert_close(ours[..., :theirs.shape[-1]], theirs, rtol=2e-4, atol=2e-4)
    back = dict(base, load=str(tmp_path / "neox"), finetune=True, optimizer=None, no_load_optim=True)
    with open(tmp_path / "back.yml", "w") as f:
        yaml.safe_dump(back, f)
    convert.convert_hf_to_neox(str(tmp_path / "hf"), str(tmp_path / "back.yml"), str(tmp_path / "neox"), tp=2,
                               architecture="llama")
    again = torch.tensor(run_distributed(_rank_logits, 2, back, tokens, 0)[0])
    torch.testing.assert_close(again[..., :theirs.shape[-1]], theirs, rtol=2e-4, atol=2e-4)
    # the command-line form with a cast and a padding token
    convert.main(["neox-to-hf", "--input_dir", str(tmp_path / "ck" / "global_step2"), "--config_file",
                  str(tmp_path / "cfg.yml"), "--output_dir", str(tmp_path / "hf16"), "--architecture", "llama",
                  "--precision", "bf16", "--pad-token-id", "3", "--no_save_tokenizer"])
    import json
    hcfg = json.load(open(tmp_path / "hf16" / "config.json"))
    assert hcfg["torch_dtype"] == "bfloat16" and hcfg["pad_token_id"] == 3
    sd = torch.load(tmp_path / "hf16" / "pytorch_model.bin")
    assert all(v.dtype == torch.bfloat16 for v in sd.values() if v.is_floating_point())


def test_checkpoint_diff_and_cli_flags(tmp_path):
    from gpt_neox_b200.ckpt import convert
    a = {"module": {"w": torch.ones(2, 3), "b": torch.zeros(3)}, "iteration": 5, "only_a": 1}
    b = {"module": {"w": torch.ones(2, 3) * 1.5, "b": torch.zeros(4)}, "iteration": 6}
    torch.save(a, tmp_path / "a.pt")
    torch.save(b, tmp_path / "b.pt")
    lines = []
    n = convert.diff(str(tmp_path / "a.pt"), str(tmp_path / "b.pt"), attributes=["mean"], out=lines.append)
    assert n == 4
    text = "\n".join(lines)
    assert "~ module.w: max |a - b| = 0.5 mean: 1 vs 1.5" in text and "! module.b" in text
    assert "< only_a" in text and "~ iteration: 5 vs 6" in text
    assert convert.diff(str(tmp_path / "a.pt"), str(tmp_path / "a.pt"), out=lines.append) == 0
    convert.main(["inspect", "--diff", str(tmp_path / "a.pt"), str(tmp_path / "b.pt"), "--attributes", "std"])
    convert.main(["inspect", str(tmp_path / "a.pt")])

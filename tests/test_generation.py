"""Text generation on CPU: sampling filters, stop sequences, and KV-cache decoding == full recompute."""
import pytest
import torch

from common import tiny_config


def _model(**over):
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
    m = training.get_model(a, use_cache=True)
    return a, m


def test_filter_logits_topk_topp():
    from gpt_neox_b200.text_generation_utils import filter_logits
    logits = torch.tensor([[1.0, 2.0, 3.0, 4.0], [4.0, 3.0, 2.0, 1.0]])
    out = filter_logits(logits.clone(), top_k=2)
    assert torch.isinf(out[0, :2]).all() and torch.isfinite(out[0, 2:]).all()
    assert torch.isinf(out[1, 2:]).all() and torch.isfinite(out[1, :2]).all()
    p = torch.tensor([[0.5, 0.3, 0.15, 0.05]]).log()
    out = filter_logits(p.clone(), top_p=0.7)
    assert torch.isfinite(out[0, :2]).all() and torch.isinf(out[0, 2:]).all()


def test_pad_batch_and_stop_tokens():
    from gpt_neox_b200.text_generation_utils import pad_batch, stop_tokens_in_completion
    toks, lens = pad_batch([[1, 2, 3], [4]], pad_id=0, pad_len=5)
    assert toks == [[1, 2, 3, 0, 0], [4, 0, 0, 0, 0]] and lens == [3, 1]
    with pytest.raises(ValueError):
        pad_batch([[1] * 6], pad_id=0, pad_len=5)
    ctx = torch.tensor([[5, 6, 7, 8, 0]])
    assert stop_tokens_in_completion([torch.tensor([7, 8])], ctx, 0, 3)
    assert not stop_tokens_in_completion([torch.tensor([6, 8])], ctx, 0, 3)


@pytest.mark.parametrize("over", [dict(), dict(pos_emb="learned"), dict(gpt_j_residual=False, num_kv_heads=2),
                                  dict(pos_emb="sinusoidal"), dict(pos_emb="alibi"), dict(sliding_window_width=4),
                                  dict(pos_emb="rpe", rpe_num_buckets=8, rpe_max_distance=16)])
def test_kv_cache_decoding_matches_recompute(over):
    from gpt_neox_b200.text_generation_utils import stream_tokens
    a, m = _model(**over)
    prompts = [[5, 9, 11, 3], [7, 2]]
    outs = []
    for recompute in (True, False):
        m.inference_mode(use_cache=not recompute)
        m.clear_cache()
        last = None
        for last in stream_tokens(a, m, prompts, maximum_tokens=6, recompute=recompute, eos_token_id=10 ** 6):
            pass
        outs.append(last[0][:, :10].clone())
    assert torch.equal(outs[0], outs[1]), (outs[0], outs[1])
    assert torch.equal(outs[0][0, :4], torch.tensor([5, 9, 11, 3]))


def test_generate_samples_from_prompt_returns_records():
    from gpt_neox_b200.text_generation_utils import generate_samples_from_prompt
    a, m = _model()
    m.inference_mode(use_cache=True)

    class _Tok:
        eod = 0

        def tokenize(self, s):
            return [min(ord(c), 99) for c in s] or [0]

        def detokenize(self, ids):
            return "".join(chr(33 + (i % 60)) for i in ids)
    a.tokenizer = _Tok()
    m.clear_cache()
    out = generate_samples_from_prompt(a, m, ["ab", ""], maximum_tokens=4, temperature=0.8, top_k=5)
    assert len(out) == 2 and all(set(r) >= {"context", "text", "length", "finished", "message"} for r in out)
    assert out[0]["length"] <= 4


def test_eval_adapter_loglikelihood_matches_direct_computation():
    from gpt_neox_b200.eval_tasks import EvalHarnessAdapter
    a, m = _model()

    class _Tok:
        eod = 0
        eod_id = 0

        def tokenize(self, s):
            return [3 + (ord(c) % 90) for c in s]

        def detokenize(self, ids):
            return "".join(chr(40 + (i % 50)) for i in ids)
    a.tokenizer = _Tok()
    ad = EvalHarnessAdapter(m, None, a, batch_size=2)
    reqs = [("hello wor", "ld"), ("", "abc"), ("a much longer context string", " x")]
    got = ad.loglikelihood(reqs)
    m.inference_mode(use_cache=False)
    for (ctx, cont), (ll, greedy) in zip(reqs, got):
        c = [0] if ctx == "" else a.tokenizer.tokenize(ctx)
        t = a.tokenizer.tokenize(cont)
        full = torch.tensor([c + t])
        pos = torch.arange(full.shape[1] - 1)[None]
        from gpt_neox_b200.utils.common import get_attn_mask
        with torch.no_grad():
            logits = m((full[:, :-1], pos, get_attn_mask(full.shape[1] - 1, "cpu", None)))
        lp = torch.log_softmax(logits.float(), -1)[0, -len(t):]
        want = lp.gather(1, torch.tensor(t)[:, None]).sum().item()
        assert ll == pytest.approx(want, rel=1e-4, abs=1e-4)
        assert greedy == bool((lp.argmax(-1) == torch.tensor(t)).all())
    assert len(ad.loglikelihood_rolling([("some document text " * 5,)])) == 1


def test_recurrent_stacks_decode_by_recompute():
    """Mamba / RWKV blocks keep no state between calls, so asking for cached decoding must still run the whole
    prefix: same tokens as an explicit recompute."""
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.text_generation_utils import stream_tokens
    a = NeoXArgs.from_dict(tiny_config(use_cpu_initialization=True, attention_config=[[["rwkv"], 2]],
                                       num_attention_heads=1))
    a.configure_distributed_args()
    a.build_tokenizer()
    mpu.destroy_model_parallel()
    initialize_megatron(a)
    m = training.get_model(a, use_cache=True)
    outs = []
    for recompute in (True, False):
        m.inference_mode(use_cache=not recompute)
        m.clear_cache()
        last = None
        for last in stream_tokens(a, m, [[5, 9, 11, 3], [7, 2]], maximum_tokens=6, recompute=recompute,
                                  eos_token_id=10 ** 6):
            pass
        outs.append(last[0][:, :10].clone())
    assert torch.equal(outs[0], outs[1])


def test_sinusoidal_table_rows_follow_position_ids():
    from gpt_neox_b200.models.positional_embeddings import SinusoidalPositionalEmbedding
    e = SinusoidalPositionalEmbedding(8, precision=torch.float32)
    full = e(torch.arange(6)[None])                     # [1, 6, 8]
    one = e(torch.tensor([[4]]))                        # the row a cached decoding step asks for
    torch.testing.assert_close(one[0, 0], full[0, 4])


def _generate(rank, world, cfg, recompute):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.text_generation_utils import stream_tokens
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world))
    a.configure_distributed_args()
    a.build_tokenizer()
    initialize_megatron(a)
    model, _, _, _ = training.setup_model_and_optimizer(neox_args=a, use_cache=True)
    model.eval()
    net = getattr(model, "module", model)
    net.inference_mode(use_cache=not recompute)
    net.clear_cache()
    last = None
    for last in stream_tokens(a, model, [[5, 9, 11, 3], [7, 2]], maximum_tokens=6, recompute=recompute,
                              eos_token_id=10 ** 6):
        pass
    return last[0][:, :10].tolist()


def test_greedy_generation_is_the_same_under_tensor_and_pipeline_parallelism():
    """Same master weights (CPU initialisation) and the same padded vocabulary: one rank, two tensor-parallel ranks
    and two pipeline stages (whose engine re-runs the prefix instead of using the KV cache) emit the same tokens."""
    from common import run_distributed
    base = dict(use_cpu_initialization=True, make_vocab_size_divisible_by=64, attention_config=[[["global"], 2]],
                optimizer=None, no_load_optim=True)
    one = run_distributed(_generate, 1, tiny_config(**base), False)[0]
    tp2 = run_distributed(_generate, 2, tiny_config(model_parallel_size=2, **base), False)[0]
    pp2 = run_distributed(_generate, 2, tiny_config(pipe_parallel_size=2, **base), False)[0]
    assert one[0][:4] == [5, 9, 11, 3] and one[1][:2] == [7, 2]
    assert tp2 == one and pp2 == one


def _loglikelihoods(rank, world, cfg, reqs):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.eval_tasks.eval_adapter import EvalHarnessAdapter
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.text_generation_utils import forward_model
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world))
    a.configure_distributed_args()
    a.build_tokenizer()
    initialize_megatron(a)
    model, _, _, _ = training.setup_model_and_optimizer(neox_args=a, use_cache=False)
    ad = EvalHarnessAdapter(model, forward_model, a, batch_size=2)
    return [(round(float(l), 3), bool(g)) for l, g in ad.loglikelihood(reqs)]


def test_eval_adapter_scores_are_layout_independent():
    """Requests of different lengths (so the batches have different shapes, which the pipeline stages must
    re-announce to each other): one rank, two pipeline stages and two tensor-parallel ranks give the same scores."""
    from common import run_distributed
    base = dict(use_cpu_initialization=True, make_vocab_size_divisible_by=64, attention_config=[[["global"], 2]],
                optimizer=None, no_load_optim=True, tokenizer_type="CharLevelTokenizer", dataset_impl="gpt2")
    reqs = [("hello wor", "ld"), ("", "abc"), ("some longer context here", " and a continuation"), ("x", "y")]
    one = run_distributed(_loglikelihoods, 1, tiny_config(**base), reqs)[0]
    pp2 = run_distributed(_loglikelihoods, 2, tiny_config(pipe_parallel_size=2, **base), reqs)[0]
    tp2 = run_distributed(_loglikelihoods, 2, tiny_config(model_parallel_size=2, **base), reqs)[0]
    assert len(one) == 4 and all(l < 0 for l, _ in one)
    assert pp2 == one and tp2 == one


def _run_local_eval(rank, world, cfg, task_dir):
    import os
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.eval_tasks import run_eval_harness
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.text_generation_utils import forward_model
    torch.set_num_threads(1)
    os.environ["NEOX_EVAL_TASK_DIR"] = task_dir
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world))
    a.configure_distributed_args()
    a.build_tokenizer()
    initialize_megatron(a)
    model, _, _, _ = training.setup_model_and_optimizer(neox_args=a, use_cache=False)
    return run_eval_harness(model, forward_model, a, batch_size=2, eval_tasks=["choice", "lastword", "wiki"])


def test_eval_harness_runs_end_to_end_on_local_task_files(tmp_path):
    """``run_eval_harness`` (what ``eval.py`` and the in-training evaluation call) on three task files of the three
    request types, without the lm_eval package: metrics of the harness's shape, identical on one rank and on two
    pipeline stages, and a task with no local file asks for lm_eval by name."""
    import json
    from common import run_distributed
    rows = [{"query": f"the number after {i} is", "choices": [f" {i + 1}", f" {i + 2}", " zero"], "gold": i % 3}
            for i in range(6)]
    (tmp_path / "choice.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    (tmp_path / "lastword.jsonl").write_text("\n".join(json.dumps({"text": f"row {i} ends with the word stop"})
                                                       for i in range(4)))
    (tmp_path / "wiki.jsonl").write_text(json.dumps({"document": "a short document of a few words " * 3}))
    base = dict(use_cpu_initialization=True, make_vocab_size_divisible_by=64, attention_config=[[["global"], 2]],
                optimizer=None, no_load_optim=True, tokenizer_type="CharLevelTokenizer", dataset_impl="gpt2")
    one = run_distributed(_run_local_eval, 1, tiny_config(**base), str(tmp_path))[0]
    res = one["results"]
    assert set(res) == {"choice", "lastword", "wiki"}
    assert 0.0 <= res["choice"]["acc"] <= 1.0 and 0.0 <= res["choice"]["acc_norm"] <= 1.0
    assert res["lastword"]["ppl"] > 1.0 and 0.0 <= res["lastword"]["acc"] <= 1.0
    assert res["wiki"]["byte_perplexity"] > 1.0 and res["wiki"]["bits_per_byte"] > 0.0
    pp2 = run_distributed(_run_local_eval, 2, tiny_config(pipe_parallel_size=2, **base), str(tmp_path))[0]
    for task in res:
        for metric, v in res[task].items():
            assert pp2["results"][task][metric] == pytest.approx(v, rel=1e-4), (task, metric)
    from gpt_neox_b200.eval_tasks import local_tasks
    assert local_tasks.resolve("hellaswag") is None

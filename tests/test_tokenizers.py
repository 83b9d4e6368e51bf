"""Tokenizer registry, the vocabulary padding rule and round trips of every backend that can be built offline."""
import json
import types

import pytest

from gpt_neox_b200.tokenizer import tokenizer as T


def _args(**kw):
    base = dict(rank=0, tokenizer_type="HFTokenizer", vocab_file=None, merge_file=None, dataset_impl="gpt2",
                synthetic_vocab_size=100, make_vocab_size_divisible_by=128, model_parallel_size=1, padded_vocab_size=None)
    base.update(kw)
    return types.SimpleNamespace(**base)


@pytest.mark.parametrize("n,div,mp,want", [(50277, 128, 1, 50304), (50277, 128, 2, 50432), (50304, 128, 1, 50304),
                                           (100, 128, 4, 512), (32000, 64, 1, 32000)])
def test_vocab_padding_rule(n, div, mp, want):
    assert T._vocab_size_with_padding(n, _args(make_vocab_size_divisible_by=div, model_parallel_size=mp, rank=1)) == want


def test_synthetic_tokenizer_is_selected_for_synthetic_data():
    a = _args(dataset_impl="synthetic", synthetic_vocab_size=1000)
    tok = T.build_tokenizer(a)
    assert isinstance(tok, T.SyntheticTokenizer) and tok.vocab_size == 1000 and a.padded_vocab_size == 1024
    assert tok.tokenize("3 17 x 1005") == [3, 17, 5] and tok.detokenize([3, 17]) == "3 17" and tok.eod == 0
    with pytest.raises(NotImplementedError):
        tok.cls


def _bpe_files(tmp_path):
    vocab = {"<|endoftext|>": 0, "<|padding|>": 1, "h": 2, "e": 3, "l": 4, "o": 5, "Ġ": 6, "w": 7, "r": 8, "d": 9,
             "he": 10, "ll": 11, "hell": 12, "hello": 13, "Ġw": 14}
    merges = ["h e", "l l", "he ll", "hell o", "Ġ w"]
    v, m = tmp_path / "vocab.json", tmp_path / "merges.txt"
    v.write_text(json.dumps(vocab))
    m.write_text("#version: 0.2\n" + "\n".join(merges) + "\n")
    return str(v), str(m), vocab


def test_gpt2_bpe_from_vocab_and_merges(tmp_path):
    v, m, vocab = _bpe_files(tmp_path)
    a = _args(tokenizer_type="GPT2BPETokenizer", vocab_file=v, merge_file=m)
    tok = T.build_tokenizer(a)
    assert tok.vocab_size == len(vocab) and a.padded_vocab_size == 128 and tok.eod == 0
    ids = tok.tokenize("hello world")
    assert ids == [13, 14, 5, 8, 4, 9] and tok.detokenize(ids) == "hello world"
    assert tok.inv_vocab[13] == "hello" and tok.vocab["Ġw"] == 14
    with pytest.raises(AssertionError):
        T.build_tokenizer(_args(tokenizer_type="GPT2BPETokenizer", vocab_file=v))          # merges missing


def test_hf_tokenizer_json(tmp_path):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    v, m, vocab = _bpe_files(tmp_path)
    t = Tokenizer(models.BPE.from_file(v, m))
    t.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    t.decoder = decoders.ByteLevel()
    path = str(tmp_path / "tok.json")
    t.save(path)
    tok = T.build_tokenizer(_args(tokenizer_type="HFTokenizer", vocab_file=path))
    assert tok.eod == 0 and tok.pad == 1 and tok.tokenize("hello") == [13]
    assert [e.ids for e in tok.tokenize_batch(["hello", "hell"])] == [[13], [12]]
    assert tok.detokenize([13, 14, 5, 8, 4, 9]) == "hello world"


def test_char_level_tokenizer():
    tok = T.build_tokenizer(_args(tokenizer_type="CharLevelTokenizer"))
    assert tok.vocab_size == 512 and tok.eod == 0
    ids = tok.tokenize("héllo")
    assert ids == list("héllo".encode("utf-8")) and tok.tokenize_batch(["a", "b"]) == [[97], [98]]
    assert tok.detokenize([104, 105, 7]) == "hi "                        # control byte clamps to a space
    with pytest.raises(NotImplementedError):
        tok.vocab


def test_sentencepiece_round_trip(tmp_path):
    spm = pytest.importorskip("sentencepiece")
    corpus = tmp_path / "c.txt"
    corpus.write_text("\n".join(["the quick brown fox jumps over the lazy dog"] * 50 +
                                ["pack my box with five dozen liquor jugs"] * 50))
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(tmp_path / "m"), vocab_size=40,
                                   user_defined_symbols=["<|endoftext|>"], minloglevel=2)
    tok = T.build_tokenizer(_args(tokenizer_type="SPMTokenizer", vocab_file=str(tmp_path / "m.model")))
    assert tok.vocab_size == 40 and tok.vocab["<|endoftext|>"] == tok.eod
    assert tok.detokenize(tok.tokenize("the lazy fox")) == "the lazy fox"


def test_unknown_type_is_rejected():
    with pytest.raises(NotImplementedError):
        T.build_tokenizer(_args(tokenizer_type="NoSuchTokenizer", vocab_file="x"))


def test_train_bpe_tokenizer_and_load_it(tmp_path):
    """Train on a small jsonl corpus (one file gzipped), load the result through HFTokenizer and round-trip text
    (reference: megatron/tokenizer/train_tokenizer.py)."""
    import gzip
    import json
    from types import SimpleNamespace
    from gpt_neox_b200.tokenizer import build_tokenizer
    from gpt_neox_b200.tokenizer.train_tokenizer import iter_documents, main, parse_args
    docs = [f"the quick brown fox number {i} jumps over the lazy dog" for i in range(200)]
    with open(tmp_path / "a.jsonl", "w") as f:
        for d in docs[:100]:
            f.write(json.dumps({"text": d}) + "\n")
    with gzip.open(tmp_path / "b.jsonl.gz", "wt") as f:
        for d in docs[100:]:
            f.write(json.dumps({"text": d, "meta": 1}) + "\n")
        f.write("\n" + json.dumps({"other": "no text"}) + "\n")
    assert sum(1 for _ in iter_documents(str(tmp_path))) == 200
    out = tmp_path / "tok" / "tokenizer.json"
    main(parse_args(["--json_input_dir", str(tmp_path), "--tokenizer_output_path", str(out), "-v", "400"]))
    args = SimpleNamespace(tokenizer_type="HFTokenizer", vocab_file=str(out), rank=0, make_vocab_size_divisible_by=128,
                           model_parallel_size=1)
    tok = build_tokenizer(args)
    assert 256 < tok.vocab_size <= 400
    ids = tok.tokenize("the quick brown fox")
    assert len(ids) < len("the quick brown fox") // 2 and tok.detokenize(ids).strip() == "the quick brown fox"
    assert tok.eod == tok.vocab["<|endoftext|>"] and tok.pad == tok.vocab["<|padding|>"]


def test_devutil_times_a_method():
    import torch
    from gpt_neox_b200.utils.devutil import Metric, monitor_method_wall_times
    m = Metric("linear forward")
    lin = torch.nn.Linear(8, 8)
    undo = monitor_method_wall_times(m, lin, "forward")
    for _ in range(5):
        lin(torch.randn(2, 8))
    undo()
    lin(torch.randn(2, 8))
    assert len(m.get_measurements()) == 5 and all(v >= 0 for v in m.measurements) and m.deciles().numel() == 10
    lines = []
    m.report(lines.append)
    assert "linear forward: n=5" in lines[0]

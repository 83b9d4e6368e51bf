"""Preprocessing tools: text -> indexed dataset round trip, label masks, chat masks, merge / count, launcher parsing."""
import json
import os

import numpy as np
import pytest

from common import ROOT  # noqa: F401  (puts the repo on sys.path)


def _write_jsonl(path, docs):
    with open(path, "w") as f:
        for d in docs:
            f.write(json.dumps({"text": d}) + "\n")


def test_preprocess_roundtrip_and_mask(tmp_path):
    from gpt_neox_b200.data import indexed_dataset, preprocess_data
    docs = ["hello world", "abc|def", "x"]
    src = tmp_path / "in.jsonl"
    _write_jsonl(src, docs)
    out = preprocess_data.main(["--input", str(src), "--output-prefix", str(tmp_path / "ds"), "--tokenizer-type",
                                "CharLevelTokenizer", "--append-eod", "--mask-before-token", str(ord("|"))])
    ds = indexed_dataset.make_dataset(out["text"], "mmap", skip_warmup=True)
    lab = indexed_dataset.make_dataset(out["text_label"], "mmap", skip_warmup=True)
    assert len(ds) == 3 and len(lab) == 3
    assert list(ds[0][:-1]) == [ord(c) for c in docs[0]]
    l1 = list(lab[1])
    assert l1[:4] == [-100] * 4 and l1[4:7] == [ord(c) for c in "def"]
    assert all(v == -100 for v in lab[0])                 # pattern absent: everything masked


def test_find_subsequence():
    from gpt_neox_b200.data.preprocess_data import find_subsequence
    assert find_subsequence([1, 2, 1, 2, 3], [1, 2, 3]) == 2
    assert find_subsequence([1, 2], [3]) == -1
    assert find_subsequence([5, 5, 5], [5, 5]) == 0


class _ChatTok:
    eos_token_id = 99

    def apply_chat_template(self, chat, add_generation_prompt=False):
        out = []
        for t in chat:
            out += [1 if t["role"] == "user" else 2] + [10 + len(t["content"])]
        return out + ([2] if add_generation_prompt else [])


def test_build_chat_masks_non_generation_roles():
    from gpt_neox_b200.data.preprocess_data import build_chat
    chat = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"}]
    toks, lab = build_chat(chat, "assistant", True, _ChatTok())
    assert toks[-1] == 99 and len(toks) == len(lab)
    assert lab[:3] == [-100, -100, -100]                  # user turn + generation prompt
    assert lab[-1] == 99 and lab[-2] == toks[-2]
    toks, lab = build_chat(chat, "assistant", True, _ChatTok(), for_rm=True)
    assert lab[-1] == 99 and set(lab[:-1]) == {-100} and len(toks) == len(lab)
    toks, lab = build_chat(chat, "assistant", False, _ChatTok())
    assert toks == lab


def test_merge_and_count(tmp_path):
    from gpt_neox_b200.data import dataset_tools, preprocess_data
    d = tmp_path / "parts"
    d.mkdir()
    for i, docs in enumerate((["aa", "bbb"], ["c"])):
        src = tmp_path / f"in{i}.jsonl"
        _write_jsonl(src, docs)
        preprocess_data.main(["--input", str(src), "--output-prefix", str(d / f"p{i}"), "--tokenizer-type",
                              "CharLevelTokenizer"])
    merged = dataset_tools.merge(str(d), str(tmp_path / "merged"))
    assert dataset_tools.token_count(merged) == 6


def test_launcher_hostfile_and_filters(tmp_path):
    from gpt_neox_b200 import launcher
    hf = tmp_path / "hosts"
    hf.write_text("n1 slots=4\nn2 slots=4\n")
    pool = launcher.fetch_hostfile(str(hf))
    assert pool == {"n1": 4, "n2": 4}
    assert launcher.parse_resource_filter(pool, include="n1:0,2") == {"n1": [0, 2]}
    assert launcher.parse_resource_filter(pool, exclude="n2@n1:3") == {"n1": [0, 1, 2]}
    with pytest.raises(ValueError):
        launcher.parse_resource_filter(pool, include="n3")
    args = launcher.parse_args(["--hostfile", str(hf), "--launcher", "pdsh", "train.py", "--x", "1"])
    cmd = launcher.build_multinode_cmd(args, launcher.parse_resource_filter(pool))
    assert cmd[0] == "pdsh" and "n1,n2" in cmd and "--node_rank=%n" in cmd[-1]


def test_launcher_runs_local_ranks(tmp_path):
    from gpt_neox_b200 import launcher
    script = tmp_path / "w.py"
    script.write_text("import os,sys\nopen(os.path.join(sys.argv[2], os.environ['RANK']), 'w')"
                      ".write(os.environ['WORLD_SIZE'] + ' ' + os.environ['MASTER_ADDR'])\n")
    rc = launcher.main(["--hostfile", "/nonexistent", "--num_gpus", "3", str(script), str(tmp_path)])
    assert rc == 0
    assert sorted(f for f in os.listdir(tmp_path) if f.isdigit()) == ["0", "1", "2"]
    assert (tmp_path / "1").read_text() == "3 127.0.0.1"
    bad = tmp_path / "bad.py"
    bad.write_text("import os,sys,time\nsys.exit(7) if os.environ['RANK']=='1' else time.sleep(30)\n")
    assert launcher.main(["--hostfile", "/nonexistent", "--num_gpus", "2", str(bad)]) == 7


def test_multinode_preprocessing_shares_and_merge(tmp_path, monkeypatch):
    """Three 'ranks' each tokenise their share of five input files; the merged parts hold every document once,
    in file order (reference: tools/datasets/multinode_prepare_data.sh)."""
    import json
    import numpy as np
    from gpt_neox_b200.data import dataset_tools, preprocess_data
    from gpt_neox_b200.data.indexed_dataset import make_dataset
    assert [preprocess_data.share_of(list(range(5)), r, 3) for r in range(3)] == [[0, 1], [2, 3], [4]]
    assert preprocess_data.process_share_from_env({"SLURM_PROCID": "2", "SLURM_NTASKS": "4"}) == (2, 4)
    assert preprocess_data.process_share_from_env({"RANK": "1", "WORLD_SIZE": "2", "SLURM_PROCID": "9",
                                                   "SLURM_NTASKS": "10"}) == (1, 2)
    assert preprocess_data.process_share_from_env({}) == (0, 1)
    paths = []
    for i in range(5):
        p = tmp_path / f"in{i}.jsonl"
        p.write_text("".join(json.dumps({"text": f"file {i} doc {j}"}) + "\n" for j in range(3)))
        paths.append(str(p))
    (tmp_path / "files.txt").write_text("\n".join(paths) + "\n")
    parts = tmp_path / "parts"
    parts.mkdir()
    for rank in range(3):
        monkeypatch.setenv("RANK", str(rank))
        monkeypatch.setenv("WORLD_SIZE", "3")
        preprocess_data.main(["--input-list", str(tmp_path / "files.txt"), "--tokenizer-type", "CharLevelTokenizer",
                              "--output-prefix", str(parts / "part"), "--append-eod"])
    assert sorted(f.name for f in parts.iterdir() if f.suffix == ".idx") == [f"part{r}_text_document.idx" for r in range(3)]
    dataset_tools.main(["merge", "--input", str(parts), "--output-prefix", str(tmp_path / "merged")])
    ds = make_dataset(str(tmp_path / "merged"), "mmap")
    assert len(ds) == 15
    texts = ["".join(chr(int(t)) for t in np.asarray(ds[i])[:-1]) for i in range(15)]
    assert texts == [f"file {i} doc {j}" for i in range(5) for j in range(3)]

"""Curriculum scheduler, gradient noise scale, weight server, pairwise / online datasets."""
import os
import pickle
import socket
import threading

import numpy as np
import pytest
import torch

from common import free_port


def test_curriculum_schedules():
    from gpt_neox_b200.engine.curriculum import CurriculumScheduler
    lin = CurriculumScheduler({"min_difficulty": 64, "max_difficulty": 1024, "schedule_type": "fixed_linear",
                               "schedule_config": {"total_curriculum_step": 100, "difficulty_step": 8}})
    assert lin.update_difficulty(0) == 64
    mid = lin.update_difficulty(50)
    assert 64 < mid < 1024 and mid % 8 == 0
    assert lin.update_difficulty(100) == 1024 and lin.update_difficulty(500) == 1024
    root = CurriculumScheduler({"min_difficulty": 64, "max_difficulty": 1024, "schedule_type": "fixed_root",
                                "schedule_config": {"total_curriculum_step": 100, "difficulty_step": 8,
                                                    "root_degree": 2}})
    assert root.get_difficulty(25) > lin.get_difficulty(25)
    disc = CurriculumScheduler({"min_difficulty": 1, "max_difficulty": 3, "schedule_type": "fixed_discrete",
                                "schedule_config": {"difficulty": [1, 2, 3], "max_step": [5, 10]}})
    assert [disc.get_difficulty(s) for s in (1, 5, 6, 10, 11)] == [1, 1, 2, 2, 3]


def test_gradient_noise_scale_recovers_known_ratio():
    """Gradients g = G + noise with known |G|^2 and tr(Sigma): the estimate approaches tr(Sigma)/|G|^2."""
    from gpt_neox_b200.gradient_noise_scale import GradientNoiseScale

    class _M:
        stored_gradients = None
    m = _M()
    torch.manual_seed(0)
    dim, bs, sigma = 4000, 8, 2.0
    G = torch.randn(dim) * 0.5
    gns = GradientNoiseScale(m, batch_size_small=bs, n_batches=5, beta=0.9)
    for _ in range(300):
        m.stored_gradients = [G + torch.randn(dim) * sigma / bs ** 0.5]
        gns.update()
    want = dim * sigma ** 2 / float(G.pow(2).sum())
    assert gns.noise_scale == pytest.approx(want, rel=0.15)


def test_weight_server_roundtrip_cpu():
    from gpt_neox_b200.models import weight_server
    model = torch.nn.Linear(4, 3)
    port = free_port()
    th = threading.Thread(target=weight_server.start_server, args=(model, [port]), kwargs={"accept_timeout_s": 20})
    th.start()
    import time
    got = None
    for _ in range(100):
        try:
            got = weight_server.receive_state_dict(port)
            break
        except ConnectionRefusedError:
            time.sleep(0.05)
    th.join(20)
    assert got is not None and set(got) == {"weight", "bias"}
    torch.testing.assert_close(got["weight"], model.weight.detach())


class _Idx:
    def __init__(self, docs, dtype=np.int64):
        self.docs = [np.asarray(d, dtype=dtype) for d in docs]
        self.sizes = np.array([len(d) for d in docs], dtype=np.int32)

    def get(self, i, offset=0, length=None):
        d = self.docs[i][offset:]
        return d if length is None else d[:length]


def test_pairwise_dataset_pairs_and_pads():
    from gpt_neox_b200.data.pairwise_dataset import PairwiseDataset
    pos = _Idx([[1, 2, 3], [4, 5, 6, 7, 8, 9, 10], [11]])
    neg = _Idx([[21, 22], [24], [31, 32, 33]])
    lab = _Idx([[-100, 2, 3], [4] * 7, [11]])
    ds = PairwiseDataset("t", "p", np.arange(3), pos, neg, num_samples=7, seq_length=4, seed=1,
                         pos_label_dataset=lab, neg_label_dataset=lab)
    assert len(ds) == 9
    seen = set()
    for i in range(3):
        s = ds[i]
        assert s["pos"].shape == (5,) and s["neg"].shape == (5,)
        doc = {1: 0, 4: 1, 11: 2}[int(s["pos"][0])]
        seen.add(doc)
        assert int(s["neg"][0]) == [21, 24, 31][doc]
        assert s["pos_label"][-1] in (-100, 4)
    assert seen == {0, 1, 2}
    ds2 = PairwiseDataset("t", "p", np.arange(3), pos, neg, num_samples=2, seq_length=4, seed=1, allow_chopped=False)
    assert set(ds2.order.tolist()) == {0, 2}


def test_online_dataset_fetches_and_centres():
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200.data.online_dataset import OnlineDataset
    mpu.destroy_model_parallel()
    mpu.initialize_model_parallel(1)
    port = free_port()
    payload = pickle.dumps([{"prefix": [1, 2], "completions": [[3], [4, 5]], "rewards": [1.0, 3.0]}])
    srv = socket.socket()
    srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    srv.bind(("127.0.0.1", port))
    srv.listen(1)

    def serve():
        c, _ = srv.accept()
        assert c.recv(64) == b"train"
        c.sendall(payload)
        c.close()
    th = threading.Thread(target=serve)
    th.start()
    ds = OnlineDataset(num_samples=4, seq_length=6, leave_one_out=True, dataserver_ips="127.0.0.1",
                       dataserver_ports=port)
    a, b = ds[0], ds[1]
    th.join(10)
    srv.close()
    assert a["text"].tolist() == [1, 2, 3, 0, 0, 0, 0] and a["label"].tolist()[:3] == [-100, -100, 3]
    assert a["reward"][0] == pytest.approx(-2.0) and b["reward"][0] == pytest.approx(2.0)
    assert b["raw_reward"][0] == pytest.approx(3.0)


def test_online_data_server_feeds_the_online_dataset(tmp_path):
    """The sampling server (toy sampler / reward, byte tokenizer) answers the OnlineDataset protocol."""
    import importlib.util
    import threading
    spec = importlib.util.spec_from_file_location(
        "online_data_server", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                           "post-training", "online_data_server.py"))
    ods = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ods)
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200.data.online_dataset import OnlineDataset
    srv = ods.OnlineDataServer(0, 1, ods.load_prompts(None), ods.ByteTokenizer(), ods.toy_sampler, ods.length_reward,
                               batch_per_rank=3, num_completions=4, max_completion_len=64, base_port=0)
    t = threading.Thread(target=srv.serve_once, daemon=True)
    t.start()
    mpu.destroy_model_parallel()
    ds = OnlineDataset(num_samples=100, seq_length=48, leave_one_out=True, dataserver_ports=srv.port)
    ds.global_rank = 0
    item = ds[0]
    t.join(timeout=20)
    groups = srv.make_batch("valid")
    srv.close()
    assert len(ds.online_batching_data) == 3 * 4 - 1                 # 3 prompts x 4 completions, one consumed
    assert item["text"].shape == (49,) and item["label"].shape == (49,)
    n_prefix = int((item["label"] == -100).nonzero()[0][-1]) + 1 if (item["label"] == -100).any() else 0
    assert n_prefix > 0 and (item["label"][:4] == -100).all()      # the prompt is masked out of the loss
    assert len(groups) == 3 and all(len(g["completions"]) == 4 and len(g["rewards"]) == 4 for g in groups)


def test_prepare_preference_data_writes_the_recipe_files(tmp_path):
    import importlib.util
    import json
    spec = importlib.util.spec_from_file_location(
        "prepare_preference_data", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                                "post-training", "prepare_preference_data.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    u = {"role": "user", "content": "q"}
    good = {"chosen": [u, {"role": "assistant", "content": "a"}], "rejected": [u, {"role": "assistant", "content": "b"}]}
    same = {"chosen": good["chosen"], "rejected": good["chosen"]}
    src = tmp_path / "in.jsonl"
    src.write_text("\n".join(json.dumps(r) for r in (good, same, good)) + "\n")
    mod.main(["--input", str(src), "--out", str(tmp_path / "data"), "--name", "t", "--split", "train"])
    rd = lambda p: [json.loads(l) for l in open(p)]
    assert len(rd(tmp_path / "data" / "pairwise" / "t_dpo_train.jsonl")) == 2
    assert rd(tmp_path / "data" / "sft" / "t_sft_train.jsonl")[0] == {"messages": good["chosen"]}
    kto = rd(tmp_path / "data" / "kto" / "t_kto_train.jsonl")
    assert [r["reward"] for r in kto] == [1, -1, 1, -1]


def _train_curriculum(rank, world, cfg, steps):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.models import utils as model_utils
    torch.set_num_threads(1)
    mpu.destroy_model_parallel()
    a = NeoXArgs.from_dict(dict(cfg, global_num_gpus=world, train_iters=steps))
    a.configure_distributed_args()
    a.build_tokenizer()
    seen, losses = [], []
    inner = model_utils.SequentialWrapper.forward

    def spy(self, forward_input, curriculum_seqlen=None, labels=None, neox_args=None):
        if self.training:
            seen.append(curriculum_seqlen)
        return inner(self, forward_input, curriculum_seqlen=curriculum_seqlen, labels=labels, neox_args=neox_args)
    model_utils.SequentialWrapper.forward = spy
    training.collect_loss_for_unit_test = lambda l: losses.append(float(l))
    try:
        training.pretrain(a)
    finally:
        model_utils.SequentialWrapper.forward = inner
    return {"seen": seen, "losses": losses}


def test_sequence_length_curriculum_reaches_the_model():
    """The engine hands the scheduled length to the model on every training step; the batch (and the loss side)
    are truncated to it, and it grows to the full length over `total_curriculum_step` steps."""
    from common import run_distributed, tiny_config
    cfg = tiny_config(use_cpu_initialization=True,
                      curriculum_learning={"enabled": True, "curriculum_type": "seqlen", "min_difficulty": 8,
                                           "max_difficulty": 32, "schedule_type": "fixed_linear",
                                           "schedule_config": {"total_curriculum_step": 4, "difficulty_step": 8}})
    r = run_distributed(_train_curriculum, 1, cfg, 6)[0]
    assert r["seen"][0] is not None and r["seen"][0] < 32
    assert r["seen"] == sorted(r["seen"]) and r["seen"][-1] == 32
    assert len(r["losses"]) == 6 and all(l == l for l in r["losses"])


def test_comet_experiment_gets_name_tags_and_parameters(monkeypatch):
    """``use_comet``: the experiment is created on rank 0 and receives the run's name, tags, extra fields and
    the non-default arguments (megatron/neox_arguments/arguments.py:190-212), here against a fake module."""
    import sys
    import types
    from common import tiny_config
    from gpt_neox_b200.config import NeoXArgs
    calls = {}

    class Experiment:
        def __init__(self, **kw):
            calls["init"] = kw

        def set_name(self, n):
            calls["name"] = n

        def add_tags(self, t):
            calls["tags"] = t

        def log_others(self, o):
            calls["others"] = o

        def __internal_api__log_parameters__(self, params, **kw):
            calls["params"] = params

    monkeypatch.setitem(sys.modules, "comet_ml", types.SimpleNamespace(Experiment=Experiment))
    a = NeoXArgs.from_dict(tiny_config(use_comet=True, comet_workspace="ws", comet_project="proj",
                                       comet_experiment_name="run-7", comet_tags=["a", "b"], comet_others={"k": 1}))
    a.rank = 0
    a.initialize_comet()
    assert calls["init"] == dict(workspace="ws", project_name="proj")
    assert calls["name"] == "run-7" and calls["tags"] == ["a", "b"] and calls["others"] == {"k": 1}
    assert calls["params"]["hidden_size"] == 64


def test_gather_slot_pool_is_deterministic():
    """Ranks agree on gather-buffer slots without communicating: the same call sequence gives the same slots, the lowest
    free index first; a reset frees everything; releasing a slot twice is an error."""
    pytest.importorskip("torch")
    from gpt_neox_b200.comm.symm import SlotPool
    a, b = SlotPool(4), SlotPool(4)
    seq = []
    for pool in (a, b):
        got = [pool.alloc(), pool.alloc(), pool.alloc()]
        pool.release(got[1])
        got.append(pool.alloc())            # the released slot comes back first
        got.append(pool.alloc())
        got.append(pool.alloc())            # exhausted
        seq.append(got)
    assert seq[0] == seq[1] == [0, 1, 2, 1, 3, None]
    with pytest.raises(ValueError):
        a.release(7)
    a.release(2)
    with pytest.raises(ValueError):
        a.release(2)
    a.reset()
    assert [a.alloc() for _ in range(5)] == [0, 1, 2, 3, None]


def test_bucketed_reduction_covers_every_element_exactly_once():
    """The ranges reduced from inside the backward pass plus the leftovers reduced at the step tile the flat gradient
    buffer without overlap: with a pre-division factor every element ends up divided exactly once."""
    torch = pytest.importorskip("torch")
    from gpt_neox_b200.engine.engine import FlatGroup
    ps = [torch.nn.Parameter(torch.randn(n)) for n in (100, 64, 7, 300)]
    g = FlatGroup([(p, 0.1 if i % 2 == 0 else 0.0) for i, p in enumerate(ps)], None, 1, 0, 1, torch.float32)
    g.predivide = 4.0
    g.main_grad.fill_(8.0)
    ranges = g.param_ranges([ps[1], ps[3]])
    assert all(lo % 64 == 0 and hi % 64 == 0 for lo, hi in ranges)
    assert sum(hi - lo for lo, hi in ranges) == 64 + 320            # alignment padding included
    for lo, hi in ranges:
        g.reduce_range_async(lo, hi)
    inside = torch.zeros(g.total, dtype=torch.bool)
    for lo, hi in ranges:
        inside[lo:hi] = True
    assert (g.main_grad[inside] == 2.0).all() and (g.main_grad[~inside] == 8.0).all()
    g.reduce_gradients()                                             # the leftovers, then the wait
    assert (g.main_grad == 2.0).all() and g._reduced == []
    g.main_grad.fill_(8.0)
    g.reduce_gradients()                                             # nothing bucketed this time: the single reduction
    assert (g.main_grad == 2.0).all()

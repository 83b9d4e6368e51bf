"""Multi-GPU checks (need >= 2 GPUs; each case is a torchrun child job): the fused NVLink
communication mode must reproduce the NCCL baseline's loss curve."""
import json
import os
import subprocess
import sys

import pytest
import torch

from common import free_port

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, *args, timeout=600, env=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(HERE, "mgpu", "train_losses.py"), *map(str, args)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=dict(os.environ, **(env or {})))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("LOSSES ")][-1]
    return json.loads(line[len("LOSSES "):])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp2_sp_matches_nccl_baseline():
    base = _run(2, "nccl_baseline", 2, 1, 6)
    fused = _run(2, "fused", 2, 1, 6)
    assert base["device_error"] == 0 and fused["device_error"] == 0
    assert fused["losses"] == pytest.approx(base["losses"], rel=2e-2)
    assert fused["losses"][-1] < fused["losses"][0]
    assert fused["gather_pool_slots"] > 0            # gathered activations stayed in pool slots (no copies)
    # the same run with every flag signal delayed by a pseudo-random time, and with the gather pool switched off:
    # neither the order in which peers arrive nor where the gathered operand is kept may change the numbers
    jit = _run(2, "fused", 2, 1, 6, env={"NEOX_COMM_JITTER_NS": "30000"})
    nopool = _run(2, "fused", 2, 1, 6, env={"NEOX_AG_POOL_GB": "0"})
    assert jit["device_error"] == 0 and nopool["gather_pool_slots"] == 0
    assert jit["losses"] == pytest.approx(fused["losses"], rel=2e-3)       # (fp32 atomics in the embedding backward
    assert nopool["losses"] == pytest.approx(fused["losses"], rel=2e-3)    # make runs differ in the last bits)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_dp2_zero1_trains():
    opt = {"optimizer": {"type": "Adam", "params": {"lr": 3e-4, "betas": [0.9, 0.95], "eps": 1e-8}}}
    two = _run(2, "fused", 1, 0, 10, json.dumps(opt))
    assert two["device_error"] == 0
    assert min(two["losses"][4:]) < two["losses"][0]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_zero_over_peer_memory_matches_nccl_zero():
    """ZeRO-1 with the gradient reduce-scatter / parameter all-gather running in place over peer memory
    reproduces the NCCL reduce-scatter / all-gather run."""
    opt = {"optimizer": {"type": "Adam", "params": {"lr": 3e-4, "betas": [0.9, 0.95], "eps": 1e-8}}}
    nccl = _run(2, "fused", 1, 0, 8, json.dumps(opt), env={"NEOX_ZERO_SYMM": "0"})
    symm = _run(2, "fused", 1, 0, 8, json.dumps(opt), env={"NEOX_ZERO_SYMM": "1"})
    assert symm["device_error"] == 0
    assert symm["losses"] == pytest.approx(nccl["losses"], rel=1e-2)
    assert symm.get("zero_symm") is True and nccl.get("zero_symm") is False


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("symm", ["1", "0"], ids=["peer_memory", "nccl"])
def test_gradient_reduction_overlapped_with_backward_matches_single_reduction(symm):
    """``overlap_comm``: one bucket per layer, reduced from a side stream (peer-memory kernel) or as an asynchronous
    NCCL all-reduce while the backward pass of the layers below runs; same loss curve as the one reduction at the
    step, no device error."""
    opt = {"optimizer": {"type": "Adam", "params": {"lr": 3e-4, "betas": [0.9, 0.95], "eps": 1e-8}},
           "gradient_clipping": 0.5}
    env = {"NEOX_ZERO_SYMM": symm}
    once = _run(2, "fused", 1, 0, 8, json.dumps(dict(opt, zero_optimization={"stage": 1, "overlap_comm": False})), env=env)
    over = _run(2, "fused", 1, 0, 8, json.dumps(dict(opt, zero_optimization={"stage": 1, "overlap_comm": True})), env=env)
    assert over["device_error"] == 0 and once["overlap_buckets"] == 0 and over["overlap_buckets"] >= 5
    assert over["zero_symm"] is (symm == "1")
    assert over["losses"] == pytest.approx(once["losses"], rel=2e-3)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pipeline_parallel_2_matches_single_stage():
    """1F1B over two pipeline stages (NCCL p2p) follows the loss curve of the unpipelined model."""
    opt = {"optimizer": {"type": "Adam", "params": {"lr": 3e-4, "betas": [0.9, 0.95], "eps": 1e-8}},
           "gradient_accumulation_steps": 4, "train_micro_batch_size_per_gpu": 2}
    one = _run(1, "fused", 1, 0, 6, json.dumps(dict(opt, pipe_parallel_size=0)))
    two = _run(2, "fused", 1, 0, 6, json.dumps(dict(opt, pipe_parallel_size=2)))
    assert two["device_error"] == 0
    assert two["losses"][0] == pytest.approx(one["losses"][0], rel=1e-2)         # same weights, same batch
    # bf16 runs on a steep part of the curve (8.5 -> 5.2 in six steps) drift apart by a few percent
    assert two["losses"] == pytest.approx(one["losses"], rel=8e-2)
    assert two["losses"][-1] < two["losses"][0] - 1.0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp2_without_sequence_parallel_matches_nccl_baseline():
    """Tensor parallel without sequence parallelism: the row-parallel all-reduce runs inside the GEMM kernel
    (reduce-scatter in the epilogue + owner broadcast); same loss curve as the NCCL all-reduce run."""
    seq = json.dumps({"gpt_j_residual": False})       # sequential residual: every row-parallel linear all-reduces
    base = _run(2, "nccl_baseline", 2, 0, 6, seq)
    fused = _run(2, "fused", 2, 0, 6, seq, env={"NEOX_FUSED_AR": "1"})
    assert fused["device_error"] == 0
    assert fused["fused_calls"]["ar_calls"] > 0                 # the fused path really ran
    assert fused["losses"] == pytest.approx(base["losses"], rel=2e-2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_2_over_peer_memory_matches_nccl_all_to_all():
    """dMoE with two expert-parallel ranks: dispatch / combine as peer loads inside the permutation kernels
    against the NCCL all-to-all path, same weights and batches."""
    moe = json.dumps({"moe_num_experts": 4, "moe_top_k": 2, "moe_expert_interval": 1, "gpt_j_residual": False,
                      "moe_expert_parallel_size": 2, "num_layers": 2, "attention_config": [[["flash"], 2]],
                      "optimizer": {"type": "Adam", "params": {"lr": 3e-4, "betas": [0.9, 0.95], "eps": 1e-8}}})
    nccl = _run(2, "fused", 1, 0, 6, moe, env={"NEOX_MOE_P2P": "0"})
    p2p = _run(2, "fused", 1, 0, 6, moe, env={"NEOX_MOE_P2P": "1"})
    assert p2p["device_error"] == 0
    assert p2p["moe_p2p"] is True and nccl["moe_p2p"] is False
    assert p2p["losses"] == pytest.approx(nccl["losses"], rel=2e-2)
    assert p2p["losses"][-1] < p2p["losses"][0]


def _run_op_checks(nproc, dtype="bf16", timeout=600, env=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(HERE, "mgpu", "op_checks.py"), dtype]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=dict(os.environ, **(env or {})))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("CHECKS ")][-1]
    return json.loads(line[len("CHECKS "):])


@pytest.mark.parametrize("ws,dtype", [(2, "bf16"), (2, "fp16"), (4, "bf16"), (8, "bf16")])
def test_communication_ops_match_fp32_references_over_nccl(ws, dtype):
    """ag_gemm / gemm_rs / gemm_ar, the peer-memory all-reduce / reduce-scatter / all-gather, the ZeRO workspace and
    the expert-parallel dispatch / combine, each against an fp32 PyTorch product or reduction gathered over NCCL
    (tests/mgpu/op_checks.py), on 2, 4 and 8 GPUs."""
    if torch.cuda.device_count() < ws:
        pytest.skip(f"needs {ws} GPUs")
    out = _run_op_checks(ws, dtype)
    assert out["ws"] == ws
    for name in ("ag_gemm_pair", "ag_gemm_single", "gemm_rs_pair", "gemm_rs_single", "all_reduce_h16", "all_reduce_f32",
                 "reduce_scatter_h16", "zero_rs_f32", "zero_ag_h16", "moe_ep"):
        assert name in out["checks"], (name, out)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_communication_ops_under_jitter_and_range_checks():
    """The same op-level checks with (a) a pseudo-random sleep of up to 20 us in front of every cross-rank signal,
    which permutes the arrival order of flags and data, and (b) the build whose communication kernels range-check
    every access into a symmetric workspace.  Results stay right, guard bands stay intact, no error is recorded."""
    out = _run_op_checks(2, "bf16", env={"NEOX_COMM_JITTER_NS": "20000"})
    assert "moe_ep" in out["checks"] and "guards_intact" in out["checks"]
    dbg = os.path.join(os.path.dirname(HERE), "gpt_neox_b200", "lib", "libneox_b200_dbg.so")
    if not os.path.exists(dbg):
        from gpt_neox_b200.build import build_cuda
        build_cuda(debug_bounds=True)
    out = _run_op_checks(2, "bf16", env={"NEOX_KERNEL_LIB": "debug", "NEOX_COMM_JITTER_NS": "5000"})
    assert out["checks"]["debug_bounds_build"] == 1.0 and "guards_intact" in out["checks"]

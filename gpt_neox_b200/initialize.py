"""Global initialisation (megatron/initialize.py:34-235): load the kernel library, start
torch.distributed (NCCL on GPUs, gloo on CPU), build the (pipe, data, model) topology and its groups,
seed every RNG (per-stage offset for pipeline stages, per-tensor-rank stream for model-parallel
regions), configure activation checkpointing, build the C++ dataset helpers."""
from __future__ import annotations

import datetime
import os
import random

import numpy as np
import torch
import torch.distributed as dist

from . import parallel as mpu
from .comm import collectives
from .parallel.random import configure_checkpointing, model_parallel_cuda_manual_seed
from .utils.common import print_rank_0


def initialize_megatron(neox_args, allow_no_cuda=False):
    """Returns None (eager init). ``allow_no_cuda`` permits CPU/gloo runs (tests, plumbing)."""
    use_cuda = torch.cuda.is_available() and neox_args.distributed_backend == "nccl"
    if not use_cuda and not allow_no_cuda and neox_args.distributed_backend == "nccl" and not torch.cuda.is_available():
        # CPU-only machine: fall back to gloo so that the same entry points work for plumbing runs
        neox_args.update_value("distributed_backend", "gloo")
    if use_cuda:
        from .ops import _lib
        _lib.lib()  # fail loudly now if the sm_100a kernel library is missing
    collectives.set_mode(neox_args.comm_mode if use_cuda else "nccl_baseline")
    _initialize_distributed(neox_args)
    if neox_args.rank == 0:
        print("> setting random seeds to {} ...".format(neox_args.seed), flush=True)
    _set_random_seed(neox_args.seed)
    setup_activation_checkpointing(neox_args)
    # dataset index helpers (C++): built once per node by local rank 0
    if neox_args.local_rank in (0, None):
        try:
            from .data.helpers import compile_helper
            compile_helper()
        except Exception as e:  # pragma: no cover
            print(f"WARNING: could not build the dataset helpers: {e}", flush=True)
    if dist.is_initialized():
        dist.barrier()
    _write_args_to_tensorboard(neox_args)
    return None


def setup_activation_checkpointing(neox_args):
    num_layers = neox_args.num_layers // neox_args.checkpoint_num_layers
    num_layers = num_layers if neox_args.num_layers % neox_args.checkpoint_num_layers == 0 else num_layers + 1
    configure_checkpointing(partition_activations=neox_args.partition_activations,
                            contiguous_checkpointing=neox_args.contiguous_checkpointing,
                            num_checkpoints=num_layers, checkpoint_in_cpu=neox_args.checkpoint_in_cpu,
                            synchronize=neox_args.synchronize_each_layer, profile=neox_args.profile_backward,
                            sequence_parallel=bool(neox_args.sequence_parallel))


def _initialize_distributed(neox_args):
    device_count = torch.cuda.device_count() if neox_args.distributed_backend == "nccl" else 0
    if dist.is_initialized():
        if neox_args.rank == 0:
            print("torch distributed is already initialized, skipping initialization ...", flush=True)
        neox_args.update_value("rank", dist.get_rank())
        neox_args.update_value("world_size", dist.get_world_size())
    else:
        if neox_args.rank is None:
            neox_args.configure_distributed_args()
        if neox_args.rank == 0:
            print("> initializing torch distributed ...", flush=True)
        if device_count > 0:
            device = neox_args.rank % device_count
            if neox_args.local_rank is not None:
                assert neox_args.local_rank == device, "expected local-rank to be the same as rank % device-count."
            else:
                neox_args.update_value("local_rank", device)
            torch.cuda.set_device(device)
        if (neox_args.world_size or 1) > 1 or "MASTER_ADDR" in os.environ:
            os.environ.setdefault("MASTER_ADDR", neox_args.master_addr or "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", str(neox_args.master_port or 29500))
            kwargs = {}
            if device_count > 0:
                kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
            dist.init_process_group(backend=neox_args.distributed_backend, rank=neox_args.rank,
                                    world_size=neox_args.world_size,
                                    timeout=datetime.timedelta(seconds=neox_args.collective_timeout_s), **kwargs)
    pp = neox_args.pipe_parallel_size if neox_args.pipe_parallel_size >= 1 else 1
    mp = neox_args.model_parallel_size if neox_args.model_parallel_size >= 1 else 1
    world = dist.get_world_size() if dist.is_initialized() else 1
    assert world % (pp * mp) == 0, f"world size {world} is not divisible by pp {pp} x mp {mp}"
    dp = world // (pp * mp)
    topo = mpu.PipeModelDataParallelTopology(num_pp=pp, num_mp=mp, num_dp=dp)
    # interior pipeline stages get a distinct seed so that dropout differs across stages
    rank = dist.get_rank() if dist.is_initialized() else 0
    stage = topo.get_coord(rank)["pipe"]
    if 0 < stage < pp - 1:
        offset = neox_args.seed + 1138
        neox_args.seed = offset + (stage * mp)
    if mpu.model_parallel_is_initialized():
        print("_initialize_distributed() model parallel is already initialized", flush=True)
    else:
        mpu.initialize_model_parallel(mp, topology=topo, fp32_allreduce=neox_args.fp32_allreduce,
                                      expert_parallel_size=neox_args.moe_expert_parallel_size)
    if collectives.get_mode() == "fused" and mp > 1 and torch.cuda.is_available():
        # symmetric workspace + peer mappings of the tensor-parallel group (collective call)
        from .comm import symm
        symm.init_group(mpu.get_model_parallel_group())
    if neox_args.rank in (0, None):
        print(f"> topology: pipe {pp} x data {dp} x model {mp} (expert-parallel "
              f"{mpu.get_expert_parallel_world_size()})", flush=True)


def _set_random_seed(seed):
    if seed is not None and seed > 0:
        random.seed(seed)
        np.random.seed(seed)
        torch.manual_seed(seed)
        model_parallel_cuda_manual_seed(seed)
    else:
        raise ValueError("Seed ({}) should be a positive integer.".format(seed))


def _write_args_to_tensorboard(neox_args):
    writer = getattr(neox_args, "tensorboard_writer", None)
    if writer:
        for name in sorted(neox_args.all_config):
            writer.add_text(name, str(getattr(neox_args, name)))

"""Process topology and communication groups ("mpu" state).

Rank layout follows the reference (megatron/initialize.py:166-170, megatron/mpu/initialize.py:54-168):
``rank = pipe * (data * model) + data_idx * model + model_idx`` — pipe outermost, model (tensor)
parallel innermost, so the ranks of one tensor-parallel group are neighbours on NVSwitch.
Groups: model (tensor) parallel, data parallel, pipe parallel, an "IO" group (tensor-rank 0 of the
first and last pipeline stage) and, new here, an expert-parallel group that is independent of the
tensor-parallel group (the reference ties experts to the tensor-parallel group,
megatron/model/moe.py:25-48): expert parallelism splits the data-parallel axis, so a 125M dMoE can
run 8 experts over 8 GPUs with tensor-parallel size 1.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ProcessTopology:
    """Cartesian rank grid with named axes, first axis outermost."""
    axes: tuple
    dims: tuple

    def world_size(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    def get_dim(self, axis: str) -> int:
        return self.dims[self.axes.index(axis)] if axis in self.axes else 1

    def get_rank(self, **coords) -> int:
        r = 0
        for a, d in zip(self.axes, self.dims):
            r = r * d + coords[a]
        return r

    def get_coord(self, rank: int) -> dict:
        out = {}
        for a, d in zip(reversed(self.axes), reversed(self.dims)):
            out[a] = rank % d
            rank //= d
        return out

    def get_axis_comm_lists(self, axis: str) -> list:
        """Rank lists of every group that varies only along ``axis``."""
        if axis not in self.axes:
            return []
        others = [a for a in self.axes if a != axis]
        lists = []
        for combo in itertools.product(*[range(self.get_dim(a)) for a in others]):
            fixed = dict(zip(others, combo))
            lists.append([self.get_rank(**fixed, **{axis: i}) for i in range(self.get_dim(axis))])
        return lists

    def filter_match(self, **filters) -> list:
        return [r for r in range(self.world_size())
                if all(self.get_coord(r)[k] == v for k, v in filters.items())]


def PipeModelDataParallelTopology(num_pp: int, num_mp: int, num_dp: int) -> ProcessTopology:
    return ProcessTopology(axes=("pipe", "data", "model"), dims=(num_pp, num_dp, num_mp))


class _State:
    def __init__(self):
        self.reset()

    def reset(self):
        self.initialized = False
        self.topology = None
        self.model_group = self.data_group = self.pipe_group = self.io_group = self.expert_group = None
        self.expert_data_group = None
        self.model_ranks = self.data_ranks = self.pipe_ranks = self.expert_ranks = None
        self.mp_size = self.dp_size = self.pp_size = self.ep_size = 1
        self.mp_rank = self.dp_rank = self.pp_rank = self.ep_rank = 0
        self.fp32_allreduce = False
        # test / single-process overrides
        self.override_mp_size = self.override_mp_rank = None


_S = _State()


def is_unitialized() -> bool:
    return not _S.initialized


def model_parallel_is_initialized() -> bool:
    return _S.initialized


def initialize_model_parallel(model_parallel_size: int, topology: ProcessTopology | None = None,
                              fp32_allreduce: bool = False, expert_parallel_size: int = 1,
                              pipe_parallel_size: int = 1):
    """Create all groups. Works without torch.distributed (single process: every group is trivial)."""
    _S.reset()
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    mp = min(max(model_parallel_size, 1), world)
    if topology is None:
        pp = max(pipe_parallel_size, 1)
        assert world % (mp * pp) == 0, f"world size {world} not divisible by mp {mp} x pp {pp}"
        topology = PipeModelDataParallelTopology(pp, mp, world // (mp * pp))
    assert topology.world_size() == world, f"topology {topology.dims} does not match world size {world}"
    _S.topology = topology
    _S.fp32_allreduce = fp32_allreduce
    coord = topology.get_coord(rank)
    _S.mp_size, _S.dp_size, _S.pp_size = topology.get_dim("model"), topology.get_dim("data"), topology.get_dim("pipe")
    _S.mp_rank, _S.dp_rank, _S.pp_rank = coord["model"], coord["data"], coord["pipe"]
    ep = max(expert_parallel_size, 1)
    assert _S.dp_size % ep == 0, f"expert_parallel_size {ep} must divide the data-parallel size {_S.dp_size}"
    _S.ep_size, _S.ep_rank = ep, _S.dp_rank % ep

    def make(lists):
        mine, mine_ranks = None, None
        for ranks in lists:
            g = dist.new_group(ranks) if dist.is_initialized() else None
            if rank in ranks:
                mine, mine_ranks = g, ranks
        return mine, mine_ranks

    _S.data_group, _S.data_ranks = make(topology.get_axis_comm_lists("data"))
    _S.pipe_group, _S.pipe_ranks = make(topology.get_axis_comm_lists("pipe"))
    # IO group: tensor-rank 0 of the first and last pipeline stage, per data-parallel index
    io_lists = []
    for d in range(_S.dp_size):
        first = topology.get_rank(pipe=0, data=d, model=0)
        last = topology.get_rank(pipe=_S.pp_size - 1, data=d, model=0)
        io_lists.append(sorted({first, last}))
    io_all = sorted({r for l in io_lists for r in l})
    _S.io_group = dist.new_group(io_all) if dist.is_initialized() else None
    _S.model_group, _S.model_ranks = make(topology.get_axis_comm_lists("model"))
    # expert groups: consecutive blocks of `ep` data-parallel indices; the complementary
    # "expert-data" group (same expert shard, different block) reduces expert gradients.
    ep_lists, epd_lists = [], []
    for ranks in topology.get_axis_comm_lists("data"):
        for b in range(0, len(ranks), ep):
            ep_lists.append(ranks[b:b + ep])
        for o in range(ep):
            epd_lists.append(ranks[o::ep])
    _S.expert_group, _S.expert_ranks = make(ep_lists)
    _S.expert_data_group, _ = make(epd_lists)
    _S.initialized = True


def destroy_model_parallel():
    _S.reset()


def get_topology():
    return _S.topology


def get_model_parallel_group():
    return _S.model_group


def get_data_parallel_group():
    return _S.data_group


def get_pipe_parallel_group():
    return _S.pipe_group


def get_io_parallel_group():
    return _S.io_group


def get_expert_parallel_group():
    return _S.expert_group


def get_expert_data_parallel_group():
    return _S.expert_data_group


def set_model_parallel_world_size(n):
    _S.override_mp_size = n


def set_model_parallel_rank(r):
    _S.override_mp_rank = r


def get_model_parallel_world_size() -> int:
    return _S.override_mp_size if _S.override_mp_size is not None else _S.mp_size


def get_model_parallel_rank() -> int:
    return _S.override_mp_rank if _S.override_mp_rank is not None else _S.mp_rank


def get_model_parallel_src_rank() -> int:
    """Global rank of tensor-rank 0 in this rank's tensor-parallel group."""
    return _S.model_ranks[0] if _S.model_ranks else 0


def get_model_parallel_ranks():
    return list(_S.model_ranks) if _S.model_ranks else [0]


# the same group under the names newer callers use (megatron/mpu/initialize.py:190-260)
get_tensor_model_parallel_group = get_model_parallel_group
get_tensor_model_parallel_world_size = get_model_parallel_world_size
get_tensor_model_parallel_rank = get_model_parallel_rank
get_tensor_model_parallel_src_rank = get_model_parallel_src_rank
set_tensor_model_parallel_world_size = set_model_parallel_world_size
set_tensor_model_parallel_rank = set_model_parallel_rank


def get_data_parallel_world_size() -> int:
    return _S.dp_size


def get_data_parallel_rank() -> int:
    return _S.dp_rank


def get_data_parallel_src_rank() -> int:
    return _S.data_ranks[0] if _S.data_ranks else 0


def get_data_parallel_ranks():
    return list(_S.data_ranks) if _S.data_ranks else [0]


def get_pipe_parallel_world_size() -> int:
    return _S.pp_size


def get_pipe_parallel_rank() -> int:
    return _S.pp_rank


def get_pipe_parallel_ranks():
    return list(_S.pipe_ranks) if _S.pipe_ranks else [0]


def get_expert_parallel_world_size() -> int:
    return _S.ep_size


def get_expert_parallel_rank() -> int:
    return _S.ep_rank


def get_expert_parallel_ranks():
    return list(_S.expert_ranks) if _S.expert_ranks else [0]


def get_fp32_allreduce() -> bool:
    return _S.fp32_allreduce


def get_expert_tokens_for_rank(routed_tokens: torch.Tensor, tokens_per_expert: torch.Tensor):
    """Rows of the expert-sorted token matrix that belong to this rank's experts
    (megatron/mpu/initialize.py:270-297), for the tensor-parallel = expert-parallel layout."""
    ws, r = get_model_parallel_world_size(), get_model_parallel_rank()
    per = tokens_per_expert.numel() // ws
    counts = tokens_per_expert.view(ws, per).sum(-1)
    start = int(counts[:r].sum())
    return routed_tokens[start:start + int(counts[r])]


def get_expert_token_counts_for_rank(tokens_per_expert: torch.Tensor):
    ws, r = get_model_parallel_world_size(), get_model_parallel_rank()
    per = tokens_per_expert.numel() // ws
    return tokens_per_expert[r * per:(r + 1) * per]

"""Broadcast of a batch of integer tensors from tensor-rank 0 to its tensor-parallel group
(megatron/mpu/data.py:79-120): sizes first, then one flat payload."""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import state as mpu

_MAX_DATA_DIM = 5


def _device():
    # GPU unless this is a CPU (gloo) run
    if torch.cuda.is_available() and (not dist.is_initialized() or dist.get_backend() == "nccl"):
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def broadcast_data(keys, data, datatype):
    """``data``: dict of tensors on tensor-rank 0 (anything elsewhere). Returns the same dict on every
    rank of the tensor-parallel group, on the compute device."""
    ws = mpu.get_model_parallel_world_size()
    dev = _device()
    if ws == 1 or not dist.is_initialized():
        return {k: data[k].to(dev, non_blocking=True) for k in keys}
    src, group = mpu.get_model_parallel_src_rank(), mpu.get_model_parallel_group()
    is_src = mpu.get_model_parallel_rank() == 0
    sizes = torch.zeros(_MAX_DATA_DIM * len(keys), dtype=torch.int64)
    if is_src:
        for i, k in enumerate(keys):
            assert data[k].dim() < _MAX_DATA_DIM, "you should increase MAX_DATA_DIM"
            for j, s in enumerate(data[k].shape):
                sizes[i * _MAX_DATA_DIM + j] = s
    sizes = sizes.to(dev)
    dist.broadcast(sizes, src, group=group)
    sizes = sizes.cpu().tolist()
    shapes, total = {}, 0
    for i, k in enumerate(keys):
        shp = [s for s in sizes[i * _MAX_DATA_DIM:(i + 1) * _MAX_DATA_DIM] if s > 0]
        shapes[k] = shp
        n = 1
        for s in shp:
            n *= s
        total += n
    if is_src:
        for k in keys:
            assert data[k].dtype == datatype, f"{k} has data type {data[k].dtype} which is different than {datatype}"
        flat = torch.cat([data[k].contiguous().view(-1) for k in keys]).to(dev)
    else:
        flat = torch.empty(total, dtype=datatype, device=dev)
    dist.broadcast(flat, src, group=group)
    out, off = {}, 0
    for k in keys:
        n = 1
        for s in shapes[k]:
            n *= s
        out[k] = flat.narrow(0, off, n).view(shapes[k])
        off += n
    return out

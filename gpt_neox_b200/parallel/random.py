"""Model-parallel RNG streams and activation checkpointing.

The reference re-exports DeepSpeed's tracker and ``checkpoint`` (megatron/mpu/random.py:18-37);
this is a self-contained equivalent: a named-stream RNG tracker (dropout inside tensor-parallel
regions draws from a per-tensor-rank stream, everything else from the default stream shared by
the tensor-parallel group) and a recompute-in-backward ``checkpoint`` that replays both the default
and the tracked RNG states.  Works on CPU (gloo tests) and CUDA.
"""
from __future__ import annotations

import contextlib

import torch

from . import state as mpu

_MODEL_PARALLEL_RNG = "model-parallel-rng"


def _get_state(device_cuda: bool):
    return torch.cuda.get_rng_state() if device_cuda else torch.get_rng_state()


def _set_state(state, device_cuda: bool):
    if device_cuda:
        torch.cuda.set_rng_state(state)
    else:
        torch.set_rng_state(state)


class RNGStatesTracker:
    """Named RNG states; ``fork(name)`` runs a block under that state and saves it back."""

    def __init__(self):
        self.states_ = {}
        self.seeds_ = set()

    def reset(self):
        self.states_ = {}
        self.seeds_ = set()

    def get_states(self):
        return {k: v.clone() for k, v in self.states_.items()}

    def set_states(self, states):
        self.states_ = states

    def add(self, name, seed):
        if seed in self.seeds_:
            raise Exception(f"seed {seed} already exists")
        if name in self.states_:
            raise Exception(f"rng state {name} already exists")
        self.seeds_.add(seed)
        cuda = torch.cuda.is_available()
        orig = _get_state(cuda)
        if cuda:
            torch.cuda.manual_seed(seed)
        else:
            torch.manual_seed(seed)
        self.states_[name] = _get_state(cuda)
        _set_state(orig, cuda)

    @contextlib.contextmanager
    def fork(self, name=_MODEL_PARALLEL_RNG):
        if name not in self.states_:
            # single-process / uninitialised use: behave like the default stream
            yield
            return
        cuda = torch.cuda.is_available()
        orig = _get_state(cuda)
        _set_state(self.states_[name], cuda)
        try:
            yield
        finally:
            self.states_[name] = _get_state(cuda)
            _set_state(orig, cuda)


_TRACKER = RNGStatesTracker()


def get_cuda_rng_tracker():
    return _TRACKER


def model_parallel_cuda_manual_seed(seed: int):
    """Default stream: ``seed`` on every rank of a tensor-parallel group (so non-parallel regions
    agree); tracked model-parallel stream: ``seed + 2718 + tensor_rank``."""
    offset = seed + 2718
    mp_seed = offset + mpu.get_model_parallel_rank()
    _TRACKER.reset()
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)
    _TRACKER.add(_MODEL_PARALLEL_RNG, mp_seed)


def _kernel_dropout_counters(new=None):
    """The call counters from which the dropout kernels derive their seeds (attention dropout, bias-dropout-add);
    returns the current pair and, if given, installs ``new``.  Part of the random state a recompute replays."""
    from ..ops import attention, elementwise
    old = (attention._DROPOUT_CALLS["n"], elementwise._DROPOUT_OFFSET["n"])
    if new is not None:
        attention._DROPOUT_CALLS["n"], elementwise._DROPOUT_OFFSET["n"] = new
    return old


class _CheckpointFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_function, n_tensor, *args):
        ctx.run_function = run_function
        ctx.cuda = any(isinstance(a, torch.Tensor) and a.is_cuda for a in args)
        ctx.cpu_state = torch.get_rng_state()
        ctx.cuda_state = torch.cuda.get_rng_state() if ctx.cuda else None
        ctx.tracker_states = _TRACKER.get_states()
        ctx.kernel_dropout = _kernel_dropout_counters()
        with torch.no_grad():
            outputs = run_function(*args)
        ctx.inputs = tuple(_stash(a) for a in args)
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        bwd_cpu = torch.get_rng_state()
        bwd_cuda = torch.cuda.get_rng_state() if ctx.cuda else None
        bwd_tracker = _TRACKER.get_states()
        torch.set_rng_state(ctx.cpu_state)
        if ctx.cuda:
            torch.cuda.set_rng_state(ctx.cuda_state)
        _TRACKER.set_states(ctx.tracker_states)
        bwd_kernel_dropout = _kernel_dropout_counters(ctx.kernel_dropout)    # replay the kernels' own dropout masks
        detached = tuple(_unstash(a) for a in ctx.inputs)
        if _CKPT_CONFIG["synchronize"] and ctx.cuda:
            torch.cuda.synchronize()
        with torch.enable_grad():
            outputs = ctx.run_function(*detached)
        torch.set_rng_state(bwd_cpu)
        if ctx.cuda:
            torch.cuda.set_rng_state(bwd_cuda)
        _TRACKER.set_states(bwd_tracker)
        _kernel_dropout_counters(bwd_kernel_dropout)
        if isinstance(outputs, torch.Tensor):
            outputs = (outputs,)
        pairs = [(o, g) for o, g in zip(outputs, grads) if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        in_grads = tuple(a.grad if isinstance(a, torch.Tensor) else None for a in detached)
        return (None, None) + in_grads


_CKPT_CONFIG = {"partition_activations": False, "contiguous": False, "cpu": False, "num_layers": None,
                "synchronize": False, "profile": False, "sequence_parallel": False}


def _stash(a):
    """What a checkpointed region keeps of one argument until backward.  ``partition_activations``: a
    floating-point tensor that is replicated over the tensor-parallel group (no sequence parallelism) is kept
    as this rank's 1/tp slice and re-assembled by an all-gather in backward.  ``checkpoint_in_cpu``: the kept
    tensor (slice) waits in host memory."""
    if not isinstance(a, torch.Tensor):
        return ("raw", a)
    from . import state as mpu
    cfg = _CKPT_CONFIG
    tp = mpu.get_model_parallel_world_size()
    keep, kind = a.detach(), "full"
    if cfg["partition_activations"] and tp > 1 and not cfg["sequence_parallel"] and a.is_floating_point() \
            and a.numel() > 0 and a.numel() % tp == 0:
        keep = keep.reshape(-1).chunk(tp)[mpu.get_model_parallel_rank()].clone()
        kind = "slice"
    if cfg["cpu"] and keep.device.type != "cpu":
        keep = keep.to("cpu", non_blocking=True)
    return (kind, keep, a.shape, a.requires_grad, a.device)


def _unstash(entry):
    if entry[0] == "raw":
        return entry[1]
    kind, keep, shape, requires_grad, device = entry
    if keep.device != device:
        keep = keep.to(device, non_blocking=True)
    if kind == "slice":
        from . import state as mpu
        from ..comm import collectives
        keep = collectives.all_gather_dim(keep, 0, mpu.get_model_parallel_group()).view(shape)
    return keep.detach().requires_grad_(requires_grad)


def configure_checkpointing(partition_activations=False, contiguous_checkpointing=False, num_checkpoints=None,
                            checkpoint_in_cpu=False, synchronize=False, profile=False, sequence_parallel=False):
    """Counterpart of ``deepspeed.checkpointing.configure`` (megatron/initialize.py:103-118). Under
    sequence parallelism the layer inputs are already sharded over the tensor-parallel group, which
    is what ``partition_activations`` buys in the reference."""
    _CKPT_CONFIG.update(partition_activations=partition_activations, contiguous=contiguous_checkpointing,
                        num_layers=num_checkpoints, cpu=checkpoint_in_cpu, synchronize=synchronize,
                        profile=profile, sequence_parallel=sequence_parallel)


def checkpoint(function, *args):
    """Run ``function(*args)`` without storing its intermediates; recompute them in backward."""
    return _CheckpointFunction.apply(function, len(args), *args)

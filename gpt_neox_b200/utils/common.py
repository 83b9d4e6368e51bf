"""General utilities (megatron/utils.py): rank-0 printing, left-to-right masks and position ids,
loss reduction, device-timed timers, overflow monitor, character counter, wandb init, local-rank
helpers and ``setup_for_inference_or_eval``."""
from __future__ import annotations

import os
import socket
import sys
import time
from collections import deque
from typing import Dict, List

import torch
import torch.distributed as dist


def is_local_main():
    return local_rank() == 0


def local_rank():
    lr = os.environ.get("LOCAL_RANK")
    return 0 if lr is None else int(lr)


def is_mp_rank_0():
    from .. import parallel as mpu
    return mpu.get_model_parallel_rank() == 0


def get_rank():
    return dist.get_rank() if dist.is_initialized() else 0


def is_bnb_available() -> bool:
    """True if the bitsandbytes package can be imported."""
    import importlib.util
    return importlib.util.find_spec("bitsandbytes") is not None


def get_total_params(model) -> int:
    """Parameters of the whole model: each model-parallel shard counted once (data-parallel rank 0 of every
    shard contributes), summed over all ranks (megatron/utils.py:403-419)."""
    from .. import parallel as mpu
    params = 0
    if mpu.get_data_parallel_rank() == 0:
        params = sum(p.nelement() for p in model.parameters())
        print(f" > number of parameters on model parallel rank {mpu.get_model_parallel_rank()}: {params}", flush=True)
    if torch.distributed.is_initialized():
        dev = next(model.parameters()).device
        t = torch.tensor([params], dtype=torch.int64, device=dev)
        torch.distributed.all_reduce(t)
        params = int(t.item())
    return params


def make_viewless_tensor(inp, requires_grad=None, keep_graph=True):
    """A tensor that shares ``inp``'s data but is not a view of another tensor (``._base is None``), so that
    its storage can be released or replaced independently (megatron/utils.py make_viewless_tensor).  With
    ``keep_graph`` the result stays connected to the autograd graph."""
    if inp._base is None:
        return inp
    if keep_graph:
        return _MakeViewless.apply(inp, inp.requires_grad if requires_grad is None else requires_grad)
    out = torch.empty((1,), dtype=inp.dtype, device=inp.device, requires_grad=bool(requires_grad))
    out.data = inp.data
    return out


class _MakeViewless(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, requires_grad):
        out = torch.empty((1,), dtype=inp.dtype, device=inp.device)
        out.data = inp.data
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad, None


MakeViewlessTensor = _MakeViewless


def print_rank_0(*message):
    if get_rank() == 0:
        print(*message, flush=True)


def human_readable_flops(num) -> str:
    for unit in ["", "KFLOPS", "MFLOPS", "GFLOPS", "TFLOPS", "PFLOPS", "EFLOPS", "ZFLOPS"]:
        if abs(num) < 1000.0:
            return "%3.1f%s" % (num, unit)
        num /= 1000.0
    return "%.1f%s" % (num, "Yi")


def reduce_losses(losses):
    """Mean over the world of a list of scalar losses (megatron/utils.py:41-49)."""
    reduced = torch.cat([l.clone().detach().view(1) for l in losses])
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(reduced)
        reduced = reduced / dist.get_world_size()
    return reduced


def report_memory(name):
    if not torch.cuda.is_available():
        return
    mb = 1024.0 * 1024.0
    s = (f"{name} memory (MB) | allocated: {torch.cuda.memory_allocated() / mb} | max allocated: "
         f"{torch.cuda.max_memory_allocated() / mb} | reserved: {torch.cuda.memory_reserved() / mb} | "
         f"max reserved: {torch.cuda.max_memory_reserved() / mb}")
    print_rank_0(s)


def get_attn_mask(seq_length, device, sliding_window_width):
    """Boolean [1,1,s,s] mask, True = masked (upper triangle, plus the band below the window)."""
    mask = torch.tril(torch.ones((1, seq_length, seq_length), device=device)).view(1, 1, seq_length, seq_length)
    if sliding_window_width is not None:
        mask = torch.triu(mask, diagonal=-sliding_window_width)
    return mask < 0.5


def get_ltor_masks_and_position_ids(data, eod_token, eod_mask_loss=False, sliding_window_width=None,
                                    build_attention_mask=True):
    """-> (attention_mask or None, loss_mask, position_ids). The dense mask is only built on request:
    the flash path never reads it (the reference builds it every step, megatron/utils.py:67-80)."""
    batch_size, seq_length = data.size()
    attention_mask = get_attn_mask(seq_length, data.device, sliding_window_width) if build_attention_mask else None
    loss_mask = torch.ones(data.size(), dtype=torch.float, device=data.device)
    if eod_mask_loss:
        loss_mask[data == eod_token] = 0.0
    position_ids = torch.arange(seq_length, dtype=torch.long, device=data.device).unsqueeze(0).expand_as(data)
    return attention_mask, loss_mask, position_ids


class Timer:
    """Device-timed when CUDA is present: ``stop`` records an event and the elapsed time is read lazily,
    so timing does not synchronise the stream on every call."""

    def __init__(self, name):
        self.name_ = name
        self.elapsed_ = 0.0
        self.started_ = False
        self._pending = []
        self._start_ev = None
        self.start_time = time.time()
        self._cuda = torch.cuda.is_available()

    def start(self):
        assert not self.started_, "timer has already been started"
        if self._cuda:
            self._start_ev = torch.cuda.Event(enable_timing=True)
            self._start_ev.record()
        self.start_time = time.time()
        self.started_ = True

    def stop(self):
        assert self.started_, "timer is not started"
        if self._cuda:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self._pending.append((self._start_ev, end))
        else:
            self.elapsed_ += time.time() - self.start_time
        self.started_ = False

    def _drain(self):
        if self._pending:
            self._pending[-1][1].synchronize()
            for s, e in self._pending:
                self.elapsed_ += s.elapsed_time(e) / 1000.0
            self._pending = []

    def reset(self):
        self._drain()
        self.elapsed_ = 0.0
        self.started_ = False

    def elapsed(self, reset=True):
        started = self.started_
        if started:
            self.stop()
        self._drain()
        e = self.elapsed_
        if reset:
            self.reset()
        if started:
            self.start()
        return e


class Timers:
    def __init__(self, use_wandb=False, tensorboard_writer=None, comet_experiment=None):
        self.timers: Dict[str, Timer] = {}
        self.use_wandb, self.tensorboard_writer, self.comet_experiment = use_wandb, tensorboard_writer, comet_experiment

    def __call__(self, name):
        if name not in self.timers:
            self.timers[name] = Timer(name)
        return self.timers[name]

    def write(self, names, iteration, normalizer=1.0, reset=False):
        assert normalizer > 0.0
        from ..obs.logging import tb_wandb_log
        for name in names:
            value = self.timers[name].elapsed(reset=reset) / normalizer
            tb_wandb_log(f"timers/{name}", value, iteration, use_wandb=self.use_wandb,
                         tensorboard_writer=self.tensorboard_writer, comet_experiment=self.comet_experiment)

    def log(self, names, normalizer=1.0, reset=True):
        assert normalizer > 0.0
        s = "time (ms)"
        for name in names:
            s += " | {}: {:.2f}".format(name, self.timers[name].elapsed(reset=reset) * 1000.0 / normalizer)
        print_rank_0(s)


class OverflowMonitor:
    """Raises after ``n`` consecutive skipped (overflowed) fp16 steps."""

    def __init__(self, optimizer, n=50):
        self.optimizer = optimizer
        self.n = n
        self.history = deque(maxlen=n)

    def check(self, skipped):
        self.history.append(skipped)
        if getattr(self.optimizer, "overflow", False) and len(self.history) == self.n and all(self.history):
            raise Exception(f"Skipped {self.n} iterations in a row due to Overflow - Exiting training.")


class CharCounter:
    """Wraps a data iterator and counts characters / tokens for character-level perplexity."""

    def __init__(self, data_iterator, tokenizer):
        self.tokenizer, self.data_iterator = tokenizer, data_iterator
        self.char_count = 0
        self.batch_count = 0
        self.token_count = 0
        self.total_time = 0

    def tokens_per_char(self):
        return self.token_count / self.char_count

    def __iter__(self):
        return self

    def __next__(self):
        start = time.time()
        batch = self.data_iterator.__next__()
        for b in batch["text"]:
            self.token_count += len(b)
            self.char_count += len(self.tokenizer.detokenize(b.tolist()))
        self.batch_count += 1
        self.total_time += time.time() - start
        return batch


def get_wandb_api_key(neox_args=None):
    if "WANDB_LOCAL" in os.environ:
        return "LOCAL"
    if "WANDB_API_KEY" in os.environ:
        return os.environ["WANDB_API_KEY"]
    try:
        import requests
        host = getattr(neox_args, "wandb_host", "https://api.wandb.ai")
        wandb_token = requests.utils.get_netrc_auth(host)
        if wandb_token is not None:
            return wandb_token[1]
    except Exception:
        pass
    return None


def init_wandb(neox_args):
    if neox_args.use_wandb is False:
        return
    if not neox_args.wandb_init_all_ranks:
        use = is_local_main() and (get_wandb_api_key(neox_args) is not None)
        neox_args.update_value("use_wandb", use)
    if neox_args.use_wandb:
        try:
            import wandb
            group_name = neox_args.wandb_group
            name = f"{socket.gethostname()}-{local_rank()}" if group_name else None
            wandb.init(project=neox_args.wandb_project, group=group_name, name=name, save_code=False,
                       force=False, entity=neox_args.wandb_team)
            wandb.config.update(neox_args.all_config)
        except Exception as e:
            neox_args.update_value("use_wandb", False)
            print(e)
            print("Skipping wandb. Execute `wandb login` on local or main node machine to enable.", flush=True)


def obtain_resource_pool(hostfile_path, include_arg, exclude_arg):
    from ..config.arguments import _parse_hostfile
    return _parse_hostfile(hostfile_path, include_arg, exclude_arg)


def natural_sort(l):
    import re
    convert = lambda text: int(text) if text.isdigit() else text.lower()
    return sorted(l, key=lambda key: [convert(c) for c in re.split("([0-9]+)", key)])


def ddb(rank=0):
    """Distributed debugger: breakpoint on one rank, barrier on the others."""
    if get_rank() == rank:
        from pdb import Pdb
        Pdb(skip=["torch.distributed.*"]).set_trace(sys._getframe().f_back)
    if dist.is_initialized():
        dist.barrier()


def setup_for_inference_or_eval(use_cache=True, overwrite_values=None, input_args=None):
    """Build args + model for generation / evaluation (megatron/utils.py:422-470): no activation
    checkpointing, no optimizer, ZeRO off, weights loaded from ``load``."""
    from ..config import NeoXArgs
    from ..initialize import initialize_megatron
    from ..training import setup_model_and_optimizer

    _overwrite = {"checkpoint_activations": False, "partition_activations": False, "no_load_optim": True,
                  "optimizer": None, "zero_optimization": None}
    if overwrite_values:
        _overwrite.update(overwrite_values)
    neox_args = NeoXArgs.consume_neox_args(overwrite_values=_overwrite, input_args=input_args)
    neox_args.configure_distributed_args()
    neox_args.build_tokenizer()
    if neox_args.load is None:
        raise ValueError("`load` parameter must be supplied to load a model`")
    initialize_megatron(neox_args)
    model, _, _, _ = setup_model_and_optimizer(neox_args=neox_args, use_cache=use_cache,
                                               iteration=neox_args.iteration)
    print_rank_0("Finished loading model")
    model.module.inference_mode(use_cache=use_cache)
    return model, neox_args


def mup_weights_reinit(neox_args, model):
    def has_method(o, name):
        return callable(getattr(o, name, None))
    for layer in model.modules():
        if has_method(layer, "mup_reinitialize_weights"):
            layer.mup_reinitialize_weights(neox_args)

"""Logging and metrics (megatron/logging.py): stdout/stderr tee, the model-FLOPs formulas, the
training log line with throughput / TFLOP/s / MFU, and the single funnel to TensorBoard, W&B and
Comet."""
from __future__ import annotations

import math
import os
import socket
import sys

import torch

from .. import parallel as mpu
from ..utils.common import Timers, get_rank, human_readable_flops, print_rank_0, report_memory


class Tee:
    """Duplicate stdout or stderr into a file."""

    def __init__(self, file, err: bool = False):
        self.err = err
        self.std = sys.stderr if err else sys.stdout
        if isinstance(file, str):
            try:
                os.makedirs(os.path.dirname(file), exist_ok=True)
                self.file = open(file, "w")
            except IOError:
                self.file = None
        else:
            self.file = file
        if err:
            sys.stderr = self
        else:
            sys.stdout = self

    def __del__(self):
        if sys is None:
            return
        if self.err:
            sys.stderr = self.std
        else:
            sys.stdout = self.std
        if getattr(self, "file", None):
            self.file.close()

    def write(self, data):
        try:
            self.std.write(data)
        except OSError:
            pass
        if self.file:
            try:
                self.file.write(data)
            except OSError:
                pass

    def flush(self):
        try:
            self.std.flush()
            if self.file:
                self.file.flush()
        except OSError:
            pass


def enable_logging(neox_args):
    if neox_args.log_dir:
        hostname = socket.gethostname()
        Tee(os.path.join(neox_args.log_dir, f"{hostname}_stdout.txt"), err=False)
        Tee(os.path.join(neox_args.log_dir, f"{hostname}_stderr.txt"), err=True)


def get_actual_flops(neox_args, iter_time_s) -> float:
    """FLOP/s per GPU actually executed (counts activation recomputation): factor 4 with
    ``checkpoint_activations`` else 3 (megatron/logging.py:83-160)."""
    return get_flops(neox_args, iter_time_s, use_checkpointing_factor=True)


def get_forward_backward_flops(neox_args, iter_time_s) -> float:
    """Model FLOP/s per GPU (factor 3 always; the MFU numerator)."""
    return get_flops(neox_args, iter_time_s, use_checkpointing_factor=False)


def get_flops(neox_args, iter_time_s, use_checkpointing_factor=True) -> float:
    world_size = torch.distributed.get_world_size() if torch.distributed.is_initialized() else 1
    vocab_size = neox_args.padded_vocab_size
    batch_size = neox_args.train_batch_size
    seq_len = neox_args.seq_length
    hidden_size = neox_args.hidden_size
    num_layers = neox_args.num_layers
    ckpt = 4 if (neox_args.checkpoint_activations and use_checkpointing_factor) else 3
    kinds = neox_args.attention_config or []
    if "rwkv" in kinds:
        num_heads = neox_args.num_attention_heads
        flops = batch_size * seq_len * (78 * hidden_size * hidden_size * num_layers
                                        + 84 * hidden_size * num_layers
                                        + 16 * hidden_size
                                        + 12 * hidden_size * vocab_size
                                        + 18 * hidden_size * hidden_size * num_layers / num_heads)
    elif "mamba" in kinds:
        d_inner = 2 * hidden_size
        d_state, d_conv, dt_rank = 16, 4, math.ceil(hidden_size / 16)
        per_layer = (2 * hidden_size * 2 * d_inner + 2 * d_inner * d_conv + 2 * d_inner * (dt_rank + 2 * d_state)
                     + 2 * dt_rank * d_inner + 9 * d_inner * d_state + 2 * d_inner * hidden_size)
        flops = ckpt * batch_size * seq_len * (num_layers * per_layer + 2 * hidden_size * vocab_size)
    else:
        flops = (24 * ckpt * batch_size * seq_len * num_layers * hidden_size ** 2
                 * (1.0 + seq_len / (6.0 * hidden_size) + vocab_size / (16.0 * num_layers * hidden_size)))
    return flops / (iter_time_s * world_size)


class CsvMonitor:
    """``csv_monitor: {enabled, output_path, job_name}``: one ``<key>.csv`` of ``step,value`` rows per scalar
    under ``output_path/job_name`` (what the reference gets from the DeepSpeed monitor,
    megatron/neox_arguments/deepspeed_args.py csv_monitor)."""

    def __init__(self, output_path="", job_name="gpt-neox-b200"):
        self.dir = os.path.join(output_path or "csv_monitor", job_name or "gpt-neox-b200")
        os.makedirs(self.dir, exist_ok=True)
        self.seen = set()

    def write(self, key, value, step):
        name = key.replace("/", "_").replace(" ", "_")
        path = os.path.join(self.dir, name + ".csv")
        new = name not in self.seen and not os.path.exists(path)
        self.seen.add(name)
        with open(path, "a") as f:
            if new:
                f.write(f"step,{name}\n")
            f.write(f"{int(step)},{float(value)}\n")


_CSV = {"monitor": None}


def configure_csv_monitor(neox_args):
    cfg = getattr(neox_args, "csv_monitor", None) or {}
    _CSV["monitor"] = CsvMonitor(cfg.get("output_path", ""), cfg.get("job_name", "")) \
        if cfg.get("enabled") and get_rank() == 0 else None
    return _CSV["monitor"]


def tb_wandb_log(key, value, iteration_no, use_wandb, tensorboard_writer=None, comet_experiment=None,
                 all_ranks=False):
    """Write one scalar to every configured sink (rank 0 unless ``all_ranks``)."""
    do_log = get_rank() == 0 or all_ranks
    if do_log and value is not None:
        if _CSV["monitor"] is not None and get_rank() == 0:
            try:
                _CSV["monitor"].write(key, value, iteration_no)
            except (TypeError, ValueError):
                pass                                   # not a scalar
        if tensorboard_writer:
            tensorboard_writer.add_scalar(key, value, iteration_no)
        if use_wandb:
            try:
                import wandb
                wandb.log({key: value}, step=iteration_no)
            except Exception:
                pass
        if comet_experiment:
            comet_experiment.__internal_api__log_metric__(key, value, framework="gpt-neox", step=iteration_no)


def training_log(neox_args, timers, loss_dict, total_loss_dict, learning_rate, iteration, loss_scale,
                 report_memory_flag, skipped_iter, model, optimizer, noise_scale_logger):
    """Accumulate losses, write per-step scalars, and every ``log_interval`` print the throughput line
    (samples/s, tokens/s, TFLOP/s per GPU, MFU / HFU when ``peak_theoretical_tflops`` is set)."""
    skipped_key, nan_key = "skipped iterations", "got nan"
    total_loss_dict[skipped_key] = total_loss_dict.get(skipped_key, 0) + skipped_iter
    got_nan = False
    for key in loss_dict:
        if not skipped_iter:
            total_loss_dict[key] = total_loss_dict.get(key, 0.0) + loss_dict[key]
        else:
            value = loss_dict[key].float().sum().item()
            got_nan = got_nan or (value in (float("inf"), -float("inf")) or value != value)
    total_loss_dict[nan_key] = total_loss_dict.get(nan_key, 0) + int(got_nan)
    sinks = dict(use_wandb=neox_args.use_wandb, tensorboard_writer=getattr(neox_args, "tensorboard_writer", None),
                 comet_experiment=getattr(neox_args, "comet_experiment", None))
    names = [n for n in ("forward", "backward", "backward-backward", "backward-allreduce", "backward-master-grad",
                         "backward-clip-grad", "optimizer", "batch generator") if n in timers.timers]
    normalizer = iteration % neox_args.log_interval or neox_args.log_interval
    if not neox_args.is_pipe_parallel and get_rank() == 0 and names:
        timers.write(names=names, iteration=iteration, normalizer=normalizer)
    elif getattr(model, "timer_values", None):
        for k, v in model.timer_values.items():
            tb_wandb_log(f"timers/{k}", v, iteration, **sinks)
    tb_wandb_log("train/learning_rate", learning_rate, iteration, **sinks)
    for key in loss_dict:
        tb_wandb_log(f'train/{key.replace(" ", "_")}', loss_dict[key], iteration, **sinks)
    if neox_args.fp16:
        tb_wandb_log("train/loss_scale", loss_scale, iteration, **sinks)
    if neox_args.log_gradient_noise_scale and noise_scale_logger is not None:
        if noise_scale_logger.noise_scale is not None:
            tb_wandb_log("train/noise_scale", noise_scale_logger.noise_scale, iteration, **sinks)
    if neox_args.log_grad_norm and hasattr(model, "get_global_grad_norm"):
        tb_wandb_log("train/global_grad_norm", model.get_global_grad_norm(), iteration, **sinks)
    if neox_args.log_param_norm or neox_args.log_grad_pct_zeros or neox_args.log_optimizer_states:
        grads = getattr(model, "stored_gradients", None)
        for i, (name, param) in enumerate(model.module.named_parameters()):
            if neox_args.log_param_norm:
                tb_wandb_log(f"parameter_norms/{name}", torch.norm(param.detach().float()).item(), iteration,
                             all_ranks=True, **sinks)
            if neox_args.log_grad_pct_zeros and grads is not None and i < len(grads):
                g = grads[i]
                tb_wandb_log(f"pct_grad_zeros/{name}", (g.eq(0).float().sum() * 100.0 / g.numel()).item(),
                             iteration, all_ranks=True, **sinks)
    if iteration % neox_args.log_interval == 0:
        elapsed_time = timers("interval time").elapsed()
        iteration_time = elapsed_time / neox_args.log_interval
        samples_per_sec = neox_args.train_batch_size / iteration_time
        steps_per_sec = 1 / iteration_time
        tokens_per_sec = samples_per_sec * neox_args.seq_length
        log_string = " samples/sec: {:.3f} |".format(samples_per_sec)
        for k, v in (("runtime/samples_per_sec", samples_per_sec), ("runtime/iteration_time", iteration_time),
                     ("runtime/steps_per_sec", steps_per_sec), ("runtime/tokens_per_sec", tokens_per_sec)):
            tb_wandb_log(k, v, iteration, **sinks)
        log_string += " iteration {:8d}/{:8d} |".format(iteration, neox_args.train_iters)
        log_string += " elapsed time per iteration (ms): {:.1f} |".format(elapsed_time * 1000.0 / neox_args.log_interval)
        log_string += " learning rate: {:.3E} |".format(learning_rate)
        num_iterations = max(1, neox_args.log_interval - total_loss_dict[skipped_key])
        for key in total_loss_dict:
            if key not in (skipped_key, nan_key):
                v = total_loss_dict[key]
                v = v.item() if hasattr(v, "item") else v
                log_string += " {}: {:.6E} |".format(key, v / num_iterations)
                total_loss_dict[key] = 0.0
        if neox_args.precision == "fp16":
            log_string += " loss scale: {:.1f} |".format(loss_scale)
        log_string += " number of skipped iterations: {:3d} |".format(total_loss_dict[skipped_key])
        log_string += " number of nan iterations: {:3d} |".format(total_loss_dict[nan_key])
        total_loss_dict[skipped_key] = 0
        total_loss_dict[nan_key] = 0
        flops_per_s_per_gpu = get_actual_flops(neox_args, iteration_time)
        log_string += f" approx flops per GPU: {human_readable_flops(flops_per_s_per_gpu)} |"
        tb_wandb_log("runtime/flops_per_sec_per_gpu", flops_per_s_per_gpu, iteration, **sinks)
        if neox_args.peak_theoretical_tflops:
            peak = neox_args.peak_theoretical_tflops * 10 ** 12
            fb = get_forward_backward_flops(neox_args, iteration_time)
            tb_wandb_log("runtime/model_flops_utilization", fb / peak, iteration, **sinks)
            log_string += f" MFU: {fb / peak * 100.0:.2f}% approx flops per GPU: {human_readable_flops(fb)} |"
            if neox_args.checkpoint_activations:
                tb_wandb_log("runtime/hardware_flops_utilization", flops_per_s_per_gpu / peak, iteration, **sinks)
                log_string += f" HFU: {flops_per_s_per_gpu / peak * 100.0:.2f}% |"
        print_rank_0(log_string)
        if report_memory_flag:
            report_memory("after {} iterations".format(iteration))
            report_memory_flag = False
        timers.log(names, normalizer=neox_args.log_interval)
    return report_memory_flag

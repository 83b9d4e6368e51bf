"""Checkpoint save / load at the training-loop level (megatron/checkpointing.py:53-483): tags
``global_step<N>``, the saved client state (iteration, model-shape args, RNG states, optional
validation logits), the ``configs/`` copy of the YAML files, pruning to the last N checkpoints,
optional S3 mirror, arg-consistency and forward-pass validation on load."""
from __future__ import annotations

import json
import os
import random
import re
import shutil
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

from .. import parallel as mpu
from ..utils.common import natural_sort, print_rank_0


def _rank():
    return dist.get_rank() if dist.is_initialized() else 0


def _barrier():
    if dist.is_initialized():
        dist.barrier()


def check_checkpoint_args(neox_args, checkpoint_args):
    """Model-shape arguments stored in the checkpoint must equal the current ones."""
    assert isinstance(checkpoint_args, dict), "args stored in checkpoint is a dict"
    for name, value in checkpoint_args.items():
        args_value = getattr(neox_args, name)
        assert value == args_value, (f"{name} value from checkpoint ({value}) is not equal to the currently set "
                                     f"argument value ({args_value}).")


def _dev():
    if torch.cuda.is_available() and (not dist.is_initialized() or dist.get_backend() == "nccl"):
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def do_forward_pass(neox_args, model, inference=False):
    """Logits of a fixed synthetic batch (token i at position i), first batch item."""
    was_training = model.training
    model.eval()
    ctx = torch.arange(neox_args.seq_length + 1).repeat((neox_args.train_micro_batch_size_per_gpu, 1)).to(_dev())
    ctx = ctx % neox_args.padded_vocab_size
    with torch.no_grad():
        if neox_args.is_pipe_parallel:
            _, logits = model.eval_batch(data_iter=iter([{"text": ctx}]), return_logits=True)
        else:
            from ..utils.common import get_ltor_masks_and_position_ids
            tokens = ctx[:, : neox_args.seq_length].contiguous()
            need_mask = any(t not in ("flash", "rwkv", "mamba") for t in (neox_args.attention_config or []))
            mask, _, pos = get_ltor_masks_and_position_ids(tokens, 0, False, neox_args.sliding_window_width, need_mask)
            logits = model((tokens, pos, mask))
    if was_training:
        model.train()
    if logits is not None:
        logits = logits.detach().float().cpu()[0]
    return logits


def check_forward_pass(neox_args, model, checkpoint_logits, inference):
    logits = do_forward_pass(neox_args=neox_args, model=model, inference=inference)
    if logits is not None and checkpoint_logits is not None:
        if not (logits == checkpoint_logits).all().item():
            if mpu.get_data_parallel_rank() == 0:
                print(" > WARNING: validate_checkpoint_forward() forward after load of checkpoint does not yield "
                      "exactly same result")
            assert torch.isclose(logits, checkpoint_logits).all().item(), \
                "validate_checkpoint_forward() forward after load of checkpoint does not yield a close result"


_PENDING_RNG = [None]      # random-stream state of the loaded checkpoint, until the training loop takes it


def apply_pending_rng_state():
    """Re-apply (once) the random-stream state of the checkpoint that was loaded last."""
    rng, _PENDING_RNG[0] = _PENDING_RNG[0], None
    if rng is not None:
        restore_rng_state(rng)


def restore_rng_state(rng):
    random.setstate(rng["random_rng_state"])
    np.random.set_state(rng["np_rng_state"])
    torch.set_rng_state(rng["torch_rng_state"])
    if torch.cuda.is_available() and rng.get("cuda_rng_state") is not None:
        torch.cuda.set_rng_state(rng["cuda_rng_state"])
    mpu.get_cuda_rng_tracker().set_states(rng["rng_tracker_states"])
    if rng.get("kernel_dropout_counters") is not None:
        # the dropout kernels derive their seeds from call counters, which are part of the random state
        from ..parallel.random import _kernel_dropout_counters
        _kernel_dropout_counters(tuple(rng["kernel_dropout_counters"]))


def ensure_directory_exists(filename):
    os.makedirs(os.path.dirname(filename), exist_ok=True)


def get_checkpoint_name(checkpoints_path, iteration, release=False, mp_rank=None):
    """Path of the single-file (Megatron-style) checkpoint of one tensor-parallel rank
    (megatron/checkpointing.py:138-151); the engine's own checkpoints are tag directories, see below."""
    sub = "release" if release else f"iter_{int(iteration):07d}"
    rank = mpu.get_model_parallel_rank() if mp_rank is None else mp_rank
    return os.path.join(checkpoints_path, sub, f"mp_rank_{rank:02d}", "model_optim_rng.pt")


def get_checkpoint_tag(iteration: int) -> str:
    return f"global_step{iteration}"


def delete_old_checkpoints(save_dir, n_to_keep):
    if _rank() == 0:
        ckpt_dir_regex = r"global_step[\d]*$"
        all_ckpts = natural_sort([i for i in os.listdir(save_dir) if os.path.isdir(os.path.join(save_dir, i))
                                  and re.search(ckpt_dir_regex, i)])
        n_to_delete = len(all_ckpts) - n_to_keep
        if n_to_delete > 0:
            for ckpt in all_ckpts[:n_to_delete]:
                try:
                    shutil.rmtree(os.path.join(save_dir, ckpt))
                except FileNotFoundError:
                    pass


def save_ds_checkpoint(iteration, model, neox_args):
    sd = {
        "iteration": iteration,
        "args": {k: getattr(neox_args, k) for k in
                 ("num_layers", "hidden_size", "num_attention_heads", "max_position_embeddings",
                  "make_vocab_size_divisible_by", "padded_vocab_size", "tokenizer_type", "model_parallel_size")},
    }
    if not neox_args.no_save_rng:
        sd["random_rng_state"] = random.getstate()
        sd["np_rng_state"] = np.random.get_state()
        sd["torch_rng_state"] = torch.get_rng_state()
        sd["cuda_rng_state"] = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
        sd["rng_tracker_states"] = mpu.get_cuda_rng_tracker().get_states()
        from ..parallel.random import _kernel_dropout_counters
        sd["kernel_dropout_counters"] = _kernel_dropout_counters()
    if neox_args.checkpoint_validation_with_forward_pass:
        sd["checkpoint_validation_logits"] = do_forward_pass(neox_args=neox_args, model=model)
    tag = get_checkpoint_tag(iteration)
    model.save_checkpoint(neox_args.save, tag=tag, client_state=sd)
    if _rank() == 0 and neox_args.config_files is not None:
        configs_directory = os.path.join(neox_args.save, tag, "configs")
        os.makedirs(configs_directory, exist_ok=True)
        for name, data in neox_args.config_files.items():
            with open(os.path.join(configs_directory, name), "w") as f:
                if isinstance(data, str):
                    f.write(data)
                else:
                    json.dump(data, f)


def _upload(file_path: str, s3_key: str, chunk_size: int = 104_857_600, max_files: int = 64, parallel: bool = True,
            max_retries: int = 5):
    """Multipart upload of one file to S3 through pre-signed URLs."""
    try:
        import boto3
        import hf_transfer
    except ModuleNotFoundError as e:
        raise RuntimeError("S3 upload needs `boto3` and `hf_transfer`, which are not installed") from e
    s3 = boto3.client("s3")
    bucket = s3_key.split("s3://")[1].split("/")[0]
    key = s3_key.split(bucket)[1].lstrip("/")
    upload = s3.create_multipart_upload(ACL="bucket-owner-full-control", Bucket=bucket, Key=key)
    upload_id = upload["UploadId"]
    file_size = os.stat(file_path).st_size
    urls = [s3.generate_presigned_url(ClientMethod="upload_part",
                                      Params={"Bucket": bucket, "Key": key, "UploadId": upload_id, "PartNumber": i + 1},
                                      ExpiresIn=86400)
            for i in range((file_size + chunk_size - 1) // chunk_size)]
    responses = hf_transfer.multipart_upload(file_path=file_path, parts_urls=urls, chunk_size=chunk_size,
                                             max_files=max_files, parallel_failures=max_files if parallel else 0,
                                             max_retries=max_retries)
    etags = [{"ETag": h.get("etag"), "PartNumber": i + 1} for i, h in enumerate(responses)]
    s3.complete_multipart_upload(Bucket=bucket, Key=key, MultipartUpload={"Parts": etags}, UploadId=upload_id)


def upload_checkpoint(iteration, neox_args):
    local = os.path.join(os.path.abspath(neox_args.save), get_checkpoint_tag(iteration))
    remote = os.path.join(neox_args.s3_path, os.path.basename(neox_args.save), get_checkpoint_tag(iteration))
    files = [os.path.join(root, f) for root, _, fs in os.walk(local) for f in fs]
    print(f"[RANK {_rank()}] Uploading checkpoint `{local}` to `{remote}`...", flush=True)
    start = time.time()
    for lp in files:
        _upload(lp, os.path.join(remote, os.path.relpath(lp, local)), chunk_size=neox_args.s3_chunk_size)
    print(f"[RANK {_rank()}] Uploaded checkpoint `{local}` to `{remote}` in {time.time() - start:.2f}s", flush=True)


def save_checkpoint(neox_args, iteration, model, optimizer, lr_scheduler):
    if neox_args.deepspeed:
        save_ds_checkpoint(iteration, model, neox_args)
    else:
        raise ValueError("Must be using deepspeed to use neox")
    _barrier()
    upload_to_s3 = _rank() == 0 and neox_args.s3_path is not None
    if upload_to_s3:
        upload_checkpoint(iteration, neox_args)
    _barrier()
    if neox_args.keep_last_n_checkpoints is not None:
        delete_old_checkpoints(neox_args.save, neox_args.keep_last_n_checkpoints)
    _barrier()


def load_checkpoint(neox_args, model, optimizer, lr_scheduler, inference=False, iteration=None):
    """-> iteration to resume from. ``finetune`` loads weights only and restarts at 0."""
    if neox_args.deepspeed:
        load_optim_and_scheduler = not neox_args.no_load_optim
        if neox_args.finetune:
            load_optim_and_scheduler = False
        tag = f"global_step{iteration}" if iteration is not None else None
        checkpoint_name, state_dict = model.load_checkpoint(
            neox_args.load, load_optimizer_states=load_optim_and_scheduler,
            load_lr_scheduler_states=load_optim_and_scheduler, load_module_only=not load_optim_and_scheduler, tag=tag,
            load_module_strict=neox_args.train_impl != "rm")
        if checkpoint_name is None:
            if iteration is not None:
                available = sorted([int(i.name.replace("global_step", "")) for i in
                                    __import__("pathlib").Path(neox_args.load).glob("global_step*")])
                raise ValueError(f"Unable to load checkpoint for iteration {iteration}. \nAvailable iterations: "
                                 f"{available}")
            if mpu.get_data_parallel_rank() == 0:
                print("Unable to load checkpoint.")
            return 0
    else:
        raise ValueError("Must be using deepspeed to use neox")
    if neox_args.finetune:
        iteration = 0
    else:
        if "iteration" in state_dict:
            iteration = state_dict["iteration"]
        else:
            iteration = state_dict.get("total_iters")
            if iteration is None:
                raise ValueError(f"Unable to load iteration from checkpoint {checkpoint_name} with keys "
                                 f"{state_dict.keys()}, exiting")
    if "args" in state_dict:
        check_checkpoint_args(neox_args=neox_args, checkpoint_args=state_dict["args"])
        print_rank_0(" > validated currently set args with arguments in the checkpoint ...")
    else:
        print_rank_0(" > could not find arguments in the checkpoint for validation...")
    if neox_args.checkpoint_validation_with_forward_pass:
        if "checkpoint_validation_logits" in state_dict:
            check_forward_pass(neox_args=neox_args, model=model,
                               checkpoint_logits=state_dict["checkpoint_validation_logits"], inference=inference)
            print_rank_0(" > validated loaded checkpoint with forward pass ...")
        elif mpu.get_data_parallel_rank() == 0:
            print(" > WARNING: checkpoint_validation_with_forward_pass is configured but no checkpoint validation "
                  f"data available in checkpoint {checkpoint_name}")
    if not neox_args.finetune and not neox_args.no_load_rng:
        try:
            rng = {k: state_dict[k] for k in ("random_rng_state", "np_rng_state", "torch_rng_state",
                                              "rng_tracker_states")}
            rng["cuda_rng_state"] = state_dict.get("cuda_rng_state")
            rng["kernel_dropout_counters"] = state_dict.get("kernel_dropout_counters")
            restore_rng_state(rng)
            # building the data iterators after this point draws from the global generators (DataLoader worker
            # seeds); the training loop re-applies the saved state right before its first step
            _PENDING_RNG[0] = rng
        except KeyError:
            print_rank_0(f"Unable to load optimizer from checkpoint {checkpoint_name}. Specify --no-load-rng or "
                         "--finetune to prevent attempting to load the optimizer state, exiting ...")
            sys.exit()
    _barrier()
    if mpu.get_data_parallel_rank() == 0:
        print("  successfully loaded {}".format(checkpoint_name))
    return iteration

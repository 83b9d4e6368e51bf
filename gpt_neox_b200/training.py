"""Pre-training / fine-tuning orchestration (megatron/training.py:219-1729): ``pretrain``, batch
construction, ``forward_step``, model / optimizer / scheduler set-up, ``train_step``, the train and
evaluate loops, checkpoint cadence and the profiler switches."""
from __future__ import annotations

import math
import sys
import time
from contextlib import nullcontext
from functools import partial

import numpy as np
import torch
import torch.distributed as dist

from . import parallel as mpu
from . import posttrain
from .ckpt.checkpointing import load_checkpoint, save_checkpoint
from .engine.engine import initialize as engine_initialize
from .engine.lr import AnnealingLR
from .initialize import initialize_megatron
from .models.gpt2_model import GPT2ModelPipe, cross_entropy
from .models.utils import get_params_for_weight_decay_optimization, mark_norms_for_sequence_parallel_grad_sync
from .obs.logging import tb_wandb_log, training_log
from .utils.common import (CharCounter, OverflowMonitor, Timers, get_ltor_masks_and_position_ids, init_wandb,
                           print_rank_0, reduce_losses)


def _nvtx_push(neox_args, name):
    if (neox_args.memory_profiling or neox_args.profile) and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)


def _nvtx_pop(neox_args):
    if (neox_args.memory_profiling or neox_args.profile) and torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


def update_iterations(neox_args, data_loaders):
    """``train_epochs`` -> ``train_iters`` (rank 0 decides, everyone follows)."""
    if neox_args.train_iters is not None or neox_args.train_epochs is None:
        return
    train_dataloader = data_loaders["train"]
    if train_dataloader is not None:
        iters_per_epoch = len(train_dataloader) / neox_args.gradient_accumulation_steps
        train_iters = math.ceil(iters_per_epoch * neox_args.train_epochs)
    else:
        train_iters = 0
    t = torch.tensor([train_iters], dtype=torch.long, device=_device())
    if dist.is_initialized():
        dist.broadcast(t, src=0)
    neox_args.train_iters = int(t[0].item())
    print_rank_0(f"> training for {neox_args.train_epochs} epochs = {neox_args.train_iters} iterations")


def _device():
    if torch.cuda.is_available() and (not dist.is_initialized() or dist.get_backend() == "nccl"):
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def pretrain(neox_args):
    """Init, build data + model + optimizer, train, evaluate, save."""
    init_wandb(neox_args=neox_args)
    timers = Timers(use_wandb=neox_args.use_wandb, tensorboard_writer=getattr(neox_args, "tensorboard_writer", None),
                    comet_experiment=getattr(neox_args, "comet_experiment", None))
    initialize_megatron(neox_args=neox_args)
    from .data.data_utils import build_train_valid_test_data_loaders, shift_and_wrap_data_loaders
    timers("train/valid/test data loaders").start()
    data_loaders = build_train_valid_test_data_loaders(neox_args=neox_args)
    update_iterations(neox_args=neox_args, data_loaders=data_loaders)
    timers("train/valid/test data loaders").stop()
    if neox_args.serve_model_weights:
        from .models.weight_server import start_server
        start_server_fn = start_server
    timers("model and optimizer").start()
    model, optimizer, lr_scheduler, reference_model = setup_model_and_optimizer(neox_args=neox_args, use_cache=False)
    timers("model and optimizer").stop()
    if neox_args.serve_model_weights:
        start_server_fn(model)
        if dist.is_initialized():
            dist.barrier()
    timers("train/valid/test data iterators").start()
    train_data_iterator, valid_data_iterator, test_data_iterator = shift_and_wrap_data_loaders(
        neox_args=neox_args, data_loaders=data_loaders)
    timers("train/valid/test data iterators").stop()
    if neox_args.use_mup and neox_args.coord_check:
        mup_coord_check(neox_args, timers, train_data_iterator)
    print_rank_0("done with setups ...")
    timers.log(["train/valid/test data loaders", "model and optimizer", "train/valid/test data iterators"])
    print_rank_0("training ...")
    iteration = neox_args.iteration
    if neox_args.save and neox_args.extra_save_iters and 0 in neox_args.extra_save_iters and iteration == 0:
        save_checkpoint(neox_args=neox_args, iteration=iteration, model=model, optimizer=optimizer,
                        lr_scheduler=lr_scheduler)
    # a resumed run continues the random streams of the interrupted one from its first step on (building the data
    # iterators above drew from them)
    from .ckpt.checkpointing import apply_pending_rng_state
    apply_pending_rng_state()
    from .obs.logging import configure_csv_monitor
    configure_csv_monitor(neox_args)
    if neox_args.do_train and neox_args.train_iters > 0:
        iteration = train(neox_args=neox_args, timers=timers, model=model, reference_model=reference_model,
                          optimizer=optimizer, lr_scheduler=lr_scheduler, train_data_iterator=train_data_iterator,
                          valid_data_iterator=valid_data_iterator)
    if neox_args.do_valid:
        prefix = "the end of training for val data"
        evaluate_and_print_results(neox_args=neox_args, prefix=prefix, forward_step_func=forward_step,
                                   data_iterator=valid_data_iterator, model=model, iteration=iteration, verbose=False,
                                   timers=timers, reference_model=reference_model)
    if neox_args.save and iteration != 0 and not is_save_iter(neox_args, iteration):
        save_checkpoint(neox_args=neox_args, iteration=iteration, model=model, optimizer=optimizer,
                        lr_scheduler=lr_scheduler)
    if neox_args.do_test:
        prefix = "the end of training for test data"
        evaluate_and_print_results(neox_args=neox_args, prefix=prefix, forward_step_func=forward_step,
                                   data_iterator=test_data_iterator, model=model, iteration=iteration, verbose=True,
                                   timers=timers, chart_name="test", reference_model=reference_model)
    comms = getattr(model, "comms_logger", None)
    if comms is not None:                       # comms_logger: the table of every collective of the run
        comms.log_summary()
        comms.uninstall()
    return model


# ----------------------------------------------------------------------------------------- batches
def _get_batch(neox_args, tokenizer, keys, data, datatype, label_mask_zero=False):
    """Broadcast over the tensor-parallel group, split into tokens / labels, build masks."""
    data_b = mpu.broadcast_data(keys, data, datatype)
    token_key = keys[0]
    label_key = keys[1] if len(keys) > 1 else None
    tokens_ = data_b[token_key].long()
    if label_key in data_b:
        label_mask = (data_b[label_key].long() >= 0)[:, 1:].contiguous()
        labels = torch.where(data_b[label_key].long() >= 0, data_b[label_key].long(),
                             torch.zeros_like(data_b[label_key].long()))[:, 1:].contiguous()
    else:
        label_mask = (tokens_.long() >= 0)[:, 1:].contiguous()
        labels = tokens_[:, 1:].contiguous()
    if label_mask_zero:
        labels = labels * label_mask
    tokens = tokens_[:, :-1].contiguous()
    need_mask = any(t not in ("flash", "rwkv", "mamba") for t in (neox_args.attention_config or []))
    attention_mask, loss_mask, position_ids = get_ltor_masks_and_position_ids(
        data=tokens, eod_token=getattr(tokenizer, "eod", 0), eod_mask_loss=neox_args.eod_mask_loss,
        sliding_window_width=neox_args.sliding_window_width, build_attention_mask=need_mask)
    loss_mask = label_mask.to(loss_mask.dtype) * loss_mask
    return tokens, labels, loss_mask, attention_mask, position_ids


def get_batch(neox_args, data_iterator):
    """Next micro-batch for ``train_impl`` in normal | kto | reinforce | dpo | rm."""
    impl = neox_args.train_impl
    if impl in ("normal", "kto", "reinforce"):
        keys = ["text", "label"] if neox_args.train_label_data_paths else ["text"]
    else:
        keys = [["pos", "pos_label"], ["neg", "neg_label"]] if neox_args.pos_train_label_data_paths \
            else [["pos"], ["neg"]]
    datatype = torch.int64
    data = next(data_iterator) if data_iterator is not None else None
    g = partial(_get_batch, neox_args=neox_args, tokenizer=neox_args.tokenizer, data=data, datatype=datatype)
    if impl == "normal":
        return g(keys=keys)
    if impl == "kto":
        assert neox_args.train_micro_batch_size_per_gpu > 1, \
            "For KTO training, the train_micro_batch_size_per_gpu must be greater than 1."
        tup = g(keys=keys)
        rw = mpu.broadcast_data(["reward"], data, torch.float)["reward"][:, :-1].contiguous()
        ref = mpu.broadcast_data(["ref"], data, torch.float)["ref"][:, :-1].contiguous() \
            if neox_args.precompute_model_name else None
        return tup + (rw, ref)
    if impl == "reinforce":
        tup = g(keys=keys)
        rw = mpu.broadcast_data(["reward"], data, torch.float)["reward"]
        raw = mpu.broadcast_data(["raw_reward"], data, torch.float)["raw_reward"]
        return tup + (rw, raw)
    pos = g(keys=keys[0], label_mask_zero=True)
    neg = g(keys=keys[1], label_mask_zero=True)
    ref = mpu.broadcast_data(["pos_ref", "neg_ref"], data, torch.float) if neox_args.precompute_model_name \
        else {"pos_ref": None}
    # tokens / labels / loss mask / position ids are stacked [chosen; rejected]; the causal attention mask is one
    # batch-broadcast [1, 1, s, s] tensor and stays that way (stacking two of them would not broadcast against
    # the doubled batch on the non-flash attention path)
    out = [None if p is None else (p if (i == 3 and p.shape[0] == 1) else torch.cat((p, n), dim=0))
           for i, (p, n) in enumerate(zip(pos, neg))]
    out.append(torch.cat((ref["pos_ref"], ref["neg_ref"]), dim=0)[:, :-1].contiguous()
               if ref["pos_ref"] is not None else None)
    return out


def get_batch_pipe(data, neox_args, curr_scheduler=None):
    """Batch function of the pipeline engine: ``((tokens, position_ids, mask), (labels, loss_mask))``."""
    assert neox_args.train_impl not in ("kto", "dpo", "rm"), \
        "Pipeline parallel is currently unsupported when using any of kto, dpo, rm. Set pipe_parallel_size to 0"
    keys = ["text", "label"] if neox_args.train_label_data_paths else ["text"]
    tokens, labels, loss_mask, attention_mask, position_ids = _get_batch(neox_args, neox_args.tokenizer, keys, data,
                                                                         torch.int64)
    if curr_scheduler is not None:
        curriculum_seqlen = curr_scheduler.update_difficulty(neox_args.iteration + 1)
        if curriculum_seqlen < tokens.size(1):
            tokens = tokens[:, :curriculum_seqlen].contiguous()
            position_ids = position_ids[:, :curriculum_seqlen].contiguous()
            if labels is not None:
                labels = labels[:, :curriculum_seqlen].contiguous()
            if loss_mask is not None:
                loss_mask = loss_mask[:, :curriculum_seqlen].contiguous()
            if attention_mask is not None:
                attention_mask = attention_mask[:, :, :curriculum_seqlen, :curriculum_seqlen].contiguous()
    return (tokens, position_ids, attention_mask), (labels, loss_mask)


def get_batch_sequential(forward_input, neox_args):
    attention_mask, _, position_ids = get_ltor_masks_and_position_ids(
        data=forward_input[0], eod_token=neox_args.tokenizer.eod, eod_mask_loss=neox_args.eod_mask_loss)
    return (forward_input[0], forward_input[1], attention_mask)


# ----------------------------------------------------------------------------------------- forward
def forward_step(data_iterator, model, neox_args, timers, return_logits=False, is_train=False,
                 reference_model=None):
    if neox_args.is_pipe_parallel:
        return model.eval_batch(data_iterator, return_logits=return_logits)
    _nvtx_push(neox_args, "Get batch")
    if timers is not None:
        timers("batch generator").start()
    batch = get_batch(neox_args=neox_args, data_iterator=data_iterator)
    impl = neox_args.train_impl
    rewards = raw_rewards = ref_logp = None
    if impl == "normal":
        tokens, labels, loss_mask, attention_mask, position_ids = batch
    elif impl == "kto":
        tokens, labels, loss_mask, attention_mask, position_ids, rewards, ref_logp = batch
    elif impl == "reinforce":
        tokens, labels, loss_mask, attention_mask, position_ids, rewards, raw_rewards = batch
    else:
        tokens, labels, loss_mask, attention_mask, position_ids, ref_logp = batch
    if timers is not None:
        timers("batch generator").stop()
    _nvtx_pop(neox_args)
    _nvtx_push(neox_args, "Forward pass")
    metrics = {}
    inputs = (tokens, position_ids, attention_mask)
    if impl == "normal":
        outputs = model(inputs, neox_args=neox_args)
        if is_train and neox_args.curriculum_learning and neox_args.curriculum_seqlen < neox_args.seq_length:
            loss_mask = loss_mask[:, : neox_args.curriculum_seqlen].contiguous()
            labels = labels[:, : neox_args.curriculum_seqlen].contiguous()
        loss = cross_entropy(outputs, (labels, loss_mask), _fp16=neox_args.fp16_lm_cross_entropy)
    elif impl == "rm":
        outputs = model(inputs, neox_args=neox_args)
        loss, metrics = posttrain.rm_loss(outputs, loss_mask, neox_args.z_loss)
    elif impl == "dpo":
        with torch.no_grad():
            pos_mask, neg_mask = torch.chunk(loss_mask, 2, 0)
            if neox_args.dpo_reference_free:
                ref_pos = ref_neg = torch.zeros((), device=tokens.device)
            elif ref_logp is None:
                ref_out = reference_model(inputs, neox_args=neox_args)
                ref_pos, ref_neg = posttrain.get_pos_neg_logp(posttrain._first(ref_out), labels, neox_args.dpo_fp32)
                ref_pos, ref_neg = (ref_pos * pos_mask).sum(-1), (ref_neg * neg_mask).sum(-1)
            else:
                ref_pos, ref_neg = torch.chunk(ref_logp, 2, 0)
                ref_pos, ref_neg = (ref_pos * pos_mask).sum(-1), (ref_neg * neg_mask).sum(-1)
        outputs = model(inputs, neox_args=neox_args)
        loss, metrics = posttrain.dpo_loss(outputs, labels, loss_mask, ref_pos, ref_neg, neox_args.dpo_beta,
                                           neox_args.dpo_reference_free, neox_args.dpo_fp32)
    elif impl == "kto":
        with torch.no_grad():
            if ref_logp is None:
                ref_out = posttrain._first(reference_model(inputs, neox_args=neox_args))
                ref_logp = posttrain.get_logp(ref_out, labels, neox_args.kto_fp32)
        outputs = model(inputs, neox_args=neox_args)
        chosen_logp = posttrain.get_logp(posttrain._first(outputs), labels, neox_args.kto_fp32)
        loss, metrics = posttrain.kto_loss(chosen_logp, ref_logp, rewards, loss_mask, neox_args.kto_beta,
                                           neox_args.kto_desirable_weight, neox_args.kto_undesirable_weight)
    else:  # reinforce
        ref_out = None
        if reference_model is not None:
            with torch.no_grad():
                ref_out = reference_model(inputs, neox_args=neox_args)
        outputs = model(inputs, neox_args=neox_args)
        loss, metrics = posttrain.reinforce_loss(outputs, ref_out, labels, loss_mask, rewards, raw_rewards,
                                                 neox_args.kl_impl, neox_args.kl_div_beta, neox_args.fp32_reinforce)
    _nvtx_pop(neox_args)
    if return_logits:
        return loss, outputs, metrics
    return loss, metrics


# ----------------------------------------------------------------------------------------- set-up
def _mup_optimizer_kind(neox_args) -> str:
    ot = (neox_args.optimizer_type or "adam").lower()
    assert ot in ("adam", "sgd"), \
        f"If use_mup == True, you must specify either the adam or sgd optimizers. You passed: {ot}"
    return ot


def save_base_shapes(neox_args, path, use_cache, base_shapes):
    """Write the muP base-shapes file of this rank and stop (megatron/training.py:86-136): the model as
    configured is the base model, a second one ``mup_width_scale`` times wider tells which dimensions grow."""
    from . import mup
    old = neox_args.hidden_size
    neox_args.hidden_size = old * neox_args.mup_width_scale
    delta = GPT2ModelPipe(neox_args=neox_args, num_tokentypes=0, parallel_output=neox_args.train_impl != "rm",
                          topology=mpu.get_topology(), use_cache=use_cache)
    if not neox_args.is_pipe_parallel:
        delta = delta.to_sequential()
    neox_args.hidden_size = old
    print(f"saving base shapes at {path}", flush=True)
    mup.make_base_shapes(base_shapes, mup.get_shapes(delta), savefile=path)
    print("base shapes saved...exiting", flush=True)
    sys.exit(1)


def mup_coord_check(neox_args, timers, train_data_iterator):
    """Activation scale against width, with muP and with the standard parametrisation
    (megatron/training.py:139-171): ``coord_check_{up,sp}.<rank>.json`` (+ ``.jpg`` with matplotlib)."""
    from . import mup
    rank = dist.get_rank() if dist.is_initialized() else 0
    widths = [neox_args.num_attention_heads * (2 ** p) for p in range(2, 9)]
    if neox_args.mup_coord_check_widths:
        widths = list(neox_args.mup_coord_check_widths)

    def lazy_model(hidden_size):
        def gen():
            old = neox_args.hidden_size
            neox_args.hidden_size = hidden_size
            try:
                model, opt, sched, _ref = setup_model_and_optimizer(neox_args=neox_args, use_cache=False)
            finally:
                neox_args.hidden_size = old
            model._coord_check_state = (opt, sched)
            return model
        return gen

    def one_step(model):
        opt, sched = model._coord_check_state
        train_step(neox_args=neox_args, timers=timers, data_iterator=train_data_iterator, model=model,
                   optimizer=opt, lr_scheduler=sched)

    out = {}
    for tag, flag in (("up", True), ("sp", False)):
        neox_args.use_mup = flag
        recs = mup.get_coord_data({w: lazy_model(w) for w in widths}, one_step, nsteps=neox_args.mup_coord_check_steps)
        mup.save_coord_data(recs, f"coord_check_{tag}.{rank}")
        out[tag] = recs
    neox_args.use_mup = True
    return out


def get_model(neox_args, use_cache=False):
    """Build the model on its device in ``params_dtype``; flatten to sequential when there is no
    pipeline parallelism; ZeRO >= 2 is refused with tensor / pipeline parallelism as in the
    reference (megatron/training.py:878-893)."""
    print_rank_0("building GPT2 model ...")
    if neox_args.zero_stage in (2, 3):
        if neox_args.pipe_parallel_size == 1:
            print_rank_0("ZeRO stage 2/3 and the PipelineModule are incompatible, please set "
                         "'pipe_parallel_size' to 0 instead")
            sys.exit()
        if neox_args.pipe_parallel_size > 1:
            print_rank_0("ZeRO stage 2/3 and pipeline paralleism are not supported simultaneously")
            sys.exit()
        if neox_args.model_parallel_size > 1:
            print_rank_0("ZeRO stage 2/3 and model paralleism are not currently supported simultaneously")
            sys.exit()
    # muP: the modules read ``use_mup`` at construction (embedding multipliers, 1/d attention scale,
    # ``mup_init_scale``); the width-dependent parts follow below, once the base shapes are attached
    model = GPT2ModelPipe(neox_args=neox_args, num_tokentypes=0, parallel_output=neox_args.train_impl != "rm",
                          topology=mpu.get_topology(), use_cache=use_cache)
    if neox_args.soft_prompt_tuning is not None and neox_args.soft_prompt_tuning.get("enabled", False):
        from .models.word_embeddings import SoftEmbedding
        soft_prompt = SoftEmbedding(neox_args, wte=getattr(model, "0").word_embeddings if hasattr(model, "0") else None,
                                    n_tokens=neox_args.soft_prompt_tuning.get("n_tokens", 10),
                                    init_string=neox_args.soft_prompt_tuning.get("init_string", ""),
                                    init_range=neox_args.soft_prompt_tuning.get("init_range", 0.5))
        model.insert_layers(layers=soft_prompt, idx=1)
        for name, param in model.named_parameters():
            if "soft_embedding" not in name:
                param.requires_grad = False
    if not neox_args.is_pipe_parallel:
        model = model.to_sequential()
    if neox_args.use_mup:
        from . import mup
        rank = dist.get_rank() if dist.is_initialized() else 0
        base_shapes = f"{neox_args.base_shapes_file}.{rank}"
        if neox_args.save_base_shapes:
            save_base_shapes(neox_args, base_shapes, use_cache, mup.get_shapes(model))
        mup.set_base_shapes(model, base_shapes)
        mup.apply_mup(model, optimizer=_mup_optimizer_kind(neox_args))
    dev = _device()
    model = model.to(device=dev)
    for p in model.parameters():
        if p.dtype != neox_args.params_dtype and p.is_floating_point() and \
                not getattr(p, "_deepspeed_no_cast", False):
            p.data = p.data.to(neox_args.params_dtype)
    for b in model.buffers():
        if b.is_floating_point() and b.dtype != torch.float32:
            b.data = b.data.float()
    return model


def get_optimizer(model, neox_args, dummy=False):
    """-> (optimizer config for the engine, param groups). ``no_load_optim`` / ``optimizer: None`` builds
    nothing (inference)."""
    if neox_args.no_load_optim and neox_args.optimizer is None:
        return None, None
    if neox_args.optimizer is None:
        print_rank_0(f"ERROR: Optimizer is None. Either set the optimizer dict in your config (if training) or set "
                     f"no_load_optim in your config (if inference)")
        exit()
    param_groups = get_params_for_weight_decay_optimization(model, neox_args)
    print_rank_0(f'Configuring Optimizer type: {neox_args.optimizer_type} with params: {neox_args.optimizer["params"]}')
    params = dict(neox_args.optimizer["params"])
    for pg in param_groups:
        pg["params"] = [p for p in pg["params"] if p.requires_grad]
    param_groups = [pg for pg in param_groups if len(pg["params"]) > 0]
    ot = neox_args.optimizer_type.lower()
    cfg = {"lr": params.get("lr", neox_args.lr), "betas": tuple(params.get("betas", (0.9, 0.999))),
           "eps": params.get("eps", 1e-8), "weight_decay": neox_args.weight_decay}
    generic = None
    if ot in ("adam", "cpu_adam", "cpu_torch_adam"):
        cfg["adam_w_mode"] = True
        # optimizer-state offload: "cpu_adam" (the reference's DeepSpeedCPUAdam, megatron/training.py:1002-1012) runs
        # this build's native host AdamW, "cpu_torch_adam" PyTorch's CPU operators; ZeRO's cpu_offload /
        # offload_optimizer switch selects the native one for plain "adam" too
        zo = neox_args.zero_optimization or {}
        wants = bool(zo.get("cpu_offload")) or (zo.get("offload_optimizer") or {}).get("device") == "cpu"
        if ot == "cpu_torch_adam":
            cfg["offload"] = "torch"
        elif ot == "cpu_adam" or wants:
            cfg["offload"] = "native"
    elif ot == "onebitadam":
        # the reference lets DeepSpeed build this one (megatron/training.py:1014-1017); here it is an in-tree
        # optimizer on the engine's generic path (optimizers.py OnebitAdam)
        from . import optimizers as opts
        if (neox_args.zero_stage or 0) != 0:
            raise ValueError("OneBitAdam keeps whole (unpartitioned) optimizer state: set zero_optimization.stage to 0")
        kw = {k: params[k] for k in ("freeze_step", "eps") if k in params}
        kw["betas"] = tuple(params.get("betas", (0.9, 0.999)))
        generic = {"generic_cls": opts.OnebitAdam, "generic_kwargs": kw}
    else:
        from . import optimizers as opts
        table = {"sm3": (opts.SM3, {}), "madgrad_wd": (opts.madgrad_wd, {k: v for k, v in params.items()
                                                                     if k in ("momentum", "eps")}),
                 "lion": (opts.Lion, {"betas": tuple(params.get("betas", (0.9, 0.99)))}),
                 "sgd": (torch.optim.SGD, {k: v for k, v in params.items() if k in ("momentum", "nesterov")})}
        if ot not in table:
            raise ValueError(f"Optimizer type {neox_args.optimizer_type} not recognized")
        generic = {"generic_cls": table[ot][0], "generic_kwargs": table[ot][1]}
    if neox_args.use_bnb_optimizer:
        # the reference swaps in bitsandbytes' Adam8bit here (megatron/training.py:1058-1067); this build keeps the
        # moments of its own fused AdamW in 8 bits block-wise (csrc/optim.cu adam8_kernel), no external package
        if generic is not None:
            raise ValueError("use_bnb_optimizer (8-bit optimizer state) is built for the Adam optimizer only, "
                             f"not for {neox_args.optimizer_type}")
        cfg["state_bits"] = 8
    return (cfg, generic), param_groups


def get_learning_rate_scheduler(optimizer, neox_args):
    if neox_args.no_load_optim:
        return None
    num_iters = neox_args.lr_decay_iters if neox_args.lr_decay_iters is not None else neox_args.train_iters
    if neox_args.lr_decay_fraction is not None and neox_args.train_iters:
        num_iters = math.floor(neox_args.train_iters * neox_args.lr_decay_fraction)
    num_iters = max(1, num_iters or 1)
    init_step = 0
    warmup_iter = neox_args.warmup * num_iters

    class _Stub:
        param_groups = []
    return AnnealingLR(optimizer if optimizer is not None else _Stub(), start_lr=neox_args.lr,
                       warmup_iter=warmup_iter, total_iters=num_iters, decay_style=neox_args.lr_decay_style,
                       last_iter=init_step, min_lr=neox_args.min_lr,
                       use_checkpoint_lr_scheduler=neox_args.use_checkpoint_lr_scheduler,
                       override_lr_scheduler=neox_args.override_lr_scheduler, use_mup=neox_args.use_mup)


def setup_model_and_optimizer(neox_args, use_cache=False, iteration=None):
    """-> (engine, optimizer, lr_scheduler, reference_model)."""
    if neox_args.memory_profiling and torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(True, trace_alloc_max_entries=100000, trace_alloc_record_context=True)
    if _device().type == "cuda" and neox_args.params_dtype == torch.float32:
        # said once, before anything is built, instead of a kernel error in the middle of the first step
        raise ValueError('"precision": "fp32" is not built for the GPU: the sm_100a kernels take 16-bit activations '
                         'and weights with fp32 accumulation, master weights and optimizer state. Use '
                         '"precision": "bfloat16" or "fp16" (an "fp16" block with dynamic loss scaling works '
                         'unchanged); fp32 runs on CPU ("distributed_backend": "gloo").')
    model = get_model(neox_args=neox_args, use_cache=use_cache)
    reference_model = None
    needs_ref = (neox_args.train_impl == "dpo" and neox_args.precompute_model_name is None
                 and not neox_args.dpo_reference_free) or \
                (neox_args.train_impl == "kto" and neox_args.precompute_model_name is None)
    if needs_ref or (neox_args.train_impl == "reinforce" and neox_args.kl_div_beta != 0.0 and neox_args.load):
        reference_model = get_model(neox_args=neox_args, use_cache=use_cache)
    opt_cfg, param_groups = get_optimizer(model=model, neox_args=neox_args)
    lr_scheduler = get_learning_rate_scheduler(optimizer=None, neox_args=neox_args) if opt_cfg is not None else None
    print_rank_0("engine.initialize is called")
    cfg, generic = opt_cfg if opt_cfg is not None else (None, None)
    if param_groups is None:
        param_groups = [{"params": [p for p in model.parameters()], "weight_decay": 0.0}]
    engine, optimizer, _, lr_scheduler = engine_initialize(model, neox_args, param_groups=param_groups,
                                                           optimizer_cfg=cfg, lr_scheduler=lr_scheduler,
                                                           generic_optimizer=generic)
    if reference_model is not None:
        ref_engine, _, _, _ = engine_initialize(reference_model, neox_args, param_groups=[
            {"params": list(reference_model.parameters()), "weight_decay": 0.0}], optimizer_cfg=None)
        for p in reference_model.parameters():
            p.requires_grad = False
        reference_model = ref_engine
    mark_norms_for_sequence_parallel_grad_sync(engine.module, neox_args)
    engine.total_params_count = engine.total_params if engine.groups else sum(p.numel() for p in engine.module.parameters())
    print_rank_0(f' > number of parameters on model parallel rank {mpu.get_model_parallel_rank()}: '
                 f'{engine.total_params_count}')
    curr_scheduler = None
    if neox_args.curriculum_learning:
        from .engine.curriculum import CurriculumScheduler
        curr_scheduler = CurriculumScheduler(neox_args.curriculum_learning)
        if iteration is not None and iteration > 0:
            curr_scheduler.update_difficulty(iteration)
    engine.curriculum_scheduler = curr_scheduler
    if neox_args.is_pipe_parallel:
        engine.set_has_attention_mask(True)
        engine.set_batch_fn(partial(get_batch_pipe, neox_args=neox_args, curr_scheduler=curr_scheduler))
    if neox_args.load is not None:
        neox_args.iteration = load_checkpoint(neox_args=neox_args, model=engine, optimizer=optimizer,
                                              lr_scheduler=lr_scheduler, iteration=iteration)
        if reference_model is not None:
            load_checkpoint(neox_args=neox_args, model=reference_model, optimizer=None, lr_scheduler=None,
                            iteration=iteration)
            reference_model.eval()
        print_rank_0(f"Loading checkpoint and starting from iteration {neox_args.iteration}")
    else:
        neox_args.iteration = 0
    if lr_scheduler is not None:
        lr_scheduler.optimizer = engine.optimizer
    return engine, optimizer, lr_scheduler, reference_model


# ----------------------------------------------------------------------------------------- steps
def backward_step(neox_args, timers, optimizer, model, loss):
    timers("backward-backward").start()
    model.backward(loss)
    timers("backward-backward").stop()


def train_step(neox_args, timers, data_iterator, model, optimizer, lr_scheduler, reference_model=None):
    """One optimizer step = ``gradient_accumulation_steps`` micro-batches."""
    if neox_args.is_pipe_parallel:
        reduced_loss = train_step_pipe(neox_args=neox_args, timers=timers, model=model, data_iterator=data_iterator)
        reduce_metrics = reduced_loss
        if neox_args.memory_profiling and neox_args.iteration >= neox_args.profile_step_stop and \
                torch.distributed.get_rank() == 0:
            save_snapshot(neox_args)
    else:
        losses, metric_dicts = [], {}
        for _ in range(neox_args.gradient_accumulation_steps):
            timers("forward").start()
            loss, metric_dict = forward_step(neox_args=neox_args, timers=timers, data_iterator=data_iterator,
                                             model=model, is_train=True, reference_model=reference_model)
            timers("forward").stop()
            losses.append(loss.detach())
            for k, v in metric_dict.items():
                metric_dicts.setdefault(k, []).append(v)
            _nvtx_push(neox_args, "Backward pass")
            timers("backward").start()
            backward_step(neox_args=neox_args, timers=timers, optimizer=optimizer, model=model, loss=loss)
            timers("backward").stop()
            _nvtx_pop(neox_args)
            _nvtx_push(neox_args, "Optimizer step")
            timers("optimizer").start()
            if neox_args.deepspeed:
                model.step()
            else:
                raise ValueError("Must be using deepspeed to run neox")
            timers("optimizer").stop()
            _nvtx_pop(neox_args)
            if neox_args.memory_profiling and neox_args.iteration >= neox_args.profile_step_stop and \
                    dist.get_rank() == 0:
                save_snapshot(neox_args)
        reduce_metrics = {k: reduce_losses(v).mean() for k, v in metric_dicts.items()}
        reduce_metrics["lm_loss"] = reduce_losses(losses).mean()
    if neox_args.precision == "fp16" and model.optimizer is not None and model.optimizer.overflow:
        skipped_iter = 1
    else:
        skipped_iter = 0
    collect_loss_for_unit_test(reduce_metrics["lm_loss"])
    return reduce_metrics, skipped_iter


def train_step_pipe(neox_args, timers, model, data_iterator):
    assert neox_args.deepspeed
    loss = model.train_batch(data_iter=data_iterator)
    loss_dict = {"lm_loss": loss}
    for t in ["forward", "backward", "allreduce", "optimizer", "batch generator", "data loader"]:
        timers(t).reset()
    return loss_dict


def is_save_iter(neox_args, iteration):
    """``extra_save_iters`` | every ``checkpoint_factor`` steps (linear) | powers of
    ``checkpoint_factor`` (log)."""
    if neox_args.extra_save_iters and iteration in neox_args.extra_save_iters:
        return True
    if neox_args.checkpoint_factor:
        if neox_args.checkpoint_scale == "linear":
            assert float(neox_args.checkpoint_factor).is_integer(), "checkpoint_factor must be a whole number when using linear checkpoint_scale"
            return iteration % neox_args.checkpoint_factor == 0
        if neox_args.checkpoint_scale == "log":
            assert neox_args.checkpoint_factor > 1, "checkpoint_factor must be greater than 1 when using log checkpoint_scale"
            power = 1
            while power < iteration + 1:
                if int(power) == iteration:
                    return True
                power *= neox_args.checkpoint_factor
    return False


def train(neox_args, timers, model, optimizer, lr_scheduler, train_data_iterator, valid_data_iterator,
          reference_model=None):
    model.train()
    total_loss_dict = {}
    iteration = neox_args.iteration
    timers("interval time").start()
    report_memory_flag = True
    noise_scale_logger = get_noise_scale_logger(neox_args, model)
    overflow_monitor = OverflowMonitor(optimizer)
    prof = None
    if neox_args.profile:
        schedule = torch.profiler.schedule(wait=neox_args.profile_step_start, warmup=1,
                                           active=neox_args.profile_step_stop - neox_args.profile_step_start)
        prof = torch.profiler.profile(schedule=schedule,
                                      on_trace_ready=torch.profiler.tensorboard_trace_handler(neox_args.tensorboard_dir),
                                      record_shapes=True, profile_memory=True, with_flops=True, with_modules=True,
                                      with_stack=True)
        prof.start()
    from .obs import heartbeat as _hb
    hb = _hb.from_args(neox_args)
    from .autotuning import ProfileWindow
    window, first_iteration = ProfileWindow.from_args(neox_args), iteration
    while iteration < neox_args.train_iters:
        if hb is not None:
            hb.beat(iteration, "train_step")
        if neox_args.profile:
            prof.step()
        if neox_args.profile and iteration == neox_args.profile_step_start and torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStart()
        loss_dict, skipped_iter = train_step(neox_args=neox_args, timers=timers, data_iterator=train_data_iterator,
                                             model=model, optimizer=optimizer, lr_scheduler=lr_scheduler,
                                             reference_model=reference_model)
        if neox_args.profile and iteration == neox_args.profile_step_stop and torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStop()
            prof.stop()
        iteration += 1
        neox_args.iteration = iteration
        if window is not None and window.after_step(iteration - first_iteration,
                                                    dist.get_rank() if dist.is_initialized() else 0):
            print_rank_0(f"autotuning: profile window closed after {iteration - first_iteration} steps, exiting")
            if dist.is_initialized():
                dist.barrier()
            sys.exit(0)
        if iteration % max(1, neox_args.log_interval) == 0:
            if torch.cuda.is_available():
                # a bounded wait inside a communication kernel that ran out surfaces here as an exception
                from .ops import _lib as _klib
                _klib.raise_on_device_error()
            if hb is not None and torch.distributed.get_rank() == 0:
                for s_ in hb.stragglers():
                    print_rank_0(f"heartbeat: rank {s_['rank']}: {s_['reason']}")
        if neox_args.precision == "fp16":
            overflow_monitor.check(skipped_iter)
        if neox_args.log_gradient_noise_scale and noise_scale_logger is not None:
            noise_scale_logger.update()
        if optimizer is not None and optimizer.param_groups:
            lr = optimizer.param_groups[0].get("lr", 0)
        else:
            lr = 0
        report_memory_flag = training_log(neox_args=neox_args, timers=timers, loss_dict=loss_dict,
                                          total_loss_dict=total_loss_dict, learning_rate=lr, iteration=iteration,
                                          loss_scale=model.cur_scale if neox_args.precision == "fp16" else None,
                                          report_memory_flag=report_memory_flag, skipped_iter=skipped_iter,
                                          model=model, optimizer=optimizer, noise_scale_logger=noise_scale_logger)
        saving = neox_args.save and is_save_iter(neox_args, iteration)
        evaluating = neox_args.eval_interval and iteration % neox_args.eval_interval == 0 and neox_args.do_valid
        if (saving or evaluating) and torch.cuda.is_available():
            # never write or score weights that a timed-out communication kernel may have left invalid
            from .ops import _lib as _klib
            _klib.raise_on_device_error()
        if saving:
            save_checkpoint(neox_args=neox_args, iteration=iteration, model=model, optimizer=optimizer,
                            lr_scheduler=lr_scheduler)
        if evaluating:
            prefix = "iteration {}".format(iteration)
            evaluate_and_print_results(neox_args=neox_args, prefix=prefix, forward_step_func=forward_step,
                                       data_iterator=valid_data_iterator, model=model, iteration=iteration,
                                       verbose=False, timers=timers, reference_model=reference_model)
        if neox_args.exit_interval and iteration % neox_args.exit_interval == 0:
            if dist.is_initialized():
                dist.barrier()
            time_str = time.strftime("%Y-%m-%d %H:%M:%S")
            rank = dist.get_rank() if dist.is_initialized() else 0
            print_rank_0("rank: {} | time: {} | exiting the program at iteration {}".format(rank, time_str, iteration))
            sys.exit()
    return iteration


def evaluate(neox_args, forward_step_fn, data_iterator, model, verbose=False, timers=None, reference_model=None):
    """Mean loss (and perplexity, optional char-level perplexity, eval-harness tasks) over
    ``eval_iters`` steps."""
    model.eval()
    losses, metric_dicts = [], {}
    if neox_args.char_level_ppl:
        data_iterator = CharCounter(data_iterator, neox_args.tokenizer)
    with torch.no_grad():
        iteration = 0
        while iteration < neox_args.eval_iters:
            iteration += 1
            if verbose and iteration % neox_args.log_interval == 0:
                print_rank_0("Evaluating iter {}/{}".format(iteration, neox_args.eval_iters))
            for _ in range(1 if neox_args.is_pipe_parallel else neox_args.gradient_accumulation_steps):
                out = forward_step_fn(model=model, data_iterator=data_iterator, neox_args=neox_args, timers=timers,
                                      reference_model=reference_model)
                if neox_args.is_pipe_parallel:
                    loss, metric_dict = out if isinstance(out, tuple) and len(out) == 2 and isinstance(out[1], dict) \
                        else (out, {})
                else:
                    loss, metric_dict = out
                losses.append(loss if torch.is_tensor(loss) else torch.tensor(float(loss)))
                for k, v in metric_dict.items():
                    metric_dicts.setdefault(k, []).append(v)
    eval_results = {"lm_loss": reduce_losses(losses).mean().item()}
    for k, v in metric_dicts.items():
        eval_results[k] = reduce_losses(v).mean().item()
    eval_results["lm_loss_ppl"] = math.exp(min(eval_results["lm_loss"], 50))
    if neox_args.char_level_ppl:
        tokens_per_char = data_iterator.tokens_per_char()
        print_rank_0(f"Counting chars took {data_iterator.total_time} seconds")
        data_iterator = data_iterator.data_iterator
        eval_results["lm_loss_char_lvl_ppl"] = math.exp(eval_results["lm_loss"] * tokens_per_char)
    if neox_args.eval_tasks:
        from .eval_tasks import run_eval_harness
        eval_results.update(run_eval_harness(model, forward_step_fn, neox_args,
                                             eval_tasks=neox_args.eval_tasks).get("results"))
    model.train()
    return eval_results


def evaluate_and_print_results(neox_args, prefix, forward_step_func, data_iterator, model, iteration, verbose=False,
                               timers=None, chart_name="validation", reference_model=None):
    total_loss_dict = evaluate(neox_args=neox_args, forward_step_fn=forward_step_func, data_iterator=data_iterator,
                               model=model, verbose=verbose, timers=timers, reference_model=reference_model)
    string = f" {chart_name} results at {prefix} | "
    sinks = dict(use_wandb=neox_args.use_wandb, tensorboard_writer=getattr(neox_args, "tensorboard_writer", None),
                 comet_experiment=getattr(neox_args, "comet_experiment", None))
    for k, v in total_loss_dict.items():
        if isinstance(v, dict):
            if neox_args.eval_tasks and "results" in v:
                v = v["results"]
            for k2, v2 in v.items():
                k3 = "_".join([k, k2])
                string += f"{k3} value: {v2:.6E} | "
                tb_wandb_log(f"{chart_name}/{k3}", v2, iteration, **sinks)
        else:
            string += f"{k} value: {v:.6E} | "
            tb_wandb_log(f"{chart_name}/{k}", v, iteration, **sinks)
    length = len(string) + 1
    print_rank_0("-" * length)
    print_rank_0(string)
    print_rank_0("-" * length)


def get_noise_scale_logger(neox_args, model=None):
    if not neox_args.log_gradient_noise_scale:
        return None
    from .gradient_noise_scale import GradientNoiseScale
    if model is not None:
        model.store_gradients = True
    return GradientNoiseScale(model=model, batch_size_small=neox_args.train_batch_size,
                              n_batches=neox_args.gradient_noise_scale_n_batches,
                              cpu_offload=neox_args.gradient_noise_scale_cpu_offload, neox_args=neox_args, mpu=mpu)


def save_snapshot(neox_args):
    assert neox_args.memory_profiling_path is not None, "Must pass memory_profiling_path config arg to use profiling"
    import os
    import pickle
    snapshot = torch.cuda.memory._snapshot()
    snapshot_path = os.path.join(neox_args.memory_profiling_path)
    os.makedirs(snapshot_path, exist_ok=True)
    with open(os.path.join(snapshot_path, "mem_snapshot.pickle"), "wb") as f:
        pickle.dump(snapshot, f)


def collect_loss_for_unit_test(lm_ss):
    """Hook patched by tests to observe the loss curve."""
    pass

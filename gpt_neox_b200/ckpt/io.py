"""Engine-level checkpoint files, in the layout the ``tools/ckpts`` converters read
(tools/ckpts/convert_neox_to_hf.py:204-238, tools/ckpts/merge20b.py:62-80):

  <dir>/latest                                      the newest tag
  <dir>/<tag>/mp_rank_<MP:02d>_model_states.pt      per tensor-parallel rank: ``module`` state dict
        (keys ``sequential.<idx>.<param>`` without pipeline parallelism; ``None`` with it), step
        counters, lr-scheduler state, data/model-parallel sizes and the caller's client state
  <dir>/<tag>/layer_<IDX:02d>-model_<MP:02d>-model_states.pt   pipeline runs: one file per layer
  <dir>/<tag>/zero_pp_rank_<DP>_mp_rank_<MP:02d>_optim_states.pt   optimizer shard of each rank
  <dir>/<tag>/expert_ep_rank_<EP:02d>_mp_rank_<MP:02d>_model_states.pt   expert parallelism > 1: the expert
        parameters of one expert-parallel rank (the per-MP-rank file above is written by data-parallel rank 0 and
        therefore only holds expert-parallel rank 0's experts)

Writes are atomic at directory level: every rank writes into ``<tag>.tmp``, then rank 0 renames it
and rewrites ``latest``; a crash never leaves a half-written tag behind ``latest``.
"""
from __future__ import annotations

import os
import re
import shutil

import torch
import torch.distributed as dist

from .. import parallel as mpu


def _barrier():
    if dist.is_initialized():
        dist.barrier()


def _rank():
    return dist.get_rank() if dist.is_initialized() else 0


def model_states_name(mp_rank: int) -> str:
    return f"mp_rank_{mp_rank:02d}_model_states.pt"


def layer_file_name(layer_idx: int, mp_rank: int) -> str:
    return f"layer_{layer_idx:02d}-model_{mp_rank:02d}-model_states.pt"


def optim_states_name(dp_rank: int, mp_rank: int, bf16: bool = False) -> str:
    prefix = "bf16_" if bf16 else ""
    return f"{prefix}zero_pp_rank_{dp_rank}_mp_rank_{mp_rank:02d}_optim_states.pt"


def expert_states_name(ep_rank: int, mp_rank: int, pp_rank: int = None) -> str:
    stage = "" if pp_rank is None else f"_pp{pp_rank:02d}"
    return f"expert_ep_rank_{ep_rank:02d}_mp_rank_{mp_rank:02d}{stage}_model_states.pt"


def _expert_param_names(module):
    return [n for n, p in module.named_parameters() if getattr(p, "expert_parallel", False)]


def _expert_state_dict(module):
    names = set(_expert_param_names(module))
    return {k: v.detach().cpu() for k, v in module.state_dict().items() if k in names}


def _module_state_dict(engine):
    with engine.gathered_parameters():             # ZeRO stage 3 keeps only slices between uses
        sd = engine.module.state_dict()
        return {k: v.detach().cpu() for k, v in sd.items()}


def _pipe_layer_states(module):
    """{global layer index: state dict with bare parameter names} for this stage's layers."""
    out = {}
    for name, child in module.named_children():
        if name.isdigit():
            out[int(name)] = {k: v.detach().cpu() for k, v in child.state_dict().items()}
    tied = getattr(module, "tied_modules", None)
    if tied is not None:
        for key, mod in tied.items():
            for idx, spec in enumerate(module.specs):
                if getattr(spec, "key", None) == key and module._local_start <= idx < module._local_stop:
                    out[idx] = {k: v.detach().cpu() for k, v in mod.state_dict().items()}
    return out


def save_engine_checkpoint(engine, save_dir, tag=None, client_state=None):
    tag = tag or f"global_step{engine.global_steps}"
    final_dir = os.path.join(save_dir, str(tag))
    tmp_dir = final_dir + ".tmp"
    if _rank() == 0:
        if os.path.isdir(tmp_dir):
            shutil.rmtree(tmp_dir)
        os.makedirs(tmp_dir, exist_ok=True)
    _barrier()
    os.makedirs(tmp_dir, exist_ok=True)
    mp_rank, dp_rank, pp_rank = mpu.get_model_parallel_rank(), mpu.get_data_parallel_rank(), mpu.get_pipe_parallel_rank()
    is_pipe = engine.neox_args.is_pipe_parallel
    if is_pipe:
        if dp_rank == 0:
            for idx, sd in _pipe_layer_states(engine.module).items():
                torch.save(sd, os.path.join(tmp_dir, layer_file_name(idx, mp_rank)))
    # collective under ZeRO stage 3 (the parameters are gathered): every rank takes part, rank 0 of the replicas writes
    module_sd = None if is_pipe else _module_state_dict(engine)
    if dp_rank == 0 and (pp_rank == 0 or not is_pipe):
        state = {
            "module": None if is_pipe else module_sd,
            "optimizer": None,
            "lr_scheduler": engine.lr_scheduler.state_dict() if engine.lr_scheduler is not None else None,
            "dp_world_size": mpu.get_data_parallel_world_size(),
            "mp_world_size": mpu.get_model_parallel_world_size(),
            "global_steps": engine.global_steps,
            "global_samples": engine.global_samples,
            "skipped_steps": engine.skipped_steps,
            "loss_scaler": engine.loss_scaler.state_dict(),
        }
        state.update(client_state or {})
        torch.save(state, os.path.join(tmp_dir, model_states_name(mp_rank)))
    ep = mpu.get_expert_parallel_world_size()
    if ep > 1 and dp_rank < ep:        # one writer per expert-parallel rank (expert-DP rank 0), per pipeline stage
        esd = _expert_state_dict(engine.module)
        if esd:
            torch.save(esd, os.path.join(tmp_dir, expert_states_name(mpu.get_expert_parallel_rank(), mp_rank,
                                                                     pp_rank if is_pipe else None)))
    if engine.optimizer is not None:
        name = optim_states_name(dp_rank + pp_rank * 0, mp_rank, bf16=engine.bfloat16_enabled)
        if is_pipe:
            name = name.replace(".pt", f"_pp{pp_rank:02d}.pt") if mpu.get_pipe_parallel_world_size() > 1 else name
        torch.save({"optimizer_state_dict": engine.optimizer.state_dict(),
                    "zero_stage": engine.zero_stage,
                    "partition_count": mpu.get_data_parallel_world_size()}, os.path.join(tmp_dir, name))
    _barrier()
    if _rank() == 0:
        if os.path.isdir(final_dir):
            shutil.rmtree(final_dir)
        os.rename(tmp_dir, final_dir)
        with open(os.path.join(save_dir, "latest.tmp"), "w") as f:
            f.write(str(tag))
            f.flush()
            os.fsync(f.fileno())
        os.replace(os.path.join(save_dir, "latest.tmp"), os.path.join(save_dir, "latest"))
    _barrier()
    return True


def read_latest_tag(load_dir):
    p = os.path.join(load_dir, "latest")
    if not os.path.isfile(p):
        return None
    with open(p) as f:
        return f.read().strip()


def load_engine_checkpoint(engine, load_dir, tag=None, load_optimizer_states=True, load_lr_scheduler_states=True,
                           load_module_only=False, load_module_strict=True):
    """-> (path or None, client_state dict)."""
    if tag is None:
        tag = read_latest_tag(load_dir)
        if tag is None:
            return None, {}
    ckpt_dir = os.path.join(load_dir, str(tag))
    mp_rank, dp_rank, pp_rank = mpu.get_model_parallel_rank(), mpu.get_data_parallel_rank(), mpu.get_pipe_parallel_rank()
    ms_path = os.path.join(ckpt_dir, model_states_name(mp_rank))
    if not os.path.isfile(ms_path):
        # a tag that was named (by the caller or by the `latest` file) but is not there is damage, not a
        # fresh start: refuse instead of silently training from scratch over an existing run directory
        raise FileNotFoundError(f"checkpoint {ckpt_dir} is named by "
                                f"{'the caller' if tag is None else 'tag ' + repr(str(tag))} but {ms_path} is missing")
    state = torch.load(ms_path, map_location="cpu", weights_only=False)
    is_pipe = engine.neox_args.is_pipe_parallel
    if is_pipe:
        module = engine.module
        for name, child in module.named_children():
            if name.isdigit():
                f = os.path.join(ckpt_dir, layer_file_name(int(name), mp_rank))
                child.load_state_dict(torch.load(f, map_location="cpu", weights_only=False), strict=load_module_strict)
        tied = getattr(module, "tied_modules", None)
        if tied is not None:
            for key, mod in tied.items():
                for idx, spec in enumerate(module.specs):
                    if getattr(spec, "key", None) == key:
                        f = os.path.join(ckpt_dir, layer_file_name(idx, mp_rank))
                        if os.path.isfile(f):
                            mod.load_state_dict(torch.load(f, map_location="cpu", weights_only=False),
                                                strict=load_module_strict)
                            break
    else:
        sd = state["module"]
        with engine.gathered_parameters(write_back=True):
            _load_into_flat(engine.module, sd, strict=load_module_strict)
    if mpu.get_expert_parallel_world_size() > 1 and _expert_param_names(engine.module):
        ef = os.path.join(ckpt_dir, expert_states_name(mpu.get_expert_parallel_rank(), mp_rank,
                                                       pp_rank if is_pipe else None))
        if os.path.isfile(ef):
            _load_into_flat(engine.module, torch.load(ef, map_location="cpu", weights_only=False), strict=False)
        elif mpu.get_expert_parallel_rank() > 0:
            raise FileNotFoundError(f"{ef} is missing: the checkpoint holds no experts for expert-parallel "
                                    f"rank {mpu.get_expert_parallel_rank()}")
    for g in engine.groups:
        g.refresh_master_from_lp()
    if not load_module_only:
        engine.global_steps = state.get("global_steps", 0)
        engine.global_samples = state.get("global_samples", 0)
        engine.skipped_steps = state.get("skipped_steps", 0)
        if "loss_scaler" in state:
            engine.loss_scaler.load_state_dict(state["loss_scaler"])
        if load_lr_scheduler_states and engine.lr_scheduler is not None and state.get("lr_scheduler") is not None:
            engine.lr_scheduler.load_state_dict(state["lr_scheduler"])
        if load_optimizer_states and engine.optimizer is not None:
            name = optim_states_name(dp_rank, mp_rank, bf16=engine.bfloat16_enabled)
            if is_pipe and mpu.get_pipe_parallel_world_size() > 1:
                name = name.replace(".pt", f"_pp{pp_rank:02d}.pt")
            p = os.path.join(ckpt_dir, name)
            ok = False
            if os.path.isfile(p) and state.get("dp_world_size") == mpu.get_data_parallel_world_size():
                osd = torch.load(p, map_location="cpu", weights_only=False)
                ok = engine.optimizer.load_state_dict(osd["optimizer_state_dict"])
            if not ok:
                # data-parallel size changed (elastic restart): re-partition the optimizer state
                ok = _reshard_optimizer_state(engine, ckpt_dir, mp_rank, pp_rank, is_pipe)
            if not ok and _rank() == 0:
                print("WARNING: optimizer state could not be restored; moments start from zero", flush=True)
    reserved = {"module", "optimizer", "lr_scheduler", "dp_world_size", "mp_world_size", "global_steps",
                "global_samples", "skipped_steps", "loss_scaler"}
    client_state = {k: v for k, v in state.items() if k not in reserved}
    return ckpt_dir, client_state


def _load_into_flat(module, sd, strict=True):
    """``load_state_dict`` that copies into the existing (flat-buffer backed) parameter storage."""
    own = module.state_dict()
    missing = [k for k in own if k not in sd]
    unexpected = [k for k in sd if k not in own]
    if strict and (missing or unexpected):
        raise RuntimeError(f"state dict mismatch: missing {missing[:5]} unexpected {unexpected[:5]}")
    with torch.no_grad():
        for k, v in sd.items():
            if k in own:
                own[k].copy_(v.to(own[k].dtype))


def _reshard_optimizer_state(engine, ckpt_dir, mp_rank, pp_rank, is_pipe):
    """Rebuild this rank's shard of (master, exp_avg, exp_avg_sq) from the shards of a run with a
    different data-parallel size: concatenate the old shards into the full flat vector, cut anew."""
    pat = re.compile(r"(bf16_)?zero_pp_rank_(\d+)_mp_rank_%02d_optim_states(_pp%02d)?\.pt$" % (mp_rank, pp_rank))
    files = {}
    for f in os.listdir(ckpt_dir):
        m = pat.match(f)
        if m and (bool(m.group(3)) == (is_pipe and mpu.get_pipe_parallel_world_size() > 1)):
            files[int(m.group(2))] = os.path.join(ckpt_dir, f)
    if not files:
        return False
    sds = [torch.load(files[i], map_location="cpu", weights_only=False)["optimizer_state_dict"] for i in sorted(files)]
    for gi, g in enumerate(engine.groups):
        full = {}
        eight_bit = g.state_bits == 8 or sds[0]["shards"][gi]["exp_avg"].dtype == torch.uint8
        if eight_bit:
            # 8-bit moments are codes relative to per-segment block scales: they do not survive a re-partition.
            # The master weights are re-cut; the moments restart from zero.
            print("WARNING: 8-bit optimizer moments are not re-partitioned across a data-parallel resize; "
                  "they restart from zero", flush=True)
            for t in (g.exp_avg, g.exp_avg_sq, *(g.q8_scales or [])):
                t.zero_()
        for key in (("master",) if eight_bit else ("master", "exp_avg", "exp_avg_sq")):
            parts = [s["shards"][gi][key] for s in sds]
            full[key] = torch.cat(parts) if sds[0]["shards"][gi]["shard_size"] != sds[0]["shards"][gi]["total"] else parts[0]
        n_used = g.offsets[-1] + g.params[-1].numel() if g.params else 0
        for key, dst in (("exp_avg", g.exp_avg), ("exp_avg_sq", g.exp_avg_sq), ("master", g.master)):
            if key not in full:
                continue
            src = torch.zeros(g.total, dtype=torch.float32)
            n = min(full[key].numel(), g.total)
            src[:n] = full[key][:n]
            if key == "master" and g.lp_dtype == torch.float32:
                continue
            dst.copy_(src[g.shard_start:g.shard_start + g.shard_size])
        del n_used
    engine.optimizer.step_count = sds[0].get("step", 0)
    return True

"""Pipeline-parallel engine: 1F1B schedule over NCCL (or gloo) point-to-point transfers.

What the reference gets from DeepSpeed's PipelineEngine through ``model.train_batch`` /
``model.eval_batch`` (megatron/training.py:1389-1405, 543-544).  Each stage owns a contiguous slice
of the layer list (``GPT2ModelPipe.forward_stage``); a step runs ``gradient_accumulation_steps``
micro-batches: ``min(stages - stage - 1, M)`` warm-up forwards, then one-forward-one-backward, then
the cool-down backwards.  Only the hidden states cross a stage boundary: the causal mask is rebuilt
on the receiver instead of being shipped with every micro-batch (the reference sends the dense
[1,1,s,s] mask along, megatron/model/gpt2_model.py:220-223).  Send and receive of one exchange are
issued as one batched p2p group so that neighbouring stages never wait on each other's sends; an
exchange that only sends is not waited for until the next exchange has been posted, so the compute
stream runs on while the activation or gradient is in flight.  (Between two stages of one NVSwitch
node a transfer of the sequence-parallel shard takes tens of microseconds against milliseconds of
compute per micro-batch: the cost of the schedule is its (stages - 1) / (micro-batches + stages - 1)
bubble, not the transfers.)
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import parallel as mpu
from ..utils.common import get_attn_mask
from .engine import Engine

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.uint8, torch.bool]


class _StageGrid:
    """The pipeline group this rank belongs to, as generation / evaluation code addresses it
    (``engine.grid.stage_to_global(stage)`` -> global rank of that stage in this rank's pipeline)."""

    def __init__(self, ranks):
        self.ranks = list(ranks)

    def stage_to_global(self, stage_id: int) -> int:
        return self.ranks[stage_id]


class PipelineEngine(Engine):
    def __init__(self, module, neox_args, param_groups, optimizer_cfg=None, lr_scheduler=None,
                 generic_optimizer=None):
        super().__init__(module, neox_args, param_groups, optimizer_cfg, lr_scheduler, generic_optimizer)
        self.num_stages = mpu.get_pipe_parallel_world_size()
        self.stage_id = mpu.get_pipe_parallel_rank()
        ranks = mpu.get_pipe_parallel_ranks()
        self.grid = _StageGrid(ranks)
        self.prev_rank = ranks[self.stage_id - 1] if self.stage_id > 0 else None
        self.next_rank = ranks[self.stage_id + 1] if self.stage_id < self.num_stages - 1 else None
        self.micro_batches = neox_args.gradient_accumulation_steps
        self.batch_fn = None
        self.has_attention_mask = True
        self._recv_meta = None          # (shape, dtype) of the activation arriving from the previous stage
        self._sent_meta = False
        self.first_output_send = True
        self._pending_sends = []         # (requests, tensors) of send-only exchanges not waited for yet
        self.pipe_recv_buf = None
        self.is_pipe_parallel = True
        self._needs_mask = any(t not in ("flash", "rwkv", "mamba") for t in (neox_args.attention_config or []))
        self.timer_values = None
        self._tied = self._find_tied()

    # ------------------------------------------------------------------ helpers
    def is_first_stage(self):
        return self.stage_id == 0

    def is_last_stage(self):
        return self.stage_id == self.num_stages - 1

    def _device(self):
        return next(self.module.parameters()).device

    def _find_tied(self):
        """Tied modules of this stage and the (first stage, last stage) group their gradients are summed
        over. ``new_group`` is collective, so every rank walks every pipe line of the topology."""
        self._tied_group = None
        if self.neox_args.no_weight_tying or self.num_stages == 1 or not dist.is_initialized():
            return []
        me = dist.get_rank()
        for ranks in mpu.get_topology().get_axis_comm_lists("pipe"):
            g = dist.new_group([ranks[0], ranks[-1]])
            if me in (ranks[0], ranks[-1]):
                self._tied_group = g
        tied = getattr(self.module, "tied_modules", None)
        return list(tied.values()) if tied is not None and len(tied) > 0 else []

    def _expects_tuple(self):
        start = self.module._local_start
        return 1 <= start <= self.neox_args.num_layers + 2

    def _wrap_input(self, hidden):
        if not self._expects_tuple():
            return hidden
        mask = None
        if self._needs_mask:
            seq = hidden.shape[0] if self.module._local_start >= 2 else hidden.shape[1]
            mask = get_attn_mask(seq, hidden.device, self.neox_args.sliding_window_width)
        return (hidden, mask)

    @staticmethod
    def _unwrap_output(out):
        return out[0] if isinstance(out, tuple) else out

    # ------------------------------------------------------------------ p2p
    def _send_meta(self, t, dst):
        meta = torch.zeros(8, dtype=torch.int64, device=t.device)
        meta[0] = t.dim()
        meta[1] = _DTYPES.index(t.dtype)
        for i, s in enumerate(t.shape):
            meta[2 + i] = s
        for req in dist.batch_isend_irecv([dist.P2POp(dist.isend, meta, dst)]):     # batched: same NCCL path as the
            req.wait()                                                              # tensors, no lone send / recv

    def _recv_meta_from(self, src):
        meta = torch.zeros(8, dtype=torch.int64, device=self._device())
        for req in dist.batch_isend_irecv([dist.P2POp(dist.irecv, meta, src)]):
            req.wait()
        meta = meta.tolist()
        return tuple(meta[2:2 + meta[0]]), _DTYPES[meta[1]]

    def _exchange(self, send_next=None, send_prev=None, recv_prev=False, recv_next=False):
        """One batched group of point-to-point operations; returns (from_prev, from_next)."""
        with self._span("pipe_comm"):
            return self._exchange_now(send_next, send_prev, recv_prev, recv_next)

    def _exchange_now(self, send_next, send_prev, recv_prev, recv_next):
        ops, from_prev, from_next = [], None, None
        if send_next is not None and self.next_rank is not None:
            if not self._sent_meta:
                self._send_meta(send_next, self.next_rank)
                self._sent_meta = True
            ops.append(dist.P2POp(dist.isend, send_next.contiguous(), self.next_rank))
        if recv_prev and self.prev_rank is not None:
            if self._recv_meta is None:
                self._recv_meta = self._recv_meta_from(self.prev_rank)
            shape, dtype = self._recv_meta
            from_prev = torch.empty(shape, dtype=dtype, device=self._device())
            ops.append(dist.P2POp(dist.irecv, from_prev, self.prev_rank))
        if send_prev is not None and self.prev_rank is not None:
            ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), self.prev_rank))
        if recv_next and self.next_rank is not None:
            from_next = torch.empty(self._out_shape, dtype=self._out_dtype, device=self._device())
            ops.append(dist.P2POp(dist.irecv, from_next, self.next_rank))
        if ops:
            reqs = dist.batch_isend_irecv(ops)
            # requests of earlier send-only groups are settled after the new operations are posted (so a
            # neighbour that is waiting for this rank's receive is never kept waiting by them)
            self._settle_sends()
            if from_prev is None and from_next is None:
                # nothing arrives in this group: the compute stream does not wait for the send to finish; the
                # tensors stay referenced until the request is settled at the next exchange
                self._pending_sends.append((reqs, [op.tensor for op in ops]))
            else:
                for req in reqs:
                    req.wait()
        return from_prev, from_next

    def _settle_sends(self):
        pending, self._pending_sends = self._pending_sends, []
        for reqs, _tensors in pending:
            for req in reqs:
                req.wait()

    # ------------------------------------------------------------------ one micro-batch
    def _forward_micro(self, recv, data_iter, losses, keep_logits=None):
        labels = None
        if self.is_first_stage() or self.is_last_stage():
            batch = next(data_iter) if data_iter is not None else None   # only tensor-rank 0 reads data
            inputs, labels = self.batch_fn(batch) if self.batch_fn is not None else batch
        if self.is_first_stage():
            x = inputs
            inp = None
        else:
            inp = recv.requires_grad_(torch.is_grad_enabled())
            x = self._wrap_input(inp)
        if self.flops_profiler is not None and self.module.training:
            self.flops_profiler.before_forward(self.global_steps + 1)
        with self._span("forward"):
            out = self._unwrap_output(self.module.forward_stage(x))
            loss = self.module.loss_fn(out, labels) if self.is_last_stage() else None
        if self.is_last_stage():
            if keep_logits is not None:
                keep_logits.append(out)
            losses.append(loss.detach())
            out = loss / self.micro_batches
        else:
            self._out_shape, self._out_dtype = tuple(out.shape), out.dtype
        return inp, out

    def _backward_micro(self, inp, out, out_grad):
        with self._span("backward"):
            return self._backward_now(inp, out, out_grad)

    def _backward_now(self, inp, out, out_grad):
        if self.is_last_stage():
            scaled = out * self.loss_scaler.cur_scale if self.fp16_enabled else out
            scaled.backward()
        else:
            torch.autograd.backward(out, out_grad)
        return inp.grad if inp is not None else None

    # ------------------------------------------------------------------ public API
    def train_batch(self, data_iter=None):
        self.module.train()
        M, S, s = self.micro_batches, self.num_stages, self.stage_id
        warmup = min(S - s - 1, M)
        remaining = M - warmup
        losses, queue = [], []
        for _ in range(warmup):
            recv, _ = self._exchange(recv_prev=True)
            inp, out = self._forward_micro(recv, data_iter, losses)
            self._exchange(send_next=None if self.is_last_stage() else out)
            queue.append((inp, out))
        recv = None
        if remaining > 0:
            recv, _ = self._exchange(recv_prev=True)
        for i in range(remaining):
            inp, out = self._forward_micro(recv, data_iter, losses)
            _, out_grad = self._exchange(send_next=None if self.is_last_stage() else out, recv_next=True)
            queue.append((inp, out))
            inp0, out0 = queue.pop(0)
            in_grad = self._backward_micro(inp0, out0, out_grad)
            if i == remaining - 1:
                self._exchange(send_prev=in_grad)
                recv = None
            else:
                recv, _ = self._exchange(send_prev=in_grad, recv_prev=True)
        for _ in range(warmup):
            inp0, out0 = queue.pop(0)
            _, out_grad = self._exchange(recv_next=True)
            in_grad = self._backward_micro(inp0, out0, out_grad)
            self._exchange(send_prev=in_grad)
        self._settle_sends()
        self._sync_tied_grads()
        self.micro_steps += M - 1          # _take_model_step is the boundary micro-step
        self.micro_steps += 1
        self.global_samples += self.neox_args.train_batch_size
        self._take_model_step()
        return self._aggregate_loss(losses)

    def _forget_shapes(self):
        """The shape of the activations between stages is announced once and then assumed; evaluation and
        generation feed other batch shapes than training does (and change them from call to call), so the
        announcement is repeated around every such call.  Both neighbours reset at the same points."""
        self._recv_meta = None
        self._sent_meta = False

    def eval_batch(self, data_iter, return_logits=False):
        was_training = self.module.training
        self.module.eval()
        self._forget_shapes()
        losses, logits = [], []
        micro = 1 if return_logits else self.micro_batches
        with torch.no_grad():
            for _ in range(micro):
                recv, _ = self._exchange(recv_prev=True)
                _, out = self._forward_micro(recv, data_iter, losses, keep_logits=logits if return_logits else None)
                self._exchange(send_next=None if self.is_last_stage() else out)
        self._settle_sends()
        if was_training:
            self.module.train()
        self._forget_shapes()
        loss = self._aggregate_loss(losses)
        if return_logits:
            return loss, (torch.cat(logits, dim=0) if logits else None)
        return loss

    def _aggregate_loss(self, losses):
        """Mean micro-batch loss of the last stage, broadcast along the pipe, averaged over data parallel."""
        dev = self._device()
        val = torch.stack(losses).mean().float() if losses else torch.zeros((), device=dev)
        val = val.reshape(1).to(dev)
        if self.num_stages > 1:
            dist.broadcast(val, mpu.get_pipe_parallel_ranks()[-1], group=mpu.get_pipe_parallel_group())
        if mpu.get_data_parallel_world_size() > 1:
            dist.all_reduce(val, group=mpu.get_data_parallel_group())
            val /= mpu.get_data_parallel_world_size()
        return val[0]

    def _sync_tied_grads(self):
        """Sum the gradients of weights shared by the first and last stage (tied embeddings)."""
        if not self._tied or self._tied_group is None:
            return
        group = self._tied_group
        for mod in self._tied:
            for p in mod.parameters():
                g = getattr(p, "main_grad", None)
                if p.grad is not None and g is not None:
                    g.add_(p.grad.to(g.dtype))
                    p.grad = None
                if g is not None:
                    dist.all_reduce(g, group=group)

    # surface the reference reads off its engine
    def set_batch_fn(self, fn):
        self.batch_fn = fn

    def wall_clock_breakdown(self):
        return False

    def steps_per_print(self):
        return self.neox_args.steps_per_print

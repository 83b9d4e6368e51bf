"""Tensor-parallel Mamba-1 block (megatron/model/mamba/mamba.py:26-413).

Structure as in the reference: column-parallel ``in_proj`` to ``2 * d_inner`` (x | z), depthwise causal
conv (width 4) + SiLU on x, ``x_proj`` (row-parallel weights, *no* cross-rank reduction: every tensor-
parallel rank derives dt / B / C from its own channels, mamba.py:112-121), ``dt_proj``, the S6 selective
scan gated by ``silu(z)``, row-parallel ``out_proj``.

Activations stay in ``[seq, batch, channel]`` memory order from end to end: the conv and scan kernels
(csrc/mamba.cu) address ``[batch, time, channel]`` views by strides, so the reference's two
``rearrange`` copies per block disappear, and the block works in eval mode as well as in training.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import parallel as mpu
from ..ops.gemm import linear
from ..ops.mamba import causal_conv1d_silu, selective_scan
from ..parallel.layers import _set_tp_attrs
from .norms import get_norm


class ParallelMambaBlock(nn.Module):
    def __init__(self, neox_args, init_method, output_layer_init_method):
        super().__init__()
        self.neox_args = neox_args
        assert not (neox_args.mamba_use_bias_in_linears and neox_args.mamba_inner_func_fusion), \
            "Mamba fused inner fn and bias in x_proj not compatible!"
        assert neox_args.intermediate_size is None or neox_args.expansion_factor is None, \
            "Must pass either the absolute intermediate size or the relative expansion factor for the mamba projections"
        self.d_model = neox_args.hidden_size
        self.d_state, self.d_conv = 16, 4
        if neox_args.intermediate_size:
            self.d_inner = neox_args.intermediate_size
        else:
            self.d_inner = int((neox_args.expansion_factor or 2) * self.d_model)
        self.dt_rank = math.ceil(self.d_model / 16)
        dt_min, dt_max, dt_init_floor = 0.001, 0.1, 1e-4
        ws = mpu.get_model_parallel_world_size()
        self.d_inner_per_rank = mpu.divide(self.d_inner, ws)
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and \
            not neox_args.use_cpu_initialization else torch.device("cpu")
        dt_ = neox_args.params_dtype
        use_bias = bool(neox_args.mamba_use_bias_in_linears)
        self.in_proj = mpu.ColumnParallelLinear(neox_args=neox_args, input_size=self.d_model,
                                                output_size=self.d_inner * 2, gather_output=False,
                                                init_method=init_method, skip_bias_add=not use_bias, bias=use_bias)
        dp = self.d_inner_per_rank
        # depthwise conv weights in the nn.Conv1d layout [d, 1, w] (checkpoint compatibility)
        self.conv1d = nn.Conv1d(dp, dp, kernel_size=self.d_conv, groups=dp, padding=self.d_conv - 1,
                                bias=bool(neox_args.mamba_use_bias_in_conv), device=dev, dtype=dt_)
        self.x_proj = mpu.RowParallelLinear(neox_args=neox_args, input_size=self.d_inner,
                                            output_size=self.dt_rank + self.d_state * 2, input_is_parallel=True,
                                            init_method=init_method, skip_bias_add=not use_bias,
                                            parallel_output=True, bias=use_bias)
        self.dt_proj = nn.Linear(self.dt_rank, dp, bias=True, device=dev, dtype=dt_)
        std = self.dt_rank ** -0.5
        nn.init.uniform_(self.dt_proj.weight, -std, std)
        dt = torch.exp(torch.rand(dp, device=dev, dtype=torch.float32) * (math.log(dt_max) - math.log(dt_min))
                       + math.log(dt_min)).clamp(min=dt_init_floor)
        with torch.no_grad():
            self.dt_proj.bias.copy_(dt + torch.log(-torch.expm1(-dt)))     # inverse softplus
        A = torch.arange(1, self.d_state + 1, dtype=torch.float32, device=dev).repeat(dp, 1).contiguous()
        self.A_log = nn.Parameter(torch.log(A))
        self.D = nn.Parameter(torch.ones(dp, device=dev, dtype=torch.float32))
        for p in (self.A_log, self.D):
            p._no_weight_decay = True
            if neox_args.mamba_selective_fp32_params:
                p._deepspeed_no_cast = True
        # per-rank channel shards: flagged tensor-parallel so norms / checkpoints treat them as such
        for p in list(self.conv1d.parameters()) + list(self.dt_proj.parameters()) + [self.A_log, self.D]:
            _set_tp_attrs(p, True, 0, 1)
        self.out_proj = mpu.RowParallelLinear(neox_args=neox_args, input_size=self.d_inner, output_size=self.d_model,
                                              input_is_parallel=True, init_method=output_layer_init_method,
                                              skip_bias_add=not use_bias, bias=use_bias, parallel_output=False)

    def selective_scan(self, x, dt, A, B, C, D, z=None, delta_bias=None, delta_softplus=True):
        assert delta_softplus
        return selective_scan(x, dt, A, B, C, D=D, z=z, dt_bias=delta_bias)

    def forward(self, hidden_states):
        """[sq, b, h] -> [sq, b, h] (sequence shards under sequence parallelism)."""
        xz, bias = self.in_proj(hidden_states)
        if bias is not None:
            xz = xz + bias
        l, b, _ = xz.shape
        dp, R, N = self.d_inner_per_rank, self.dt_rank, self.d_state
        x = xz[..., :dp].transpose(0, 1)                    # [b, l, d] views, no copies
        z = xz[..., dp:].transpose(0, 1)
        x = causal_conv1d_silu(x, self.conv1d.weight.view(dp, self.d_conv), self.conv1d.bias)
        x_lm = x.transpose(0, 1)                            # [l, b, d]
        if not x_lm.is_contiguous():
            x_lm = x_lm.contiguous()
            x = x_lm.transpose(0, 1)
        rows = x_lm.reshape(l * b, dp)
        width = R + 2 * N
        pad = (-width) % 8 if rows.is_cuda else 0
        w_x = self.x_proj.weight
        if pad:
            w_x = F.pad(w_x, (0, 0, 0, pad))
        x_dbl = linear(rows, w_x, None)                     # [(l b), R + 2N (+pad)], not reduced over TP
        if self.x_proj.bias is not None:
            x_dbl = x_dbl + F.pad(self.x_proj.bias, (0, pad))
        if rows.is_cuda:
            # dt_proj over the whole row with a zero-extended weight: no strided / odd-K operand
            w_dt = F.pad(self.dt_proj.weight, (0, x_dbl.shape[1] - R))
            dt = linear(x_dbl, w_dt, None)
        else:
            dt = x_dbl[:, :R] @ self.dt_proj.weight.t()
        x3 = x_dbl.view(l, b, -1).transpose(0, 1)
        Bm, Cm = x3[..., R:R + N], x3[..., R + N:R + 2 * N]
        dt = dt.view(l, b, dp).transpose(0, 1)
        A = -torch.exp(self.A_log.float())
        y = self.selective_scan(x, dt, A, Bm, Cm, self.D.float(), z=z, delta_bias=self.dt_proj.bias.float())
        y = y.transpose(0, 1)                               # [l, b, d]
        if not y.is_contiguous():
            y = y.contiguous()
        out, bias = self.out_proj(y)
        if bias is not None:
            out = out + bias
        return out


class ParallelMambaResidualLayer(nn.Module):
    """Pre-norm residual wrapper: ``x + mixer(norm(x))``."""

    def __init__(self, neox_args, init_method, output_layer_init_method, layer_number):
        super().__init__()
        self.layer_number = layer_number
        norm, eps = get_norm(neox_args)
        self.norm = norm(neox_args.hidden_size, eps=eps)
        self.mixer = ParallelMambaBlock(neox_args=neox_args, init_method=init_method,
                                        output_layer_init_method=output_layer_init_method)

    def forward(self, x, attention_mask=None, layer_past=None):
        return self.mixer(self.norm(x)) + x


class ParallelMambaResidualLayerPipe(ParallelMambaResidualLayer):
    """Pipeline form: threads the attention mask through."""

    def forward(self, args):
        assert len(args) == 2, "MambaResidualLayerPipe expects 2 arguments - hidden_states and attention_mask"
        hidden_states, attention_mask = args
        return super().forward(hidden_states, attention_mask), attention_mask

"""The fused bf16 CUDA model against the fp32 PyTorch statement of the same model (same weights)."""
import pytest
import torch

from common import tiny_config

pytestmark = pytest.mark.gpu


def _build(cfg):
    from gpt_neox_b200 import parallel as mpu
    from gpt_neox_b200 import training
    from gpt_neox_b200.config import NeoXArgs
    from gpt_neox_b200.initialize import initialize_megatron
    a = NeoXArgs.from_dict(cfg)
    a.configure_distributed_args()
    a.build_tokenizer()
    mpu.destroy_model_parallel()
    initialize_megatron(a)
    return a, training.get_model(a)


@pytest.mark.parametrize("variant", [
    dict(), dict(gpt_j_residual=False), dict(norm="rmsnorm", activation="swiglu", use_bias_in_mlp=False,
                                             use_bias_in_attn_linear=False, mlp_multiple_of=64),
    dict(num_kv_heads=2), dict(pos_emb="alibi"), dict(sliding_window_width=64), dict(bias_gelu_fusion=True)])
@pytest.mark.parametrize("precision", ["bfloat16", "fp16"])
def test_fused_model_matches_fp32_oracle(variant, precision):
    from gpt_neox_b200.models.gpt2_model import cross_entropy
    base = dict(num_layers=2, hidden_size=256, num_attention_heads=4, seq_length=256, max_position_embeddings=256,
                synthetic_vocab_size=1000, attention_config=[[["flash"], 2]], distributed_backend="nccl")
    base.update(variant)
    a_gpu, m_gpu = _build(tiny_config(precision=precision, **base))
    assert next(m_gpu.parameters()).dtype == (torch.float16 if precision == "fp16" else torch.bfloat16)
    sd = {k: v.detach().float().cpu() for k, v in m_gpu.state_dict().items()}
    a_cpu, m_cpu = _build(tiny_config(precision="fp32", use_cpu_initialization=True, **base))
    m_cpu = m_cpu.cpu().float()
    m_cpu.load_state_dict(sd, strict=False)
    torch.manual_seed(0)
    tokens = torch.randint(0, 1000, (2, 257))
    x, y = tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()
    pos = torch.arange(256)[None].expand(2, -1)
    mask = torch.ones(2, 256)
    out_g = m_gpu((x.cuda(), pos.cuda(), None))
    loss_g = cross_entropy(out_g, (y.cuda(), mask.cuda()))
    scale = 1024.0 if precision == "fp16" else 1.0            # fp16 gradients need a loss scale, as in training
    (loss_g * scale).backward()
    out_c = m_cpu((x, pos, None))
    loss_c = cross_entropy(out_c, (y, mask))
    loss_c.backward()
    assert abs(loss_g.item() - loss_c.item()) < 3e-2, (loss_g.item(), loss_c.item())
    gg = {n: p.grad for n, p in m_gpu.named_parameters() if p.grad is not None}
    worst = 0.0
    for n, p in m_cpu.named_parameters():
        if n in gg and p.grad is not None and p.grad.abs().max() > 1e-6:
            r = ((gg[n].float().cpu() / scale - p.grad).norm() / (p.grad.norm() + 1e-8)).item()
            worst = max(worst, r)
    assert worst < 8e-2, f"worst relative gradient error {worst}"


@pytest.mark.parametrize("family,variant", [
    ("mamba", dict(attention_config=[[["mamba"], 2]], pos_emb="none", gpt_j_residual=False, norm="rmsnorm")),
    ("rwkv", dict(attention_config=[[["rwkv"], 2]], pos_emb="none", gpt_j_residual=False)),
    ("gmlp", dict(attention_config=[[["gmlp"], 2]], pos_emb="none", gpt_j_residual=False)),
    ("dmoe", dict(moe_num_experts=4, moe_top_k=2, moe_expert_interval=1, gpt_j_residual=False)),
])
@pytest.mark.parametrize("precision", ["bfloat16", "fp16"])
def test_other_model_families_match_fp32_oracle_loss(family, variant, precision):
    """Mamba / RWKV-6 / gMLP / dMoE stacks: the 16-bit CUDA-kernel model and the fp32 PyTorch statement of the
    same model (same weights) agree on the loss and on the gradient of every parameter."""
    from gpt_neox_b200.models.gpt2_model import cross_entropy
    base = dict(num_layers=2, hidden_size=256, num_attention_heads=4, seq_length=256, max_position_embeddings=256,
                synthetic_vocab_size=1000, attention_config=[[["flash"], 2]], distributed_backend="nccl")
    base.update(variant)
    a_gpu, m_gpu = _build(tiny_config(precision=precision, **base))
    sd = {k: v.detach().float().cpu() for k, v in m_gpu.state_dict().items()}
    a_cpu, m_cpu = _build(tiny_config(precision="fp32", use_cpu_initialization=True, **base))
    m_cpu = m_cpu.cpu().float()
    m_cpu.load_state_dict(sd, strict=False)
    torch.manual_seed(0)
    tokens = torch.randint(0, 1000, (2, 257))
    x, y = tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()
    pos = torch.arange(256)[None].expand(2, -1)
    mask = torch.ones(2, 256)
    from gpt_neox_b200.utils.common import get_attn_mask
    am = get_attn_mask(256, "cpu", None) if family == "gmlp" else None
    out_g = m_gpu((x.cuda(), pos.cuda(), am.cuda() if am is not None else None))
    loss_g = cross_entropy(out_g, (y.cuda(), mask.cuda()))
    scale = 1024.0 if precision == "fp16" else 1.0            # fp16 gradients need a loss scale, as in training
    (loss_g * scale).backward()
    loss_c = cross_entropy(m_cpu((x, pos, am)), (y, mask))
    loss_c.backward()
    assert abs(loss_g.item() - loss_c.item()) < 5e-2 * max(1.0, abs(loss_c.item())) * 0.5, (loss_g.item(), loss_c.item())
    gg = {n: p.grad for n, p in m_gpu.named_parameters() if p.grad is not None}
    assert len(gg) > 4
    worst, where, compared = 0.0, None, 0
    # gradients that are zero up to cancellation (the bias in front of gMLP's gate: 1e-3 of the others) are rounding
    # noise in any 16-bit run, the PyTorch one included: compare what is at least 1 % of the largest gradient
    floor = 1e-2 * max(p.grad.norm().item() for n, p in m_cpu.named_parameters() if n in gg and p.grad is not None)
    for n, p in m_cpu.named_parameters():
        if n in gg:
            assert torch.isfinite(gg[n]).all(), n
            if p.grad is not None and p.grad.norm() > floor:
                r = ((gg[n].float().cpu() / scale - p.grad).norm() / (p.grad.norm() + 1e-8)).item()
                compared += 1
                if r > worst:
                    worst, where = r, n
    assert compared > 4
    # the router of a top-k MoE is discontinuous (a 16-bit rounding can move a token to another expert), so its
    # stack gets a wider band than the smooth mixers
    assert worst < (0.25 if family == "dmoe" else 0.12), f"worst relative gradient error {worst} at {where}"

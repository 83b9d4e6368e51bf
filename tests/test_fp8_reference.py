"""The PyTorch statements of the block-scaled fp8 format (CPU): what the CUDA quantiser and GEMM are tested against."""
import pytest
import torch

from gpt_neox_b200.ops import fp8


@pytest.mark.parametrize("rows,cols,e5m2", [(5, 32, False), (130, 160, False), (64, 416, True)])
def test_mxfp8_reference_round_trip_and_scale_layout(rows, cols, e5m2):
    torch.manual_seed(0)
    x = (torch.randn(rows, cols) * (torch.rand(rows, 1) * 40)).bfloat16()
    x[0, :32] = 0
    q, sf = fp8.mxfp8_quantize_reference(x, e5m2=e5m2)
    assert q.shape == (rows, cols) and q.dtype == torch.uint8
    assert sf.shape == ((cols + 127) // 128, (rows + 127) // 128 * 128) and sf.dtype == torch.int32
    # padding rows and the groups past the last column keep scale 1 (byte 0x7f)
    assert (sf[:, rows:] == 0x7F7F7F7F).all()
    groups = cols // 32
    if groups % 4:
        last = sf[-1, :rows].to(torch.int64) & 0xFFFFFFFF
        for b in range(groups % 4, 4):
            assert (((last >> (8 * b)) & 0xFF) == 0x7F).all()
    # an all-zero group: scale 1; every group: the smallest power of two that brings it into range
    assert (sf[0, 0].item() & 0xFF) == 0x7F
    fmax = fp8.E5M2_MAX if e5m2 else fp8.E4M3_MAX
    w = sf[:, :rows].to(torch.int64) & 0xFFFFFFFF
    by = torch.stack([(w >> (8 * i)) & 0xFF for i in range(4)], dim=-1).permute(1, 0, 2).reshape(rows, -1)[:, :groups]
    scale = torch.exp2((by - 127).float())
    amax = x.float().reshape(rows, groups, 32).abs().amax(-1)
    assert (amax <= scale * fmax).all()
    nz = amax > 0
    assert (amax[nz] > scale[nz] * fmax / 2).all()
    back = fp8.mxfp8_dequantize_reference(q, sf, e5m2=e5m2)
    step = 2.0 ** -3 if e5m2 else 2.0 ** -4        # half a unit in the last place at the top of a binade, relative to amax
    assert ((back - x.float()).abs() <= step * amax.unsqueeze(-1).expand(rows, groups, 32).reshape(rows, cols) + 1e-30).all()


def test_mxfp8_linear_refuses_cpu_tensors():
    from gpt_neox_b200.ops import _lib
    with pytest.raises(_lib.KernelError):
        fp8.mxfp8_linear(torch.randn(32, 64).bfloat16(), torch.randn(32, 64).bfloat16())

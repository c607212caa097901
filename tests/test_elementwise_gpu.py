"""The fused element-wise steps of a DiT block (csrc/elementwise.cu) against their torch fp32 definitions
(reference: nunchaku/models/normalization.py:60-159, transformer_flux_v2.py:174-343)."""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DTYPES = [torch.bfloat16, torch.float16]


@pytest.fixture(scope="module")
def cuda_dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,T,D,n", [(1, 300, 3072, 6), (2, 77, 1024, 3), (3, 5, 4096, 1)])
def test_layernorm_modulate(cuda_dev, dtype, B, T, D, n):
    from nunchaku_rocm_b200.ops.elementwise import layernorm_modulate

    g = torch.Generator().manual_seed(B + T + D)
    x = (torch.randn(B, T, D, generator=g) * 2 + 0.5).to(dtype)
    e = (torch.randn(B, D * n, generator=g) * 0.3).to(dtype)  # the modulation linear's interleaved [dim, n] output
    parts = e.view(B, D, n).permute(2, 0, 1)
    shift, scale = parts[0], parts[n - 1]
    want = (F.layer_norm(x, (D,), eps=1e-6) * (scale + 1.0)[:, None] + shift[:, None]).float()  # the reference's sequence
    ed = e.to(cuda_dev)
    pd = ed.view(B, D, n).permute(2, 0, 1)
    got = layernorm_modulate(x.to(cuda_dev), pd[n - 1], pd[0], scale_add=1.0)
    assert got.shape == (B, T, D) and got.dtype == dtype
    eps = 2.0**-7 if dtype == torch.bfloat16 else 2.0**-10
    diff = (got.float().cpu() - want).abs()
    # at most a rounding step of an intermediate (|LayerNorm * scale| stays below 8 here) where an fp32 sum fell on the other side
    assert (diff <= eps * (want.abs() + 8.0)).all()
    assert (diff > 0).float().mean() < 0.02
    # rows taken out of a wider buffer (row stride > dim)
    wide = torch.zeros(B, T, D + 64, dtype=dtype, device=cuda_dev)
    wide[..., :D] = x.to(cuda_dev)
    if B == 1:
        assert torch.equal(layernorm_modulate(wide[..., :D], pd[n - 1], pd[0], scale_add=1.0), got)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,T,D,with_y2", [(1, 300, 3072, False), (2, 77, 1024, True), (1, 33, 3080, True)])
def test_gated_residual(cuda_dev, dtype, B, T, D, with_y2):
    from nunchaku_rocm_b200.ops.elementwise import gated_residual

    g = torch.Generator().manual_seed(B + T + D)
    x = torch.randn(B, T, D, generator=g).to(dtype)
    y = torch.randn(B, T, D, generator=g).to(dtype)
    y2 = torch.randn(B, T, D, generator=g).to(dtype) if with_y2 else None
    e = (torch.randn(B, D * 3, generator=g) * 0.3).to(dtype)
    gate = e.view(B, D, 3).permute(2, 0, 1)[2]
    want = (x + gate[:, None] * ((y + y2) if with_y2 else y)).float()  # the reference's sequence, rounded at every step
    gd = e.to(cuda_dev).view(B, D, 3).permute(2, 0, 1)[2]
    got = gated_residual(x.to(cuda_dev), gd, y.to(cuda_dev), y2.to(cuda_dev) if with_y2 else None)
    assert torch.equal(got.float().cpu(), want)

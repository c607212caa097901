"""
Runtime LoRA on one layer (reference: nunchaku/lora/runtime.py:475-535, exercised there by
tests/test_lora_runtime.py): the extra factors are appended to the layer's 16-bit low-rank branch, so the
CPU tests check the bookkeeping and the GPU test checks the forward against the oracle with the concatenated branch.
"""

import pytest
import torch
from torch import nn

from nunchaku_rocm_b200.lora import attach_lora, attached_rank, detach_lora
from nunchaku_rocm_b200.models.linear import SVDQW4A4Linear


def _layer(cin=256, cout=128, rank=32, device="cpu", seed=0):
    g = torch.Generator().manual_seed(seed)
    lin = SVDQW4A4Linear(cin, cout, rank=rank, bias=True, torch_dtype=torch.bfloat16, device=device)
    with torch.no_grad():
        lin.qweight.copy_(torch.randint(-128, 128, lin.qweight.shape, dtype=torch.int8, generator=g))
        lin.wscales.copy_((torch.rand(lin.wscales.shape, generator=g) * 0.02 + 0.005).to(torch.bfloat16))
        lin.bias.copy_((torch.randn(cout, generator=g) * 0.1).to(torch.bfloat16))
        lin.smooth_factor.copy_((torch.rand(cin, generator=g) + 0.5).to(torch.bfloat16))
        lin.proj_down.copy_((torch.randn(cin, rank, generator=g) * 0.05).to(torch.bfloat16))
        lin.proj_up.copy_((torch.randn(cout, rank, generator=g) * 0.05).to(torch.bfloat16))
    return lin, g


def test_attach_appends_ranks_padded_to_16_and_detach_restores():
    lin, g = _layer()
    down0, up0 = lin.proj_down.data.clone(), lin.proj_up.data.clone()
    pairs = [(torch.randn(4, 256, generator=g), torch.randn(128, 4, generator=g)),
             (torch.randn(9, 256, generator=g), torch.randn(128, 9, generator=g))]
    attach_lora(lin, pairs)
    assert lin.proj_down.shape == (256, 48) and lin.proj_up.shape == (128, 48) and lin.rank == 48  # 32 + 13 -> 48
    assert attached_rank(lin) == 16
    assert torch.equal(lin.proj_down[:, :32], down0) and torch.equal(lin.proj_up[:, :32], up0)
    assert torch.equal(lin.proj_down[:, 32:36], pairs[0][0].t().to(torch.bfloat16))
    assert torch.equal(lin.proj_up[:, 36:45], pairs[1][1].to(torch.bfloat16))
    assert not lin.proj_down[:, 45:].any() and not lin.proj_up[:, 45:].any()
    # a second attachment replaces the first
    attach_lora(lin, pairs[:1])
    assert lin.proj_down.shape == (256, 48) and attached_rank(lin) == 16 and not lin.proj_down[:, 36:].any()
    detach_lora(lin)
    assert lin.rank == 32 and torch.equal(lin.proj_down.data, down0) and torch.equal(lin.proj_up.data, up0)
    assert attached_rank(lin) == 0
    detach_lora(lin)  # no-op


def test_attach_rejects_misshapen_factors():
    lin, g = _layer()
    with pytest.raises(ValueError):
        attach_lora(lin, [(torch.zeros(4, 255), torch.zeros(128, 4))])
    with pytest.raises(ValueError):
        attach_lora(lin, [(torch.zeros(4, 256), torch.zeros(128, 5))])
    assert attached_rank(lin) == 0 and lin.rank == 32


def test_hook_path_on_a_plain_linear():
    torch.manual_seed(0)
    lin = nn.Linear(32, 16)
    x = torch.randn(5, 32)
    base = lin(x)
    down, up = torch.randn(3, 32), torch.randn(16, 3)
    attach_lora(lin, [(down, up)])
    assert attached_rank(lin) == 3
    torch.testing.assert_close(lin(x), base + (x @ down.t()) @ up.t())
    detach_lora(lin)
    torch.testing.assert_close(lin(x), base)


@pytest.mark.gpu
@pytest.mark.parametrize("extra", [[8], [16, 64], [3, 5, 200]])
def test_forward_with_attached_lora_matches_oracle(extra):
    from oracle import w4a4

    dev = torch.device("cuda", 0)
    lin, g = _layer(cin=512, cout=384, rank=32)
    lin = lin.to(dev)
    pairs = [(torch.randn(r, 512, generator=g) * 0.05, torch.randn(384, r, generator=g) * 0.05) for r in extra]
    x = torch.randn(1, 200, 512, generator=g).to(torch.bfloat16).to(dev)
    base = lin(x).float().cpu()
    attach_lora(lin, pairs)
    assert lin.rank % 16 == 0 and lin.rank >= 32 + sum(extra)
    y = lin(x).float().cpu()

    # the oracle evaluates the layer with the concatenated low-rank branch
    q, s, la, _ = w4a4.quantize_act(x[0].cpu(), lin.proj_down.data.cpu(), lin.smooth_factor.data.cpu())
    ref = w4a4.gemm_w4a4(q, lin.qweight.data.cpu().view(torch.uint8), s, lin.wscales.data.cpu(), lin.bias.data.cpu(), la,
                         lin.proj_up.data.cpu())
    err = w4a4.rel_fro(y[0], ref.float())
    assert err <= 1e-2, err
    assert (y - base).abs().max() > 0  # the LoRA did something
    detach_lora(lin)
    assert torch.equal(lin(x).float().cpu(), base)

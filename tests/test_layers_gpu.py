"""
Layer-level parity: the parameter containers and the fused operators (the calls the reference's model classes make)
against the same chain evaluated by the CPU oracle.  The chains re-quantise intermediate activations, where a value on a
rounding boundary may land on the neighbouring code in one implementation and not in the other; the final 16-bit outputs are
therefore held to a relative Frobenius error of 2e-2 (twice the single-GEMM bar), as the reference's own fused-MLP tests
bound the extra error of the fused re-quantisation (tests/triton/test_w4a4.py:319-380).
"""

import pytest
import torch
import torch.nn as nn

from oracle import w4a4

pytestmark = pytest.mark.gpu
T = torch.bfloat16


def _layer(cin, cout, rank, dev, seed, precision="int4", unsigned=False):
    from nunchaku_rocm_b200.models.linear import SVDQW4A4Linear

    g = torch.Generator().manual_seed(seed)
    lin = SVDQW4A4Linear(cin, cout, rank=rank, bias=True, precision=precision, act_unsigned=unsigned, torch_dtype=T, device=dev)
    G = 16 if precision == "nvfp4" else 64
    p = dict(
        qweight=torch.randint(-128, 128, (cout, cin // 2), dtype=torch.int8, generator=g),
        bias=(torch.randn(cout, generator=g) * 0.1).to(T),
        smooth_factor=(torch.rand(cin, generator=g) + 0.5).to(T),
        proj_down=(torch.randn(cin, rank, generator=g) * 0.05).to(T),
        proj_up=(torch.randn(cout, rank, generator=g) * 0.05).to(T),
    )
    ws = torch.rand(cin // G, cout, generator=g) * 0.015 + 0.005
    p["wscales"] = ws.to(torch.float8_e4m3fn) if precision == "nvfp4" else ws.to(T)
    with torch.no_grad():
        for k, v in p.items():
            getattr(lin, k).copy_(v.to(dev))
    if precision == "nvfp4":
        lin.wtscale = 0.75
        wc = (torch.rand(cout, generator=g) * 0.5 + 0.5).to(T)
        with torch.no_grad():
            lin.wcscales.copy_(wc.to(dev))
        p["wcscales"], p["alpha"] = wc, 0.75
    return lin, p


def _oracle_linear(x2d, p, fp4=False, act_unsigned=False):
    q, s, l, _ = w4a4.quantize_act(x2d, p["proj_down"], p["smooth_factor"], fp4=fp4)
    return w4a4.gemm_w4a4(q, p["qweight"].view(torch.uint8), s, p["wscales"], p["bias"], l, p["proj_up"], fp4=fp4,
                          act_unsigned=act_unsigned, alpha=p.get("alpha", 1.0), wcscales=p.get("wcscales"))


def _check(out, ref, tol, what):
    err = w4a4.rel_fro(out.float().cpu(), ref.float())
    assert err <= tol, f"{what}: relative Frobenius error {err:.3g} > {tol}"


@pytest.mark.parametrize("precision", ["int4", "nvfp4"])
def test_svdq_linear_forward(cuda_dev, precision):
    B, S, cin, cout = 2, 100, 256, 384
    lin, p = _layer(cin, cout, 32, cuda_dev, 1, precision)
    x = torch.randn(B, S, cin, generator=torch.Generator().manual_seed(2)).to(T)
    y = lin(x.to(cuda_dev))
    assert y.shape == (B, S, cout) and y.dtype == T
    ref = _oracle_linear(x.view(-1, cin), p, fp4=precision == "nvfp4")
    _check(y.view(-1, cout), ref, 1e-2, f"SVDQW4A4Linear {precision}")


def test_fused_gelu_mlp(cuda_dev):
    from nunchaku_rocm_b200.ops.fused import fused_gelu_mlp

    B, S, c, h = 2, 72, 256, 512
    fc1, p1 = _layer(c, h, 16, cuda_dev, 3)
    fc2, p2 = _layer(h, c, 16, cuda_dev, 4, unsigned=True)
    x = torch.randn(B, S, c, generator=torch.Generator().manual_seed(5)).to(T)
    y = fused_gelu_mlp(x.to(cuda_dev), fc1, fc2)
    assert y.shape == (B, S, c)
    lin1 = _oracle_linear(x.view(-1, c), p1)
    codes, scale, lora = w4a4.gelu_quant(lin1, p2["smooth_factor"], p2["proj_down"], T)
    ref = w4a4.gemm_w4a4(w4a4.pack_nibbles(codes), p2["qweight"].view(torch.uint8), scale.to(T), p2["wscales"], p2["bias"], lora,
                         p2["proj_up"], act_unsigned=True)
    _check(y.view(-1, c), ref, 2e-2, "fused_gelu_mlp")


def test_fused_swiglu_mlp(cuda_dev):
    from nunchaku_rocm_b200.ops.fused import fused_swiglu_mlp, interleave_swiglu_linear_

    B, S, c, h = 1, 136, 256, 256  # fc1: c -> 2 h ([gate | up]), fc2: h -> c
    fc1, p1 = _layer(c, 2 * h, 16, cuda_dev, 6)
    fc2, p2 = _layer(h, c, 16, cuda_dev, 7)
    x = torch.randn(B, S, c, generator=torch.Generator().manual_seed(8)).to(T)
    lin1 = _oracle_linear(x.view(-1, c), p1)  # the oracle works on the un-interleaved layer
    codes, scale, lora = w4a4.swiglu_quant(lin1, p2["smooth_factor"], p2["proj_down"], T)
    ref = w4a4.gemm_w4a4(w4a4.pack_nibbles(codes), p2["qweight"].view(torch.uint8), scale.to(T), p2["wscales"], p2["bias"], lora,
                         p2["proj_up"])
    interleave_swiglu_linear_(fc1)
    y = fused_swiglu_mlp(x.to(cuda_dev), fc1, fc2)
    assert y.shape == (B, S, c)
    _check(y.view(-1, c), ref, 2e-2, "fused_swiglu_mlp")


def test_fused_qkv_norm_rotary(cuda_dev):
    from nunchaku_rocm_b200.ops.fused import fused_qkv_norm_rottary

    class RMS(nn.Module):
        def __init__(self, w):
            super().__init__()
            self.weight, self.eps = nn.Parameter(w, requires_grad=False), 1e-6

    B, S, c, heads = 2, 130, 256, 2
    proj, p = _layer(c, 3 * heads * 128, 32, cuda_dev, 9)
    g = torch.Generator().manual_seed(10)
    wq, wk = (1 + torch.randn(128, generator=g) * 0.05).to(T), (1 + torch.randn(128, generator=g) * 0.05).to(T)
    th = torch.rand(S, 64, generator=g) * 6.28
    rot = torch.stack([torch.sin(th), torch.cos(th)], -1).reshape(S, 64, 1, 2).float().contiguous()
    x = torch.randn(B, S, c, generator=g).to(T)
    y = fused_qkv_norm_rottary(x.to(cuda_dev), proj, RMS(wq.to(cuda_dev)), RMS(wk.to(cuda_dev)), rot.to(cuda_dev))
    assert y.shape == (B, S, 3 * heads * 128)
    lin = _oracle_linear(x.view(-1, c), p)
    ref = w4a4.qk_norm_rope(lin, wq, wk, rot.reshape(S, 128).repeat(B, 1))
    _check(y.view(-1, 3 * heads * 128), ref, 1e-2, "fused_qkv_norm_rottary")

"""
The CUDA kernels against outputs of the reference's own Triton kernels (fixtures written on a B200 by
tests/golden/make_golden_gpu.py): same seeded inputs, the reference's results on one side, this library's on the other.
Codes and scales of the quantizer are compared bit for bit where the arithmetic is exact, 16-bit outputs within two
rounding steps (the reference's own bar between its two implementations, tests/triton/test_native_gemm.py:130-142).
"""

import pytest
import torch

from oracle import w4a4
from tests.conftest import load_golden

pytestmark = pytest.mark.gpu
T = torch.bfloat16


def _two_steps(out, ref, what):
    out, ref = out.float().cpu(), ref.float()
    err = (out - ref).abs()
    tol = 2 * 2.0**-8 * torch.maximum(ref.abs(), out.abs()) + 1e-3
    assert (err <= tol).all(), f"{what}: {(err > tol).sum().item()} beyond two rounding steps, max {err.max().item():.3g}"


def test_quantizer_against_reference_kernel_outputs(cuda_dev):
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import quantize_w4a4_act_fuse_lora as quant

    g = load_golden("triton_quantize")
    d = lambda t: t.to(cuda_dev)
    q, s, l = quant(d(g["x"]), lora_down=d(g["lora_down"]), smooth=d(g["smooth"]))
    assert torch.equal(q.cpu(), g["q_signed"])
    assert torch.equal(s.cpu().view(torch.int16), g["s_signed"].view(torch.int16))
    torch.testing.assert_close(l.cpu(), g["l_signed"], rtol=2e-3, atol=2e-3)
    q, s, _ = quant(d(g["x"]), fp4=True)
    assert torch.equal(s.cpu().view(torch.uint8), g["s_fp4"].view(torch.uint8))
    c, ref = w4a4.unpack_nibbles(q.cpu()), w4a4.unpack_nibbles(g["q_fp4"])
    dd = ((c & 7) - (ref & 7)).abs()
    assert dd.max() <= 1 and (dd != 0).float().mean() < 1e-3  # threshold ties (fast division in the reference's build)
    q, s, l = quant(d(g["x"]), lora_down=d(g["lora_down"]), smooth=d(g["smooth"]), fuse_gelu=True, shift_value=0.171875,
                    unsigned=True)
    dd = (w4a4.unpack_nibbles(q.cpu()) - w4a4.unpack_nibbles(g["q_gelu_u"])).abs()
    assert dd.max() <= 1 and (dd != 0).float().mean() < 1e-3
    assert ((s.float().cpu() - g["s_gelu_u"].float()).abs() <= 2.0**-7 * g["s_gelu_u"].float().abs()).all()


@pytest.mark.parametrize("impl", [0, 2])
def test_nvfp4_gemm_against_reference_kernel_output(cuda_dev, impl):
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import gemm_w4a4

    g = load_golden("triton_gemm_fp4")
    d = lambda t: t.to(cuda_dev)
    out = gemm_w4a4(d(g["act"]), d(g["wgt"]), None, d(g["ascales"]), d(g["wscales"]), d(g["bias"]), d(g["lora_act"]),
                    d(g["lora_up"]), wcscales=d(g["wcscales"]), alpha=float(g["alpha"]), fp4=True, out_dtype=T, _impl=impl)
    _two_steps(out, g["out"], "NVFP4 GEMM")


@pytest.mark.parametrize("impl", [0, 2, 3, 4])
def test_int4_gemm_against_reference_kernel_outputs(cuda_dev, impl):
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import gemm_w4a4

    g = load_golden("triton_gemm_int4")
    d = lambda t: t.to(cuda_dev)
    args = (d(g["act"]), d(g["wgt"]), None, d(g["ascales"]), d(g["wscales"]), d(g["bias"]), d(g["lora_act"]), d(g["lora_up"]))
    _two_steps(gemm_w4a4(*args, _impl=impl), g["out_plain"], "int4 GEMM")
    out = gemm_w4a4(*args, norm_q=d(g["norm_q"]), norm_k=d(g["norm_k"]), rotary_emb=d(g["rot"]), _impl=impl)
    _two_steps(out, g["out_qk"], "fused Q/K epilogue")
    if impl == 4:
        return  # the single-CTA kernel has no fused re-quantisation
    M, N = g["act"].shape[0], g["wgt"].shape[0]
    for uns, tag in ((False, "s"), (True, "u")):
        qout = torch.zeros(M, N // 2, dtype=torch.uint8, device=cuda_dev)
        osc = torch.zeros(N // 64, M, dtype=T, device=cuda_dev)
        lao = torch.zeros(M, g["lora_down"].shape[1], dtype=torch.float32, device=cuda_dev)
        gemm_w4a4(*args, qout=qout, oscales=osc, smooth_factor=d(g["smooth"]), lora_down=d(g["lora_down"]),
                  lora_act_out=lao, act_unsigned=uns, _impl=impl)
        dd = (w4a4.unpack_nibbles(qout.cpu()) - w4a4.unpack_nibbles(g[f"gq_q_{tag}"])).abs()
        rate = (dd != 0).float().mean().item()
        # the fused kernels work on the fp32 tile like the reference's; the unfused path (no fused kernel for the shape)
        # rounds the tile to 16 bits first, as the reference's own fallback does
        assert dd.max() <= 1 and rate < 1e-2, rate
        sr = g[f"gq_s_{tag}"].float()
        assert ((osc.float().cpu() - sr).abs() <= 2.0**-7 * sr.abs()).all()
        assert (lao.cpu() - g[f"gq_l_{tag}"]).abs().max() <= 1e-2 * g[f"gq_l_{tag}"].abs().max()


def test_attention_and_awq_against_reference_kernel_outputs(cuda_dev):
    from nunchaku_rocm_b200.ops.gemv import awq_gemv_w4a16_cuda
    from nunchaku_rocm_b200.ops.triton.attention import attention_fp16

    g = load_golden("triton_attention")
    d = lambda t: t.to(cuda_dev)
    o = torch.empty_like(g["o"], device=cuda_dev)
    attention_fp16(d(g["q"]), d(g["k"]), d(g["v"]), o, 128**-0.5)
    torch.testing.assert_close(o.float().cpu(), g["o"].float(), rtol=2 * 2.0**-7, atol=2.0**-8)
    g = load_golden("triton_awq_gemv")
    n, k = g["scales"].shape[1], g["x"].shape[1]
    out = awq_gemv_w4a16_cuda(d(g["x"]), d(g["kernel"]), d(g["scales"]), d(g["zeros"]), g["x"].shape[0], n, k, 64)
    _two_steps(out, g["out"], "AWQ GEMV")

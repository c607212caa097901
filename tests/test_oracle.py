"""The CPU oracle against the fixtures written by the reference's own code (tests/golden/make_golden.py)."""

import torch

from oracle import awq_attn, w4a4
from tests.conftest import load_golden


def test_gemm_matches_reference_outputs():
    for tag in ("a", "b"):
        g = load_golden(f"gemm_{tag}")
        for uns, key in ((False, "out_s"), (True, "out_u")):
            out = w4a4.gemm_w4a4(
                g["act"], g["wgt"], g["ascales"], g["wscales"], g["bias"], g["lora_act"], g["lora_up"], act_unsigned=uns
            )
            # same fp32 operations in the same order: identical up to matmul blocking
            torch.testing.assert_close(out, g[key], rtol=1e-6, atol=1e-5)
        out = w4a4.gemm_w4a4(g["act"], g["wgt"], g["ascales"], g["wscales"])
        torch.testing.assert_close(out, g["out_nolora_s"], rtol=1e-6, atol=1e-5)


def test_group_dots_are_exact_integers():
    g = load_golden("gemm_b")
    p = w4a4.group_dots_int32(g["act"], g["wgt"], False)
    a = w4a4.int4_values(g["act"], True).long()
    w = w4a4.int4_values(g["wgt"], True).long()
    for gi in range(p.shape[0]):
        ref = a[:, 64 * gi : 64 * gi + 64] @ w[:, 64 * gi : 64 * gi + 64].T
        assert torch.equal(p[gi].long(), ref)
    # and the scaled sum of them is the GEMM core
    core = sum(
        p[gi].float() * g["ascales"][gi].float()[:, None] * g["wscales"][gi].float()[None, :] for gi in range(p.shape[0])
    )
    torch.testing.assert_close(core, g["out_nolora_s"], rtol=1e-6, atol=1e-5)


def test_qk_matches_reference():
    g = load_golden("qk")
    out = w4a4.qk_norm_rope(g["lin"], g["norm_q"], g["norm_k"], g["rot"])
    torch.testing.assert_close(out, g["out"], rtol=1e-6, atol=1e-6)


def _check_quant(codes, scales, lora, g):
    # the reference's torch form divides, the kernels multiply by reciprocals: codes may differ by one
    # at exact rounding boundaries (bars of nunchaku/ops/triton/native/w4a4.py:689-702)
    d = (codes - g["codes"]).abs()
    assert d.max() <= 1 and (d != 0).float().mean() < 1e-3
    torch.testing.assert_close(scales, g["scales"], rtol=1e-6, atol=0)
    torch.testing.assert_close(lora, g["lora"], rtol=1e-5, atol=1e-5)


def test_gelu_quant_matches_reference():
    g = load_golden("gelu_quant")
    _check_quant(*w4a4.gelu_quant(g["lin"], g["smooth"], g["lora_down"], torch.bfloat16), g)


def test_swiglu_quant_matches_reference():
    g = load_golden("swiglu_quant")
    _check_quant(*w4a4.swiglu_quant(g["lin"], g["smooth"], g["lora_down"], torch.bfloat16), g)
    assert torch.equal(w4a4.interleave_swiglu(256), g["interleave"])


def test_quantizer_signed_roundtrip_bound():
    # bound of the reference's own test (tests/triton/test_w4a4.py:187-204)
    torch.manual_seed(0)
    x = torch.randn(64, 512).to(torch.bfloat16)
    for fp4 in (False, True):
        packed, scales, _, codes = w4a4.quantize_act(x, fp4=fp4)
        G = 16 if fp4 else 64
        vals = w4a4.e2m1_decode(codes) if fp4 else torch.where(codes >= 8, codes - 16, codes).float()
        deq = vals * scales.float().t().repeat_interleave(G, dim=1)
        assert (deq - x.float()).abs().amax() <= scales.float().amax() * 1.01
        assert torch.equal(w4a4.unpack_nibbles(packed), codes)


def test_quantizer_equals_gelu_quant_tail():
    # the unsigned quantizer with fuse_gelu + shift is the GELU epilogue applied to a stored 16-bit tensor
    torch.manual_seed(1)
    lin = (torch.randn(32, 256) * 2).to(torch.bfloat16)
    smooth = (torch.rand(256) + 0.5).to(torch.bfloat16)
    ld = (torch.randn(256, 32) * 0.1).to(torch.bfloat16)
    packed, scales, lora, codes = w4a4.quantize_act(
        lin, ld, smooth, fuse_gelu=True, shift_value=w4a4.GELU_SHIFT, unsigned=True
    )
    c2, s2, l2 = w4a4.gelu_quant(lin.float(), smooth, ld, torch.bfloat16)
    assert torch.equal(codes, c2)
    assert torch.equal(scales, s2.to(torch.bfloat16))
    torch.testing.assert_close(lora, l2)


def test_e2m1_ties_go_up():
    x = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, 0.2499, 7.0, -9.0, -0.0])
    assert w4a4.e2m1_encode(x).tolist() == [1, 2, 3, 4, 5, 6, 7, 9, 0, 7, 15, 0]


def test_awq_pack_matches_reference():
    g = load_golden("awq_pack")
    packed = awq_attn.awq_pack(g["q"])
    assert torch.equal(packed.view(torch.int16), g["packed_i16"])
    assert torch.equal(awq_attn.awq_unpack(packed, 64, 128), g["q"])


def test_awq_gemv_is_dequant_matmul():
    torch.manual_seed(2)
    n, k = 64, 256
    q = torch.randint(0, 16, (n, k), dtype=torch.int32)
    s = (torch.rand(k // 64, n) * 0.1 + 0.01).to(torch.bfloat16)
    z = (torch.randn(k // 64, n) * 0.1).to(torch.bfloat16)
    x = torch.randn(3, k).to(torch.bfloat16)
    packed = awq_attn.awq_pack(q)
    ref = x.float() @ awq_attn.awq_dequant(packed, s, z, n, k).T
    torch.testing.assert_close(awq_attn.awq_gemv(x, packed, s, z, n, k), ref, rtol=1e-4, atol=1e-4)


def test_rope_matches_reference():
    g = load_golden("rope")
    torch.testing.assert_close(awq_attn.rope(g["pos"], 16), g["out16"], rtol=0, atol=1e-6)
    torch.testing.assert_close(awq_attn.rope(g["pos"], 56), g["out56"], rtol=0, atol=1e-6)
    t = awq_attn.flux_rotary_table(8, 4, 4)
    assert t.shape == (24, 64, 1, 2)
    assert torch.all(t[:8, :, 0, 0] == 0) and torch.all(t[:8, :, 0, 1] == 1)


def test_attention_roundings_are_small():
    torch.manual_seed(3)
    q, k, v = (torch.randn(1, 2, 100, 64).to(torch.bfloat16) for _ in range(3))
    torch.testing.assert_close(awq_attn.attention(q, k, v), awq_attn.attention_exact(q, k, v), rtol=3e-2, atol=3e-2)

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


def test_quantizer_equals_swiglu_tail():
    # The signed activation quantizer is the tail of the SwiGLU epilogue (nunchaku/ops/triton/native/w4a4.py:762-766)
    # applied to y = silu(gate) * up.  The fixture holds what the reference's own `reference_swiglu_quant` returned, so
    # this ties the signed path of `quantize_act` (codes, unrounded-scale arithmetic, LoRA-down before smoothing) to
    # a reference-run vector.
    g = load_golden("swiglu_quant")
    H = g["lin"].shape[1] // 2
    y = w4a4.silu(g["lin"][:, :H]) * g["lin"][:, H:].float()
    packed, scales, lora, codes = w4a4.quantize_act(y, g["lora_down"], g["smooth"])  # fp32 input: scales stay fp32
    signed = torch.where(codes >= 8, codes - 16, codes)
    _check_quant(signed, scales, lora, g)
    assert torch.equal(w4a4.unpack_nibbles(packed), codes)
    # and the two oracle functions agree with each other exactly
    c2, s2, l2 = w4a4.swiglu_quant(g["lin"], g["smooth"], g["lora_down"], torch.bfloat16)
    assert torch.equal(signed, c2) and torch.equal(scales, s2)
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


# ------------------------------------------------------------------------------------------------
# The oracle against outputs of the reference's own Triton kernels, run on a B200 through Triton's NVIDIA backend
# (tests/golden/make_golden_gpu.py).  These pin the pieces the reference has no pure-PyTorch form of.
# ------------------------------------------------------------------------------------------------
def _signed(c):
    return torch.where(c >= 8, c - 16, c)


def test_quantizer_matches_the_reference_kernel():
    g = load_golden("triton_quantize")
    x, ld, sm = g["x"], g["lora_down"], g["smooth"]
    # signed, smooth, LoRA-down: codes and 16-bit scales bit for bit
    p, s, l, _ = w4a4.quantize_act(x, ld, sm)
    assert torch.equal(p, g["q_signed"])
    assert torch.equal(s.view(torch.int16), g["s_signed"].view(torch.int16))
    torch.testing.assert_close(l, g["l_signed"], rtol=1e-4, atol=1e-4)
    # NVFP4: e4m3 scales bit for bit; e2m1 codes equal except where v / scale sits on an encoding threshold (+-0.25,
    # +-0.75, ...) to the last bit: Triton's NVIDIA backend divides and takes reciprocals with its fast instructions,
    # the oracle with IEEE ones (10 of 36864 codes here, each on the neighbouring code)
    p, s, _, c = w4a4.quantize_act(x, fp4=True)
    assert torch.equal(s.view(torch.uint8), g["s_fp4"].view(torch.uint8))
    ref = w4a4.unpack_nibbles(g["q_fp4"])
    d = ((c & 7) - (ref & 7)).abs()
    assert d.max() <= 1 and (d != 0).float().mean() < 1e-3
    near_zero = ((c & 7) + (ref & 7)) <= 1
    assert (((c & 8) == (ref & 8)) | near_zero).all()
    # GELU + shift + unsigned and GLU: the activation's exp differs in the last bits between libraries, so a code may
    # move by one at a rounding boundary
    for kw, tag, sgn in ((dict(smooth=sm, fuse_gelu=True, shift_value=w4a4.GELU_SHIFT, unsigned=True), "gelu_u", False),
                         (dict(fuse_glu=True), "glu", True)):
        xin = g["x_glu"] if tag == "glu" else x
        p, s, l, c = w4a4.quantize_act(xin, ld, **kw)
        ref = w4a4.unpack_nibbles(g[f"q_{tag}"])
        d = ((_signed(c) - _signed(ref)) if sgn else (c - ref)).abs()
        assert d.max() <= 1 and (d != 0).float().mean() < 1e-3
        assert ((s.float() - g[f"s_{tag}"].float()).abs() <= 2.0**-7 * g[f"s_{tag}"].float().abs()).all()
        torch.testing.assert_close(l, g[f"l_{tag}"], rtol=1e-3, atol=1e-3)


def _two_steps(out16, ref32, what):
    # a 16-bit output within two rounding steps of the fp32 oracle (the reference's own bar for its kernels,
    # tests/triton/test_native_gemm.py:130-142)
    err = (out16.float() - ref32).abs()
    tol = 2 * 2.0**-8 * torch.maximum(ref32.abs(), out16.float().abs()) + 1e-3
    assert (err <= tol).all(), f"{what}: {(err > tol).sum().item()} elements beyond two rounding steps, max {err.max().item():.3g}"
    assert w4a4.rel_fro(out16.float(), ref32) <= 1e-2


def test_nvfp4_gemm_matches_the_reference_kernel():
    g = load_golden("triton_gemm_fp4")
    ref = w4a4.gemm_w4a4(g["act"], g["wgt"], g["ascales"], g["wscales"], g["bias"], g["lora_act"], g["lora_up"], fp4=True,
                         alpha=float(g["alpha"]), wcscales=g["wcscales"])
    _two_steps(g["out"], ref, "NVFP4 GEMM")


def test_int4_gemm_and_fused_epilogues_match_the_reference_kernel():
    g = load_golden("triton_gemm_int4")
    lin = w4a4.gemm_w4a4(g["act"], g["wgt"], g["ascales"], g["wscales"], g["bias"], g["lora_act"], g["lora_up"])
    _two_steps(g["out_plain"], lin, "int4 GEMM")
    M = lin.shape[0]
    _two_steps(g["out_qk"], w4a4.qk_norm_rope(lin, g["norm_q"], g["norm_k"], g["rot"].reshape(M, 128)), "fused Q/K epilogue")
    for uns, tag in ((False, "s"), (True, "u")):
        lin = w4a4.gemm_w4a4(g["act"], g["wgt"], g["ascales"], g["wscales"], g["bias"], g["lora_act"], g["lora_up"],
                             act_unsigned=uns)
        c, s, l = w4a4.gelu_quant(lin, g["smooth"], g["lora_down"], torch.bfloat16)
        ref = w4a4.unpack_nibbles(g[f"gq_q_{tag}"])
        d = (c - ref).abs()
        assert d.max() <= 1 and (d != 0).float().mean() < 1e-3, (d != 0).float().mean()
        sr = g[f"gq_s_{tag}"].float()
        assert ((s.to(torch.bfloat16).float() - sr).abs() <= 2.0**-7 * sr.abs()).all()
        assert (l - g[f"gq_l_{tag}"]).abs().max() <= 1e-3 * l.abs().max()


def test_attention_and_awq_gemv_match_the_reference_kernels():
    g = load_golden("triton_attention")
    ref = awq_attn.attention(g["q"], g["k"], g["v"], 128**-0.5)
    torch.testing.assert_close(g["o"].float(), ref, rtol=2 * 2.0**-8, atol=2.0**-9)
    g = load_golden("triton_awq_gemv")
    n, k = g["scales"].shape[1], g["x"].shape[1]
    ref = awq_attn.awq_gemv(g["x"], g["kernel"], g["scales"], g["zeros"], n, k)
    _two_steps(g["out"], ref, "AWQ GEMV")

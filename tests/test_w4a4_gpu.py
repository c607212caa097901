"""
GPU parity tests of the W4A4 GEMM, its epilogues and the activation quantizer against the CPU oracle
and the golden fixtures, through the C ABI (``nunchaku_rocm_b200.ops``).  Bars follow the reference's
own tests: bit-exact int32 group sums (tests/triton/test_native_gemm.py:166-179), 1e-2 of the output
range / 1e-2 relative Frobenius error for 16-bit outputs (native/w4a4.py:549-558), codes at most one
apart in a small fraction of positions and scales within a rounding step for the fused quantisers
(tests/triton/test_native_epilogues.py:214-268), canary rows past ``actual_m``.
"""

import pytest
import torch

from oracle import awq_attn, w4a4
from tests.conftest import load_golden

pytestmark = pytest.mark.gpu

TC, GENERIC, PAIR, SINGLE = 1, 2, 3, 4  # nb_gemm_args.impl: any tcgen05 kernel, CUDA cores, CTA-pair kernel, single-CTA kernel
DTYPES = [torch.bfloat16, torch.float16]


def _ops():
    from nunchaku_rocm_b200.ops.triton import gemm_w4a4 as K

    return K


def _status_clean(dev):
    from nunchaku_rocm_b200 import _lib

    torch.cuda.synchronize(dev)
    code = _lib.device_status(dev)
    _lib.status_word(dev).zero_()  # one failure must not fail every later test
    assert code == 0, f"a kernel gave up on a bounded wait: code {code:#x}"


def _rand_problem(M, N, K, R, dtype, seed=0, act_unsigned=False):
    g = torch.Generator().manual_seed(seed)
    act = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    wgt = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    asc = (torch.rand(K // 64, M, generator=g) * 0.02 + 0.01).to(dtype)
    wsc = (torch.rand(K // 64, N, generator=g) * 0.02 + 0.01).to(dtype)
    bias = torch.randn(N, generator=g).to(dtype)
    la = torch.randn(M, R, generator=g) if R else None
    lu = (torch.randn(N, R, generator=g) * 0.1).to(dtype) if R else None
    return act, wgt, asc, wsc, bias, la, lu


def _cuda(dev, *ts):
    return [t.to(dev) if t is not None else None for t in ts]


def _close(out, ref, what=""):
    out, ref = out.float().cpu(), ref.float()
    err = (out - ref).abs().max().item()
    tol = 1e-2 * ref.abs().max().item()
    assert err <= tol, f"{what}: max error {err:.4g} > {tol:.4g}"
    assert w4a4.rel_fro(out, ref) <= 1e-2, f"{what}: rel-Frobenius {w4a4.rel_fro(out, ref):.3g}"


# ------------------------------------------------------------------------------------------------
# golden fixtures (outputs of the reference's own `reference()`), every kernel
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("impl", [GENERIC, SINGLE, PAIR])
@pytest.mark.parametrize("tag", ["a", "b"])
def test_gemm_matches_golden(cuda_dev, impl, tag):
    K = _ops()
    g = load_golden(f"gemm_{tag}")
    act, wgt, asc, wsc, bias, la, lu = _cuda(
        cuda_dev, g["act"], g["wgt"], g["ascales"], g["wscales"], g["bias"], g["lora_act"], g["lora_up"]
    )
    M, N = act.shape[0], wgt.shape[0]
    for uns, key in ((False, "out_s"), (True, "out_u")):
        actual_m = M - 6
        buf = torch.full((actual_m + 8, N), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
        K.gemm_w4a4(act, wgt, buf[:actual_m], asc, wsc, bias, la, lu, act_unsigned=uns, _impl=impl)
        _close(buf[:actual_m], g[key][:actual_m], f"golden {tag} unsigned={uns}")
        assert bool(buf[actual_m:].isnan().all()), "rows past actual_m were written"
    out = K.gemm_w4a4(act, wgt, None, asc, wsc, _impl=impl)
    _close(out, g["out_nolora_s"], "golden no-lora")
    _status_clean(cuda_dev)


# ------------------------------------------------------------------------------------------------
# the integer contract: exact int32 group sums
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("impl", [GENERIC, SINGLE, PAIR])
@pytest.mark.parametrize("act_unsigned", [False, True])
@pytest.mark.parametrize("M,N,K", [(256, 512, 512), (136, 264, 256), (8, 8, 128)])
def test_group_sums_bit_exact(cuda_dev, impl, act_unsigned, M, N, K):
    Kn = _ops()
    act, wgt, *_ = _rand_problem(M, N, K, 0, torch.bfloat16, seed=M + N)
    p = Kn.gemm_w4a4_group_sums(act.to(cuda_dev), wgt.to(cuda_dev), act_unsigned=act_unsigned, _impl=impl)
    ref = w4a4.group_dots_int32(act, wgt, act_unsigned)
    assert torch.equal(p.cpu(), ref)
    _status_clean(cuda_dev)


@pytest.mark.parametrize("impl", [GENERIC, SINGLE, PAIR])
@pytest.mark.parametrize("act_unsigned", [False, True])
def test_group_sums_extreme_codes_bit_exact(cuda_dev, impl, act_unsigned):
    # The largest sums the format allows (|p| up to 64 * 15 * 8 = 7680) and every code pair at least once: the
    # tensor-core path accumulates on a floating-point pipe and must still return the exact integers.
    Kn = _ops()
    M, N, K = 128, 128, 256
    lo_a, hi_a = (0, 15) if act_unsigned else (-8, 7)
    a = torch.empty(M, K, dtype=torch.int64)
    w = torch.empty(N, K, dtype=torch.int64)
    a[:32], w[:32] = hi_a, -8            # most negative sum
    a[32:64], w[32:64] = lo_a if not act_unsigned else hi_a, 7
    a[64:96] = (torch.arange(K)[None, :] + torch.arange(32)[:, None]) % 16 + lo_a   # every activation code
    w[64:96] = (torch.arange(K)[None, :] // 16 + torch.arange(32)[:, None]) % 16 - 8  # against every weight code
    g = torch.Generator().manual_seed(3)
    a[96:] = torch.where(torch.rand(32, K, generator=g) < 0.5, lo_a, hi_a)
    w[96:] = torch.where(torch.rand(32, K, generator=g) < 0.5, -8, 7)
    act, wgt = w4a4.pack_nibbles(a), w4a4.pack_nibbles(w)
    p = Kn.gemm_w4a4_group_sums(act.to(cuda_dev), wgt.to(cuda_dev), act_unsigned=act_unsigned, _impl=impl)
    ref = w4a4.group_dots_int32(act, wgt, act_unsigned)
    assert int(ref.abs().max()) == (7680 if act_unsigned else 4096)
    assert torch.equal(p.cpu(), ref)
    _status_clean(cuda_dev)


@pytest.mark.parametrize("impl", [GENERIC, SINGLE, PAIR])
def test_unit_scale_output_is_exact_integer_sum(cuda_dev, impl):
    # with unit scales the fp32 tile is sum_g p_g exactly (tests/triton/test_native_gemm.py:166-179)
    Kn = _ops()
    M, N, K = 128, 256, 256
    g = torch.Generator().manual_seed(5)
    # keep |sum| < 256 so the bf16 store is exact: small codes
    a_codes = torch.randint(-1, 2, (M, K), generator=g)
    w_codes = torch.randint(-1, 2, (N, K), generator=g)
    act, wgt = w4a4.pack_nibbles(a_codes), w4a4.pack_nibbles(w_codes)
    ones_a = torch.ones(K // 64, M, dtype=torch.bfloat16)
    ones_w = torch.ones(K // 64, N, dtype=torch.bfloat16)
    out = Kn.gemm_w4a4(*_cuda(cuda_dev, act, wgt), None, *_cuda(cuda_dev, ones_a, ones_w), _impl=impl)
    ref = (a_codes.float() @ w_codes.float().T)
    assert ref.abs().max() < 256
    assert torch.equal(out.float().cpu(), ref)


# ------------------------------------------------------------------------------------------------
# shapes, dtypes, tails, strides, determinism
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("impl", [GENERIC, SINGLE, PAIR])
@pytest.mark.parametrize(
    "M,N,K,R", [(256, 256, 512, 32), (128, 512, 1024, 16), (64, 128, 256, 0), (264, 72, 384, 48), (520, 776, 128, 288)]
)
def test_gemm_bias_lora_shapes(cuda_dev, dtype, impl, M, N, K, R):
    Kn = _ops()
    for uns in (False, True):
        act, wgt, asc, wsc, bias, la, lu = _rand_problem(M, N, K, R, dtype, seed=K + R, act_unsigned=uns)
        ref = w4a4.gemm_w4a4(act, wgt, asc, wsc, bias, la, lu, act_unsigned=uns)
        out = Kn.gemm_w4a4(*_cuda(cuda_dev, act, wgt), None, *_cuda(cuda_dev, asc, wsc, bias, la, lu),
                           act_unsigned=uns, out_dtype=dtype, _impl=impl)
        _close(out, ref, f"{M}x{N}x{K} R={R} unsigned={uns}")
    _status_clean(cuda_dev)


@pytest.mark.parametrize("impl", [GENERIC, SINGLE, PAIR])
def test_gemm_strided_views_and_determinism(cuda_dev, impl):
    Kn = _ops()
    M, N, K, R = 200, 320, 256, 32
    act, wgt, asc, wsc, bias, la, lu = _rand_problem(M, N, K, R, torch.bfloat16, seed=9)
    ref = w4a4.gemm_w4a4(act, wgt, asc, wsc, bias, la, lu)
    dev = cuda_dev
    # operands as views into wider buffers (tests/triton/test_native_gemm.py:234-248)
    act_w = torch.zeros(M, K // 2 + 32, dtype=torch.uint8, device=dev)
    act_w[:, : K // 2] = act.to(dev)
    wgt_w = torch.zeros(N, K // 2 + 16, dtype=torch.uint8, device=dev)
    wgt_w[:, : K // 2] = wgt.to(dev)
    asc_w = torch.zeros(K // 64, M + 56, dtype=torch.bfloat16, device=dev)
    asc_w[:, :M] = asc.to(dev)
    out_w = torch.zeros(M, N + 64, dtype=torch.bfloat16, device=dev)
    args = (act_w[:, : K // 2], wgt_w[:, : K // 2], out_w[:, :N], asc_w[:, :M], wsc.to(dev), bias.to(dev), la.to(dev), lu.to(dev))
    Kn.gemm_w4a4(*args, _impl=impl)
    _close(out_w[:, :N], ref, "strided")
    assert bool((out_w[:, N:] == 0).all())
    first = out_w[:, :N].clone()
    Kn.gemm_w4a4(*args, _impl=impl)
    assert torch.equal(first, out_w[:, :N]), "two runs differ"
    _status_clean(dev)


def test_tc_and_generic_agree_closely(cuda_dev):
    Kn = _ops()
    M, N, K, R = 384, 512, 768, 32
    act, wgt, asc, wsc, bias, la, lu = _cuda(cuda_dev, *_rand_problem(M, N, K, R, torch.bfloat16, seed=21))
    a = Kn.gemm_w4a4(act, wgt, None, asc, wsc, bias, la, lu, _impl=TC).float()
    b = Kn.gemm_w4a4(act, wgt, None, asc, wsc, bias, la, lu, _impl=GENERIC).float()
    # same exact integers, fp32 summation order differs: at most one 16-bit rounding step apart
    assert ((a - b).abs() <= 2.0**-7 * b.abs() + 1e-6).all()


# ------------------------------------------------------------------------------------------------
# fused Q/K RMSNorm + RoPE
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("impl", [GENERIC, SINGLE, PAIR])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("batch,S,heads", [(1, 130, 2), (2, 72, 1), (1, 256, 4)])
def test_qk_norm_rope(cuda_dev, impl, dtype, batch, S, heads):
    Kn = _ops()
    M_real = batch * S
    M = (M_real + 7) // 8 * 8
    N, K, R = 3 * heads * 128, 256, 16
    act, wgt, asc, wsc, bias, la, lu = _rand_problem(M, N, K, R, dtype, seed=S)
    g = torch.Generator().manual_seed(S + 1)
    nq = (torch.rand(128, generator=g) + 0.5).to(dtype)
    nk = (torch.rand(128, generator=g) + 0.5).to(dtype)
    theta = torch.rand(S, 64, generator=g) * 6.28
    rot = torch.stack([torch.sin(theta), torch.cos(theta)], -1).reshape(S, 64, 1, 2).float()
    lin = w4a4.gemm_w4a4(act, wgt, asc, wsc, bias, la, lu)[:M_real]
    ref = w4a4.qk_norm_rope(lin, nq, nk, rot.reshape(S, 128).repeat(batch, 1))
    buf = torch.full((M_real + 8, N), float("nan"), dtype=dtype, device=cuda_dev)
    Kn.gemm_w4a4(*_cuda(cuda_dev, act, wgt), buf[:M_real], *_cuda(cuda_dev, asc, wsc, bias, la, lu),
                 norm_q=nq.to(cuda_dev), norm_k=nk.to(cuda_dev), rotary_emb=rot.to(cuda_dev), _impl=impl)
    _close(buf[:M_real], ref, "qk")
    assert bool(buf[M_real:].isnan().all())
    _status_clean(cuda_dev)


def test_qk_matches_golden_unfused(cuda_dev):
    Kn = _ops()
    g = load_golden("qk")
    out = g["lin"].to(torch.bfloat16).to(cuda_dev)
    ref = w4a4.qk_norm_rope(out.float().cpu(), g["norm_q"], g["norm_k"], g["rot"])
    Kn._apply_rmsnorm_rope_qk(out, g["norm_q"].to(cuda_dev), g["norm_k"].to(cuda_dev), g["rot"].to(cuda_dev))
    _close(out, ref, "unfused qk")
    _close(out, g["out"], "unfused qk vs golden")  # golden used the unrounded lin: still within the bar


# ------------------------------------------------------------------------------------------------
# activation quantizer
# ------------------------------------------------------------------------------------------------
def _unpack_codes(packed, signed):
    c = w4a4.unpack_nibbles(packed.cpu())
    return torch.where(c >= 8, c - 16, c) if signed else c


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,K,R", [(64, 512, 32), (130, 3072, 32), (33, 256, 288), (1, 64, 16)])
def test_quantize_signed_exact(cuda_dev, dtype, M, K, R):
    Kn = _ops()
    g = torch.Generator().manual_seed(M + K)
    x = torch.randn(M, K, generator=g)
    x[:, ::97] *= 20
    x = x.to(dtype)
    ld = (torch.randn(K, R, generator=g) * 0.1).to(dtype)
    smooth = (torch.rand(K, generator=g) + 0.5).to(dtype)
    for sm in (None, smooth):
        packed, scales, lora = Kn.quantize_w4a4_act_fuse_lora(
            x.to(cuda_dev), lora_down=ld.to(cuda_dev), smooth=sm.to(cuda_dev) if sm is not None else None
        )
        rp, rs, rl, _ = w4a4.quantize_act(x, ld, sm)
        assert torch.equal(packed.cpu(), rp), "codes differ from the oracle"
        assert torch.equal(scales.cpu().view(torch.int16), rs.view(torch.int16)), "scales differ from the oracle"
        torch.testing.assert_close(lora.cpu(), rl, rtol=2e-3, atol=2e-3)
    # run twice: identical LoRA sums
    _, _, lora2 = Kn.quantize_w4a4_act_fuse_lora(x.to(cuda_dev), lora_down=ld.to(cuda_dev))
    _, _, lora3 = Kn.quantize_w4a4_act_fuse_lora(x.to(cuda_dev), lora_down=ld.to(cuda_dev))
    assert torch.equal(lora2, lora3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_quantize_fp4_exact(cuda_dev, dtype):
    Kn = _ops()
    torch.manual_seed(3)
    x = torch.randn(70, 512).to(dtype)
    packed, scales, _ = Kn.quantize_w4a4_act_fuse_lora(x.to(cuda_dev), fp4=True)
    rp, rs, _, _ = w4a4.quantize_act(x, fp4=True)
    assert scales.dtype == torch.float8_e4m3fn and scales.shape == (32, 70)
    assert torch.equal(packed.cpu(), rp)
    assert torch.equal(scales.cpu().view(torch.uint8), rs.view(torch.uint8))


@pytest.mark.parametrize("dtype", DTYPES)
def test_quantize_glu_gelu_unsigned(cuda_dev, dtype):
    Kn = _ops()
    torch.manual_seed(4)
    M, K, R = 48, 512, 32
    ld = (torch.randn(K, R) * 0.1).to(dtype)
    smooth = (torch.rand(K) + 0.5).to(dtype)
    # GLU (tests/triton/test_w4a4.py:229-238)
    x2 = torch.randn(M, 2 * K).to(dtype)
    packed, scales, lora = Kn.quantize_w4a4_act_fuse_lora(x2.to(cuda_dev), lora_down=ld.to(cuda_dev), fuse_glu=True)
    rp, rs, rl, rc = w4a4.quantize_act(x2, ld, fuse_glu=True)
    d = (_unpack_codes(packed, True) - torch.where(rc >= 8, rc - 16, rc)).abs()
    assert d.max() <= 1 and (d != 0).float().mean() < 1e-3
    torch.testing.assert_close(scales.float().cpu(), rs.float(), rtol=2**-7, atol=1e-7)
    torch.testing.assert_close(lora.cpu(), rl, rtol=1e-2, atol=1e-2)
    # GELU + shift + unsigned: the unfused next-layer quantisation (gemm_w4a4.py:1298-1312)
    x = (torch.randn(M, K) * 2).to(dtype)
    packed, scales, lora = Kn.quantize_w4a4_act_fuse_lora(
        x.to(cuda_dev), lora_down=ld.to(cuda_dev), smooth=smooth.to(cuda_dev), fuse_gelu=True,
        shift_value=w4a4.GELU_SHIFT, unsigned=True,
    )
    rp, rs, rl, rc = w4a4.quantize_act(x, ld, smooth, fuse_gelu=True, shift_value=w4a4.GELU_SHIFT, unsigned=True)
    d = (_unpack_codes(packed, False) - rc).abs()
    assert d.max() <= 1 and (d != 0).float().mean() < 1e-3
    torch.testing.assert_close(scales.float().cpu(), rs.float(), rtol=2**-7, atol=1e-7)
    torch.testing.assert_close(lora.cpu(), rl, rtol=1e-2, atol=1e-2)


def test_quantize_op_pads_rows(cuda_dev):
    from nunchaku_rocm_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    x = torch.randn(300, 256, dtype=torch.bfloat16, device=cuda_dev)
    ld = torch.randn(256, 32, dtype=torch.bfloat16, device=cuda_dev) * 0.1
    q, s, l = svdq_quantize_w4a4_act_fuse_lora_cuda(x, lora_down=ld)
    assert q.shape == (512, 128) and s.shape == (4, 512) and l.shape == (512, 32)
    rp, rs, rl, _ = w4a4.quantize_act(x.cpu(), ld.cpu())
    assert torch.equal(q[:300].cpu(), rp)


# ------------------------------------------------------------------------------------------------
# fused GELU / SwiGLU + next-layer quantisation (generic fused kernel and the unfused composition)
# ------------------------------------------------------------------------------------------------
def _check_requant(qout, osc, lao, codes_ref, scale_ref, lora_ref, M, signed, fused=False):
    # bars of the reference's self-test against its torch form (native/w4a4.py:689-702); a kernel that re-quantises
    # the fp32 tile inside the GEMM is held to a ten times smaller mismatch rate and to scales within one 16-bit step
    codes = _unpack_codes(qout[:M], signed)
    d = (codes - codes_ref).abs()
    rate = (d != 0).float().mean().item()
    assert d.max() <= 1 and rate < (2e-3 if fused else 1e-2), rate
    s = osc[:, :M].float().cpu()
    tol = 2.0**-7 if fused else 1e-2
    assert ((s - scale_ref).abs() <= tol * scale_ref.abs() + 1e-6).all()
    assert (lao[:M].cpu() - lora_ref).abs().max() <= 1e-2 * lora_ref.abs().max()


@pytest.mark.parametrize("impl", [0, GENERIC, SINGLE])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("R2", [32, 48])
def test_gelu_quant(cuda_dev, impl, dtype, R2):
    Kn = _ops()
    M, N, K, R = 144, 256, 256, 16
    for uns in (False, True):
        act, wgt, asc, wsc, bias, la, lu = _rand_problem(M, N, K, R, dtype, seed=R2, act_unsigned=uns)
        g = torch.Generator().manual_seed(R2)
        smooth = (torch.rand(N, generator=g) + 0.5).to(dtype)
        ld = (torch.randn(N, R2, generator=g) * 0.1).to(dtype)
        lin = w4a4.gemm_w4a4(act, wgt, asc, wsc, bias, la, lu, act_unsigned=uns)
        cr, sr, lr = w4a4.gelu_quant(lin, smooth, ld, dtype)
        qout = torch.zeros(M + 16, N // 2, dtype=torch.uint8, device=cuda_dev)
        osc = torch.empty(N // 64, M, dtype=dtype, device=cuda_dev)
        lao = torch.empty(M, R2, device=cuda_dev)
        Kn.gemm_w4a4(*_cuda(cuda_dev, act, wgt), None, *_cuda(cuda_dev, asc, wsc, bias, la, lu), qout=qout[:M],
                     oscales=osc, smooth_factor=smooth.to(cuda_dev), lora_down=ld.to(cuda_dev), lora_act_out=lao,
                     act_unsigned=uns, out_dtype=dtype, _impl=impl)
        _check_requant(qout, osc, lao, cr, sr, lr, M, signed=False, fused=impl != SINGLE)
        assert bool((qout[M:] == 0).all())
    _status_clean(cuda_dev)


@pytest.mark.parametrize("impl", [PAIR, GENERIC])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K,R,R2", [(144, 256, 256, 16, 48), (300, 1024, 384, 32, 32)])
def test_swiglu_quant(cuda_dev, impl, dtype, M, N, K, R, R2):
    Kn = _ops()
    H = N // 2
    act, wgt, asc, wsc, bias, la, lu = _rand_problem(M, N, K, R, dtype, seed=77)
    g = torch.Generator().manual_seed(78)
    smooth = (torch.rand(H, generator=g) + 0.5).to(dtype)
    ld = (torch.randn(H, R2, generator=g) * 0.1).to(dtype)
    lin = w4a4.gemm_w4a4(act, wgt, asc, wsc, bias, la, lu)  # [gate | up]
    cr, sr, lr = w4a4.swiglu_quant(lin, smooth, ld, dtype)
    idx = w4a4.interleave_swiglu(N)
    qout = torch.zeros(M, H // 2, dtype=torch.uint8, device=cuda_dev)
    osc = torch.empty(H // 64, M, dtype=dtype, device=cuda_dev)
    lao = torch.empty(M, R2, device=cuda_dev)
    Kn.gemm_w4a4(act.to(cuda_dev), wgt[idx].to(cuda_dev), None, asc.to(cuda_dev), wsc[:, idx].contiguous().to(cuda_dev),
                 bias[idx].to(cuda_dev), la.to(cuda_dev), lu[idx].to(cuda_dev), qout=qout, oscales=osc,
                 smooth_factor=smooth.to(cuda_dev), lora_down=ld.to(cuda_dev), lora_act_out=lao, fuse_swiglu=True, _impl=impl)
    _check_requant(qout, osc, lao, cr, sr, lr, M, signed=True, fused=True)
    _status_clean(cuda_dev)


# ------------------------------------------------------------------------------------------------
# NVFP4: the generic kernel and the block-scaled tensor-core kernel (kind::mxf4nvf4)
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_gemm_fp4_wcscales_alpha(cuda_dev, dtype):
    Kn = _ops()
    M, N, K = 128, 256, 512
    g = torch.Generator().manual_seed(11)
    act = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    wgt = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    asc = (torch.rand(K // 16, M, generator=g) * 0.05 + 0.01).to(torch.float8_e4m3fn)
    wsc = (torch.rand(K // 16, N, generator=g) * 0.05 + 0.01).to(torch.float8_e4m3fn)
    wcs = (torch.rand(N, generator=g) * 0.5 + 0.5).to(dtype)
    ref = w4a4.gemm_w4a4(act, wgt, asc, wsc, fp4=True, alpha=0.75, wcscales=wcs)
    out = Kn.gemm_w4a4(*_cuda(cuda_dev, act, wgt), None, *_cuda(cuda_dev, asc, wsc), wcscales=wcs.to(cuda_dev),
                       alpha=0.75, fp4=True, out_dtype=dtype)
    _close(out, ref, "fp4")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("impl", [GENERIC, 0])  # 0 = automatic: the block-scaled tensor-core kernel when the shape allows
@pytest.mark.parametrize("M,N,K,R", [
    (128, 128, 256, 0), (200, 264, 512, 32), (384, 640, 1024, 16), (130, 136, 768, 48),
    # N % 256 == 0 or N >= 2048: the 128 x 256 tile (low-rank slot served per 128-column half, ragged last tile)
    (128, 256, 256, 0), (300, 512, 512, 32), (257, 768, 1024, 80), (130, 2056, 512, 16),
    # K % 256 != 0: the last ring stage holds one, two or three 64-k steps
    (200, 264, 64, 16), (130, 512, 320, 32), (384, 640, 448, 0), (129, 256, 1216, 16),
])
def test_gemm_fp4_shapes_lora_bias(cuda_dev, dtype, impl, M, N, K, R):
    Kn = _ops()
    g = torch.Generator().manual_seed(M + N + K + R)
    act = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    wgt = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    asc = (torch.rand(K // 16, M, generator=g) * 0.05 + 0.01).to(torch.float8_e4m3fn)
    wsc = (torch.rand(K // 16, N, generator=g) * 0.05 + 0.01).to(torch.float8_e4m3fn)
    wcs = (torch.rand(N, generator=g) * 0.5 + 0.5).to(dtype)
    bias = torch.randn(N, generator=g).to(dtype)
    la = torch.randn(M, R, generator=g) * 0.5 if R else None
    lu = (torch.randn(N, R, generator=g) * 0.1).to(dtype) if R else None
    ref = w4a4.gemm_w4a4(act, wgt, asc, wsc, bias=bias, lora_act=la, lora_up=lu, fp4=True, alpha=1.25, wcscales=wcs)
    dv = lambda t: None if t is None else t.to(cuda_dev)
    out = Kn.gemm_w4a4(dv(act), dv(wgt), None, dv(asc), dv(wsc), dv(bias), dv(la), dv(lu), wcscales=dv(wcs), alpha=1.25,
                       fp4=True, out_dtype=dtype, _impl=impl)
    assert out.shape == (M, N)
    _close(out, ref, f"fp4 {M}x{N}x{K} R={R} impl={impl}")
    again = Kn.gemm_w4a4(dv(act), dv(wgt), None, dv(asc), dv(wsc), dv(bias), dv(la), dv(lu), wcscales=dv(wcs), alpha=1.25,
                         fp4=True, out_dtype=dtype, _impl=impl)
    assert torch.equal(out, again)
    _status_clean(cuda_dev)


def test_library_selftest(cuda_dev):
    # the C-level self-test (tensor-core kernel against the generic one) that a host without Python can call
    from nunchaku_rocm_b200 import _lib

    with torch.cuda.device(cuda_dev):
        assert _lib.lib().nb_selftest() == 0


def test_gemm_fp4_tensor_core_kernel_is_selected(cuda_dev):
    # the shapes above (K % 64 == 0) must run on the block-scaled kernel, not silently on the generic one
    import ctypes as C

    from nunchaku_rocm_b200 import _lib as L
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import _gemm_args

    for M, N, K in [(256, 256, 512), (130, 512, 320)]:
        act = torch.zeros(M, K // 2, dtype=torch.uint8, device=cuda_dev)
        wgt = torch.zeros(N, K // 2, dtype=torch.uint8, device=cuda_dev)
        asc = torch.zeros(K // 16, M, dtype=torch.float8_e4m3fn, device=cuda_dev)
        wsc = torch.zeros(K // 16, N, dtype=torch.float8_e4m3fn, device=cuda_dev)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=cuda_dev)
        a = _gemm_args(act, wgt, out, asc, wsc, None, None, None, None, False, False, True, 1.0, torch.bfloat16, L.IMPL_AUTO)
        assert L.lib().nb_gemm_w4a4_uses_tcgen05(C.byref(a), None, L.EPI_STORE) == 1


# ------------------------------------------------------------------------------------------------
# the benchmark configurations at full size
# ------------------------------------------------------------------------------------------------
def _cfg_problem(N, dev):
    from bench import make_cfg_inputs

    return make_cfg_inputs(4608, 3072, N, 32, dev)


def test_cfg0_full_size_parity(cuda_dev):
    from nunchaku_rocm_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    Kn = _ops()
    p = _cfg_problem(3072, cuda_dev)
    q, s, l = svdq_quantize_w4a4_act_fuse_lora_cuda(p["x"], lora_down=p["proj_down"], smooth=p["smooth"])
    rp, rs, rl, _ = w4a4.quantize_act(p["x"].cpu(), p["proj_down"].cpu(), p["smooth"].cpu())
    M = p["x"].shape[0]
    assert torch.equal(q[:M].cpu(), rp) and torch.equal(s[:, :M].cpu().view(torch.int16), rs.view(torch.int16))
    out = torch.empty(M, 3072, dtype=torch.bfloat16, device=cuda_dev)
    Kn.gemm_w4a4(q, p["qweight"], out, s, p["wscales"], p["bias"], l, p["proj_up"])
    ref = w4a4.gemm_w4a4(rp, p["qweight"].cpu(), rs, p["wscales"].cpu(), p["bias"].cpu(), rl, p["proj_up"].cpu())
    _close(out, ref, "cfg0")
    _status_clean(cuda_dev)


def test_cfg1_full_size_parity(cuda_dev):
    from nunchaku_rocm_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda

    Kn = _ops()
    p = _cfg_problem(9216, cuda_dev)
    q, s, l = svdq_quantize_w4a4_act_fuse_lora_cuda(p["x"], lora_down=p["proj_down"], smooth=p["smooth"])
    M = p["x"].shape[0]
    out = torch.empty(M, 9216, dtype=torch.bfloat16, device=cuda_dev)
    Kn.gemm_w4a4(q, p["qweight"], out, s, p["wscales"], p["bias"], l, p["proj_up"], norm_q=p["norm_q"],
                 norm_k=p["norm_k"], rotary_emb=p["rotary_emb"])
    lin = w4a4.gemm_w4a4(q[:M].cpu(), p["qweight"].cpu(), s[:, :M].cpu(), p["wscales"].cpu(), p["bias"].cpu(),
                         l[:M].cpu(), p["proj_up"].cpu())
    ref = w4a4.qk_norm_rope(lin, p["norm_q"].cpu(), p["norm_k"].cpu(), p["rotary_emb"].cpu().reshape(M, 128))
    _close(out, ref, "cfg1")
    _status_clean(cuda_dev)

"""
GPU parity tests of the AWQ W4A16 operators and the attention operator against the CPU oracle, with the bars of
the reference's own tests (tests/triton/test_gemm.py:98-159: exact dequantisation round trip, rtol/atol 3e-2 for the
GEMV / GEMM; tests/triton/test_w4a4.py:241-254: rtol/atol 3e-2 for attention).
"""

import pytest
import torch

from oracle import awq_attn

pytestmark = pytest.mark.gpu
DTYPES = [torch.bfloat16, torch.float16]


def _awq_problem(n, k, m, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 16, (n, k), dtype=torch.int32, generator=g)
    s = (torch.rand(k // 64, n, generator=g) * 0.1 + 0.01).to(dtype)
    z = (torch.randn(k // 64, n, generator=g) * 0.1).to(dtype)
    x = torch.randn(m, k, generator=g).to(dtype)
    return q, awq_attn.awq_pack(q), s, z, x


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,k", [(64, 128), (256, 3072), (72, 192)])
def test_awq_dequantize_exact(cuda_dev, dtype, n, k):
    from nunchaku_rocm_b200.ops.triton.awq import awq_dequantize

    q, packed, s, z, _ = _awq_problem(n, k, 1, dtype, seed=n)
    w = awq_dequantize(packed.to(cuda_dev), s.to(cuda_dev), z.to(cuda_dev), n, k, 64, dtype)
    ref = awq_attn.awq_dequant(packed, s, z, n, k).to(dtype)
    assert torch.equal(w.cpu(), ref)
    # unit scale, zero offset: the codes come back exactly
    ones, zeros = torch.ones_like(s), torch.zeros_like(z)
    w = awq_dequantize(packed.to(cuda_dev), ones.to(cuda_dev), zeros.to(cuda_dev), n, k, 64, dtype)
    assert torch.equal(w.cpu().to(torch.int32), q)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [1, 2, 3, 8, 11])
@pytest.mark.parametrize("n,k", [(256, 512), (18432, 3072)])
def test_awq_gemv(cuda_dev, dtype, m, n, k):
    from nunchaku_rocm_b200.ops.gemv import awq_gemv_w4a16_cuda

    _, packed, s, z, x = _awq_problem(n, k, m, dtype, seed=m + n)
    out = awq_gemv_w4a16_cuda(x.to(cuda_dev), packed.to(cuda_dev), s.to(cuda_dev), z.to(cuda_dev), m, n, k, 64)
    assert out.shape == (m, n) and out.dtype == dtype
    ref = awq_attn.awq_gemv(x, packed, s, z, n, k)
    torch.testing.assert_close(out.float().cpu(), ref, rtol=3e-2, atol=3e-2)
    # tighter: within two 16-bit rounding steps of the fp32 sum
    eps = 2.0**-7 if dtype == torch.bfloat16 else 2.0**-10
    assert ((out.float().cpu() - ref).abs() <= eps * ref.abs() + 2e-2).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k,group", [(40, 384, 256, 128), (300, 1000, 512, 64), (129, 132, 64, 64), (1024, 4096, 1024, 128)])
def test_awq_gemm_kernel(cuda_dev, dtype, m, n, k, group):
    """The one-kernel W4A16 GEMM against ``x @ T(q * s + z)^T`` in fp32 (reference: awq.py:232-251), tails included."""
    from nunchaku_rocm_b200.ops.triton.awq import awq_gemm_w4a16

    g = torch.Generator().manual_seed(m + n + k)
    q = torch.randint(0, 16, (n, k), dtype=torch.int32, generator=g)
    s = (torch.rand(k // group, n, generator=g) * 0.1 + 0.01).to(dtype)
    z = (torch.randn(k // group, n, generator=g) * 0.1).to(dtype)
    x = torch.randn(m, k, generator=g).to(dtype)
    packed = awq_attn.awq_pack(q)
    canvas = torch.full((m + 2, n), 7.0, dtype=dtype, device=cuda_dev)  # (the op allocates its own output; canary for the view below)
    out = awq_gemm_w4a16(x.to(cuda_dev), packed.to(cuda_dev), s.to(cuda_dev), z.to(cuda_dev), group)
    assert out.shape == (m, n) and (canvas == 7.0).all()
    w = awq_attn.awq_dequant(packed, s, z, n, k, group).to(dtype).float()  # the weight as the kernel rounds it
    ref = x.float() @ w.T
    eps = 2.0**-8 if dtype == torch.bfloat16 else 2.0**-11
    # one rounding of the fp32 sum to the 16-bit dtype, plus the order of the fp32 additions
    assert ((out.float().cpu() - ref).abs() <= eps * ref.abs() + 1e-3 * ref.abs().max()).all()
    # a strided activation view (rows 16-byte aligned) goes through the same kernel
    xx = torch.zeros(m, k + 8, dtype=dtype, device=cuda_dev)
    xx[:, :k] = x.to(cuda_dev)
    out2 = awq_gemm_w4a16(xx[:, :k], packed.to(cuda_dev), s.to(cuda_dev), z.to(cuda_dev), group)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_awq_gemm_and_linear(cuda_dev, dtype):
    from nunchaku_rocm_b200.models.linear import AWQW4A16Linear
    from nunchaku_rocm_b200.ops.dispatch import gemm_awq

    n, k, m = 384, 256, 40
    g = torch.Generator().manual_seed(5)
    q = torch.randint(0, 16, (n, k), dtype=torch.int32, generator=g)
    s128 = (torch.rand(k // 128, n, generator=g) * 0.1 + 0.01).to(dtype)
    z128 = (torch.randn(k // 128, n, generator=g) * 0.1).to(dtype)
    x = torch.randn(m, k, generator=g).to(dtype)
    packed = awq_attn.awq_pack(q)
    out = gemm_awq(x.to(cuda_dev), packed.to(cuda_dev), s128.to(cuda_dev), z128.to(cuda_dev))
    ref = x.float() @ awq_attn.awq_dequant(packed, s128, z128, n, k, 128).float().T
    # 16-bit weights and a 16-bit output of magnitude ~10: assess the tile as a whole
    err = (out.float().cpu() - ref).norm() / ref.norm()
    assert err <= 1e-2, err

    lin = AWQW4A16Linear(k, n, bias=True, group_size=64, torch_dtype=dtype, device=cuda_dev)
    _, packed, s, z, x = _awq_problem(n, k, 4, dtype, seed=9)
    bias = torch.randn(n, generator=g).to(dtype)
    lin.qweight.data.copy_(packed)
    lin.wscales.data.copy_(s)
    lin.wzeros.data.copy_(z)
    lin.bias.data.copy_(bias)
    y = lin(x.to(cuda_dev))
    ref = awq_attn.awq_gemv(x, packed, s, z, n, k).to(dtype).float() + bias.float()
    torch.testing.assert_close(y.float().cpu(), ref, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("impl", [0, 1, 2])  # 0: automatic, 1: the tcgen05 kernel or an error (D = 128), 2: the mma.sync kernel
@pytest.mark.parametrize(
    "B,H,TQ,TKV,D",
    [(2, 8, 256, 256, 64), (1, 4, 128, 512, 128), (2, 2, 100, 77, 64), (1, 3, 333, 1000, 128), (2, 3, 640, 1, 128),
     (1, 2, 130, 129, 128)],
)
def test_attention(cuda_dev, dtype, impl, B, H, TQ, TKV, D):
    from nunchaku_rocm_b200 import _lib
    from nunchaku_rocm_b200.ops.triton.attention import attention_fp16

    if impl != 0 and D == 64:
        pytest.skip("D = 64 always runs on the mma.sync kernel; covered by impl 0")
    g = torch.Generator().manual_seed(TQ)
    q = torch.randn(B, H, TQ, D, generator=g).to(dtype)
    k = torch.randn(B, H, TKV, D, generator=g).to(dtype)
    v = torch.randn(B, H, TKV, D, generator=g).to(dtype)
    # larger scores in some rows, so that the running maximum grows a lot along the keys
    q[:, :, ::7] *= 6.0
    o = torch.empty(B, TQ, H * D, dtype=dtype, device=cuda_dev)
    attention_fp16(q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev), o, D**-0.5, _impl=impl)
    torch.cuda.synchronize(cuda_dev)
    assert _lib.device_status(cuda_dev) == 0
    # against exact fp32 attention: the reference's bar (rtol 3e-2); the rows with scores scaled by 6 make the bf16 rounding
    # of q * scale * log2(e) visible, hence the wider absolute bar for bf16
    tol = 3e-2 if dtype == torch.float16 else 6e-2
    torch.testing.assert_close(o.float().cpu(), awq_attn.attention_exact(q, k, v, D**-0.5), rtol=3e-2, atol=tol)
    # against the oracle with the kernel's rounding points: one 16-bit rounding step
    eps = 2.0**-7 if dtype == torch.bfloat16 else 2.0**-10
    torch.testing.assert_close(o.float().cpu(), awq_attn.attention(q, k, v, D**-0.5), rtol=2 * eps, atol=2 * eps)


def test_attention_with_keys_broadcast_over_heads(cuda_dev):
    # one K / V head expanded over all query heads (stride 0 on the head axis): the strides are the contract
    # (nunchaku/ops/triton/attention.py:120-169 passes them to the kernel as they are)
    from nunchaku_rocm_b200 import _lib
    from nunchaku_rocm_b200.ops.triton.attention import attention_fp16

    B, H, TQ, TKV, D = 2, 4, 160, 200, 128
    g = torch.Generator().manual_seed(11)
    q = torch.randn(B, H, TQ, D, generator=g).to(torch.bfloat16)
    k1 = torch.randn(B, 1, TKV, D, generator=g).to(torch.bfloat16)
    v1 = torch.randn(B, 1, TKV, D, generator=g).to(torch.bfloat16)
    kd, vd = k1.to(cuda_dev).expand(B, H, TKV, D), v1.to(cuda_dev).expand(B, H, TKV, D)
    assert kd.stride(1) == 0
    o = torch.empty(B, TQ, H * D, dtype=torch.bfloat16, device=cuda_dev)
    attention_fp16(q.to(cuda_dev), kd, vd, o, D**-0.5)
    torch.cuda.synchronize(cuda_dev)
    assert _lib.device_status(cuda_dev) == 0
    want = awq_attn.attention(q, k1.expand(B, H, TKV, D), v1.expand(B, H, TKV, D), D**-0.5)
    torch.testing.assert_close(o.float().cpu(), want, rtol=2.0**-6, atol=2.0**-6)


def test_sdpa_wrapper_strided_views_and_fallback(cuda_dev):
    # (B, S, 3 * H * D) fused projection viewed as q, k, v, the way the FLUX processor slices it
    from nunchaku_rocm_b200.ops.dispatch import scaled_dot_product_attention

    B, S, H, D = 2, 300, 4, 128
    torch.manual_seed(0)
    qkv = torch.randn(B, S, 3 * H * D, dtype=torch.bfloat16, device=cuda_dev)
    q, k, v = (t.view(B, S, H, D).transpose(1, 2) for t in qkv.chunk(3, dim=-1))
    out = scaled_dot_product_attention(q, k, v)
    assert out.shape == (B, H, S, D)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
    torch.testing.assert_close(out.float(), ref, rtol=3e-2, atol=3e-2)
    # a mask goes to torch
    mask = torch.ones(S, S, dtype=torch.bool, device=cuda_dev)
    out2 = scaled_dot_product_attention(q, k, v, attn_mask=mask)
    torch.testing.assert_close(out2.float(), ref, rtol=3e-2, atol=3e-2)

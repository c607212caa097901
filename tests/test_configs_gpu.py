"""
Parity at the sizes the benchmark configurations state, through the public operators and the C ABI.

The GPU computes the full problem; the CPU oracle evaluates a seeded SAMPLE OF ROWS of the same problem at the full K and
N (rows of a GEMM, of the quantizer and of the row-wise epilogues are independent, so a row sample is a complete check of
those rows).  Configurations:

* MLP pair 3072 -> 12288 -> 3072 with the GELU / next-layer int4 re-quantisation between the two GEMMs, M in
  {256, 1024, 4608, 8192}; bars of the reference's own test of that epilogue (tests/triton/test_native_epilogues.py:214-268):
  codes at most one apart, mismatches counted and reported, scales within one rounding step, de-quantised RMS error no
  worse than the oracle's own codes.
* NVFP4 GEMMs of the Qwen-Image block at 7168 rows (7168 x 9216 x 3072, 7168 x 3072 x 12288) with rank-32 branch, bias,
  per-channel scale and alpha, and the NVFP4 quantizer at that width.
* attention at B = 1, H = 24, D = 128 for T = 4608 (FLUX, 36 full key tiles) and T = 7145 (Qwen-Image, ragged last tile),
  three heads checked.
"""

import ctypes as C

import pytest
import torch

from oracle import awq_attn, w4a4

pytestmark = pytest.mark.gpu
T = torch.bfloat16
N_SAMPLE = 96


def _sample_rows(M, n, seed):
    g = torch.Generator().manual_seed(seed)
    n = min(n, M)
    rows = torch.randperm(M, generator=g)[:n].sort().values
    rows[0], rows[-1] = 0, M - 1  # the edges of the first and the last tile are always in
    return rows.unique()


def _svdq_weights(cin, cout, rank, seed, dev):
    """int4 weights U[-8, 7], per-64 scales U(0.005, 0.02), rank-`rank` branch N(0, 0.02), bias, smooth U(0.5, 1.5)."""
    g = torch.Generator().manual_seed(seed)
    p = dict(
        qweight=torch.randint(0, 256, (cout, cin // 2), dtype=torch.uint8, generator=g),
        wscales=(torch.rand(cin // 64, cout, generator=g) * 0.015 + 0.005).to(T),
        bias=(torch.randn(cout, generator=g) * 0.1).to(T),
        smooth=(torch.rand(cin, generator=g) + 0.5).to(T),
        proj_down=(torch.randn(cin, rank, generator=g) * 0.02).to(T),
        proj_up=(torch.randn(cout, rank, generator=g) * 0.02).to(T),
    )
    return p, {k: v.to(dev) for k, v in p.items()}


@pytest.fixture(scope="module")
def mlp_weights(cuda_dev):
    return _svdq_weights(3072, 12288, 32, 21, cuda_dev), _svdq_weights(12288, 3072, 32, 22, cuda_dev)


def _ulp(x, dtype):
    """Size of one rounding step of `dtype` at |x| (x fp32)."""
    bits = 8 if dtype == torch.bfloat16 else 11
    return torch.exp2(torch.floor(torch.log2(x.abs().clamp_min(1e-30))) - (bits - 1))


@pytest.mark.parametrize("M", [256, 1024, 4608, 8192])
def test_mlp_pair_at_stated_size(cuda_dev, mlp_weights, M):
    from nunchaku_rocm_b200 import _lib as L
    from nunchaku_rocm_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda as quantize
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import GELU_SHIFT, _gemm_args, _requant_args, gemm_w4a4

    (c1, d1), (c2, d2) = mlp_weights
    g = torch.Generator().manual_seed(1000 + M)
    x = torch.randn(M, 3072, generator=g)
    x[:, torch.randperm(3072, generator=g)[:8]] *= 20
    x = x.to(T)
    xd = x.to(cuda_dev)

    # ---- GPU: quantize -> fc1 (+ GELU, shift, unsigned requant, fc2's LoRA-down) -> fc2 --------------------------------
    q, s, l = quantize(xd, lora_down=d1["proj_down"], smooth=d1["smooth"])
    m_pad = q.shape[0]
    qout = torch.zeros(m_pad, 12288 // 2, dtype=torch.uint8, device=cuda_dev)
    osc = torch.zeros(12288 // 64, m_pad, dtype=T, device=cuda_dev)
    lao = torch.zeros(m_pad, 32, dtype=torch.float32, device=cuda_dev)
    gemm_w4a4(q, d1["qweight"], None, s, d1["wscales"], d1["bias"], l, d1["proj_up"], qout=qout, oscales=osc,
              smooth_factor=d2["smooth"], lora_down=d2["proj_down"], lora_act_out=lao)
    out = torch.empty(M, 3072, dtype=T, device=cuda_dev)
    gemm_w4a4(qout, d2["qweight"], out, osc, d2["wscales"], d2["bias"], lao, d2["proj_up"], act_unsigned=True)
    torch.cuda.synchronize(cuda_dev)
    assert L.device_status(cuda_dev) == 0
    a = _gemm_args(q, d1["qweight"], None, s, d1["wscales"], d1["bias"], l, d1["proj_up"], None, False, False, False, 1.0,
                   T, L.IMPL_AUTO)
    rq, _keep = _requant_args(qout, osc, d2["smooth"], d2["proj_down"], lao, GELU_SHIFT, 12288, m_pad, T)
    fused = L.lib().nb_gemm_w4a4_uses_tcgen05(C.byref(a), C.byref(rq), L.EPI_GELU_QUANT) == 1

    # ---- oracle on sampled rows, full K and N ---------------------------------------------------------------------------
    rows = _sample_rows(M, N_SAMPLE, M)
    rp, rs, rl, _ = w4a4.quantize_act(x[rows], c1["proj_down"], c1["smooth"])
    assert torch.equal(q[rows.to(cuda_dev)].cpu(), rp), "quantizer codes differ from the oracle"
    assert torch.equal(s[:, rows.to(cuda_dev)].cpu().view(torch.int16), rs.view(torch.int16)), "quantizer scales differ"
    lin = w4a4.gemm_w4a4(rp, c1["qweight"], rs, c1["wscales"], c1["bias"], rl, c1["proj_up"])
    cr, sr, lr = w4a4.gelu_quant(lin, c2["smooth"], c2["proj_down"], T)

    rd = rows.to(cuda_dev)
    codes = w4a4.unpack_nibbles(qout[rd].cpu())
    d = (codes - cr).abs()
    mismatch = (d != 0).float().mean().item()
    sg = osc[:, rd].float().cpu()
    s_ulps = ((sg - sr.to(T).float()).abs() / _ulp(sr, T)).max().item()
    x2 = (w4a4.gelu_tanh(lin) + GELU_SHIFT) * (1.0 / c2["smooth"].float())[None, :]

    def deq_err(c, sc):
        deq = c.float().view(len(rows), -1, 64) * sc.t().float()[..., None]
        return ((deq.reshape(len(rows), -1) - x2).pow(2).mean().sqrt() / x2.pow(2).mean().sqrt()).item()

    ratio = deq_err(codes, sg) / deq_err(cr, sr.to(T).float())
    lora_err = ((lao[rd].cpu() - lr).abs().max() / lr.abs().max()).item()
    print(f"\nMLP pair M={M} fused={fused}: code mismatches {mismatch:.2e} (max distance {int(d.max())}), "
          f"scales within {s_ulps:.2f} ulp, de-quantised RMS ratio {ratio:.5f}, lora_act_out error {lora_err:.2e}")
    assert d.max() <= 1
    if fused:
        # the epilogue works on the fp32 tile, like the reference's fused kernel: only fp32 summation order differs
        assert mismatch < 2e-3 and s_ulps <= 1.0 and ratio <= 1.001
    else:
        # GEMM -> 16-bit tile -> quantizer with the GELU fused (the reference's own path for calls its fused kernel does
        # not take, gemm_w4a4.py:1298-1312): one more rounding before the GELU
        assert mismatch < 3e-2 and s_ulps <= 2.0 and ratio <= 1.02
    assert lora_err <= 1e-2

    # ---- fc2: on the GPU's own re-quantised activations (isolates the second GEMM), and the whole chain -----------------
    ref_own = w4a4.gemm_w4a4(qout[rd].cpu(), c2["qweight"], osc[:, rd].cpu(), c2["wscales"], c2["bias"], lao[rd].cpu(),
                             c2["proj_up"], act_unsigned=True)
    err_own = w4a4.rel_fro(out[rd].float().cpu(), ref_own)
    ref_chain = w4a4.gemm_w4a4(w4a4.pack_nibbles(cr), c2["qweight"], sr.to(T), c2["wscales"], c2["bias"], lr, c2["proj_up"],
                               act_unsigned=True)
    err_chain = w4a4.rel_fro(out[rd].float().cpu(), ref_chain)
    print(f"fc2 rel-Frobenius {err_own:.2e} on its own input, {err_chain:.2e} for the chain")
    assert err_own <= 1e-2
    assert err_chain <= 2e-2


@pytest.mark.parametrize("N,K", [(9216, 3072), (3072, 12288)])
def test_nvfp4_gemm_at_qwen_image_size(cuda_dev, N, K):
    from nunchaku_rocm_b200 import _lib as L
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import gemm_w4a4

    M, R = 7168, 32
    g = torch.Generator().manual_seed(N + K)
    act = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    wgt = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    asc = (torch.rand(K // 16, M, generator=g) * 0.05 + 0.01).to(torch.float8_e4m3fn)
    wsc = (torch.rand(K // 16, N, generator=g) * 0.05 + 0.01).to(torch.float8_e4m3fn)
    wcs = (torch.rand(N, generator=g) * 0.5 + 0.5).to(T)
    bias = (torch.randn(N, generator=g) * 0.1).to(T)
    la = torch.randn(M, R, generator=g) * 0.5
    lu = (torch.randn(N, R, generator=g) * 0.02).to(T)
    dv = lambda t: t.to(cuda_dev)
    out = gemm_w4a4(dv(act), dv(wgt), None, dv(asc), dv(wsc), dv(bias), dv(la), dv(lu), wcscales=dv(wcs), alpha=0.8,
                    fp4=True, out_dtype=T)
    torch.cuda.synchronize(cuda_dev)
    assert L.device_status(cuda_dev) == 0
    rows = _sample_rows(M, 512, N)
    ref = w4a4.gemm_w4a4(act[rows], wgt, asc[:, rows].contiguous(), wsc, bias=bias, lora_act=la[rows], lora_up=lu, fp4=True,
                         alpha=0.8, wcscales=wcs)
    got = out[rows.to(cuda_dev)].float().cpu()
    err = w4a4.rel_fro(got, ref)
    print(f"\nNVFP4 7168x{N}x{K}: rel-Frobenius {err:.2e} on {len(rows)} rows")
    assert err <= 1e-2
    assert (got - ref).abs().max() <= 1e-2 * ref.abs().max()


def test_nvfp4_quantizer_at_qwen_image_mlp_width(cuda_dev):
    # the re-quantisation between the two MLP GEMMs of the NVFP4 model: 7168 rows x 12288 columns, group 16, e4m3 scales
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import quantize_w4a4_act_fuse_lora

    M, K = 7168, 12288
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(M, K, generator=g) * 1.5).to(T)
    ld = (torch.randn(K, 32, generator=g) * 0.02).to(T)
    sm = (torch.rand(K, generator=g) + 0.5).to(T)
    q, s, l = quantize_w4a4_act_fuse_lora(x.to(cuda_dev), lora_down=ld.to(cuda_dev), smooth=sm.to(cuda_dev), fp4=True)
    rows = _sample_rows(M, 128, 9)
    rp, rs, rl, _ = w4a4.quantize_act(x[rows], ld, sm, fp4=True)
    rd = rows.to(cuda_dev)
    assert torch.equal(q[rd].cpu(), rp)
    assert torch.equal(s[:, rd].cpu().view(torch.uint8), rs.view(torch.uint8))
    torch.testing.assert_close(l[rd].cpu(), rl, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("Tk", [4608, 7145])
def test_attention_at_model_sequence_length(cuda_dev, Tk):
    from nunchaku_rocm_b200 import _lib as L
    from nunchaku_rocm_b200.ops.triton.attention import attention_fp16

    B, H, D = 1, 24, 128
    g = torch.Generator().manual_seed(Tk)
    # the fused projection's layout: one (B, T, 3 H D) tensor viewed as strided q, k, v
    qkv = torch.randn(B, Tk, 3 * H * D, generator=g).to(T)
    q, k, v = (t.view(B, Tk, H, D).transpose(1, 2) for t in qkv.chunk(3, dim=-1))
    qkv_d = qkv.to(cuda_dev)
    qd, kd, vd = (t.view(B, Tk, H, D).transpose(1, 2) for t in qkv_d.chunk(3, dim=-1))
    o = torch.empty(B, Tk, H * D, dtype=T, device=cuda_dev)
    attention_fp16(qd, kd, vd, o, D**-0.5)
    torch.cuda.synchronize(cuda_dev)
    assert L.device_status(cuda_dev) == 0
    heads = [0, 11, 23]
    got = o.view(B, Tk, H, D)[:, :, heads].reshape(B, Tk, len(heads) * D).float().cpu()
    qs, ks, vs = (t[:, heads].contiguous() for t in (q, k, v))
    exact = awq_attn.attention_exact(qs, ks, vs, D**-0.5)
    torch.testing.assert_close(got, exact, rtol=3e-2, atol=3e-2)  # the reference's bar (tests/triton/test_w4a4.py:241-254)
    # against the oracle with the kernel's rounding points: outputs are averages of ~T values of size ~1, i.e. ~T^-0.5
    rounded = awq_attn.attention(qs, ks, vs, D**-0.5)
    torch.testing.assert_close(got, rounded, rtol=2.0**-6, atol=2.0**-9)
    steps = (got - rounded).abs().max().item() / 2.0**-8
    err = w4a4.rel_fro(got, exact)
    print(f"\nattention T={Tk}: rel-Frobenius {err:.2e} vs exact fp32, max |diff| {steps:.3f} bf16 steps at 1.0 vs the oracle")
    assert err <= 1e-2

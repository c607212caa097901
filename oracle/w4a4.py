"""
CPU restatement of the SVDQuant W4A4 path of nunchaku-rocm (test infrastructure, not product code).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the
product path never does. Every function names the reference lines it follows
(paths are relative to the reference project's root).

Data conventions (nunchaku/ops/triton/gemm_w4a4.py:12-19):
  packed 4-bit tensors are uint8 ``[rows, K // 2]``; element ``k`` is the low nibble of byte
  ``k // 2`` when ``k`` is even, the high nibble when odd.  Scales are group-major
  ``[K // G, rows]`` with ``G = 64`` (int4) or ``16`` (NVFP4).

Parity status: pinned.  ``tests/golden/make_golden.py`` runs the reference's own pure-PyTorch
functions (nunchaku/ops/triton/native/w4a4.py:707-766, the packer and layout modules) on seeded
inputs and the fixtures it wrote are compared with this module in ``tests/test_oracle.py``.
The pieces that exist only as Triton kernels in the reference (plain activation quantizer, NVFP4
decode/encode) are restated from the cited kernel lines and pinned through the reference's
own test bounds (tests/triton/test_w4a4.py:187-238, 319-380).
"""

from __future__ import annotations

import torch

GELU_SHIFT = 0.171875  # nunchaku/ops/triton/native/w4a4.py:75
HEAD_DIM = 128  # nunchaku/ops/triton/native/w4a4.py:74
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)  # nunchaku/ops/triton/gemm_w4a4.py:85-86


# ----------------------------------------------------------------------------------------------
# nibble packing
# ----------------------------------------------------------------------------------------------
def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    """``[rows, K/2]`` bytes -> ``[rows, K]`` raw codes 0..15 (tests/triton/test_w4a4.py:23-29)."""
    b = packed.view(torch.uint8).to(torch.int32)
    return torch.stack([b & 0xF, b >> 4], dim=-1).reshape(packed.shape[0], -1)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`unpack_nibbles` (nunchaku/ops/triton/gemm_w4a4.py:1448-1455)."""
    c = (codes.to(torch.int32) & 0xF).reshape(codes.shape[0], -1, 2)
    return (c[..., 0] | (c[..., 1] << 4)).to(torch.uint8)


def int4_values(packed: torch.Tensor, signed: bool) -> torch.Tensor:
    """Integer values of packed int4 (nunchaku/ops/triton/native/w4a4.py:707-710)."""
    x = unpack_nibbles(packed)
    return torch.where(x >= 8, x - 16, x) if signed else x


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    """4-bit e2m1 code -> fp32 (nunchaku/ops/triton/gemm_w4a4.py:89-113)."""
    table = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32)
    return table[codes.long()]


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """
    fp32 -> e2m1 code with the reference's thresholds (nunchaku/ops/triton/gemm_w4a4.py:116-135):
    strict ``<`` against the midpoints, so an exact tie goes to the larger magnitude; sign bit 8
    is set only for ``x < 0``.
    """
    a = x.abs()
    code = torch.zeros_like(a, dtype=torch.int32)
    for mid in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        code += (a >= mid).to(torch.int32)
    return code | torch.where(x < 0, 8, 0).to(torch.int32)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """nunchaku/ops/triton/_common.py:70-78 (exp form of tanh), fp32."""
    x = x.float()
    inner = 0.79788456 * (x + 0.044715 * x * x * x)
    t = 2.0 / (1.0 + torch.exp(-2.0 * inner)) - 1.0
    return 0.5 * x * (1.0 + t)


def silu(x: torch.Tensor) -> torch.Tensor:
    """nunchaku/ops/triton/_common.py:90-94."""
    x = x.float()
    return x / (1.0 + torch.exp(-x))


# ----------------------------------------------------------------------------------------------
# activation quantizer (A.1)
# ----------------------------------------------------------------------------------------------
def quantize_act(
    x: torch.Tensor,
    lora_down: torch.Tensor | None = None,
    smooth: torch.Tensor | None = None,
    fuse_glu: bool = False,
    fp4: bool = False,
    fuse_gelu: bool = False,
    shift_value: float = 0.0,
    unsigned: bool = False,
):
    """
    ``_quantize_tile_kernel`` (nunchaku/ops/triton/gemm_w4a4.py:1338-1462) in evaluation order.

    Returns ``(packed [M, K/2] uint8, scales [K/G, M] in x.dtype (or e4m3 for fp4),
    lora_act [M, R] fp32 or None, codes [M, K] int32)``.
    """
    T = x.dtype
    xf = x.float()
    if fuse_glu:  # :1401-1405
        K = x.shape[1] // 2
        xf = xf[:, :K] * silu(xf[:, K:])
    if fuse_gelu:  # :1406-1407
        xf = gelu_tanh(xf)
    M, K = xf.shape
    G = 16 if fp4 else 64
    lora_act = None
    if lora_down is not None:  # :1409-1417 - before shift and smoothing, x rounded to the 16-bit dtype
        lora_act = xf.to(lora_down.dtype).float() @ lora_down.float()
    xf = xf + shift_value  # :1420
    if smooth is not None:  # :1421-1422 reciprocal-multiply
        xf = xf * (1.0 / smooth.float())[None, :]
    xg = xf.view(M, K // G, G)
    gmax = xg.amax(-1) if unsigned else xg.abs().amax(-1)  # :1424-1428
    gmax = gmax.clamp_min(0.0)
    qmax = 6.0 if fp4 else (15.0 if unsigned else 7.0)  # :1385-1390
    scale = gmax / qmax
    scale_safe = torch.where(scale == 0, torch.ones_like(scale), scale)  # :1431
    q = xg * (1.0 / scale_safe)[..., None]  # :1440 - unrounded fp32 scale
    if fp4:
        codes = e2m1_encode(q)
        scales_out = scale.t().contiguous().to(torch.float8_e4m3fn)
    else:
        r = torch.round(q)  # half-to-even, as the magic-number add (:1317-1325)
        r = r.clamp(0, 15) if unsigned else r.clamp(-8, 7)
        codes = r.to(torch.int32) & 0xF
        scales_out = scale.t().contiguous().to(T)  # :1433-1438 stored rounded, transposed
    codes = codes.view(M, K)
    return pack_nibbles(codes), scales_out, lora_act, codes


# ----------------------------------------------------------------------------------------------
# GEMM core + epilogue stage 1 (A.2, A.3)
# ----------------------------------------------------------------------------------------------
def group_dots_int32(act: torch.Tensor, wgt: torch.Tensor, act_unsigned: bool) -> torch.Tensor:
    """
    Exact int32 ``p_g[m, n]`` for every 64-group: ``[K/64, M, N]`` (the quantity the GEMM's
    integer path must reproduce bit-for-bit; nunchaku/ops/triton/gemm_w4a4.py:477-483).
    """
    a = int4_values(act, not act_unsigned).float()
    w = int4_values(wgt, True).float()
    G = a.shape[1] // 64
    out = torch.empty(G, a.shape[0], w.shape[0], dtype=torch.int32)
    for g in range(G):
        sl = slice(64 * g, 64 * g + 64)
        out[g] = (a[:, sl] @ w[:, sl].T).to(torch.int32)  # |p| <= 7680: exact in fp32
    return out


def gemm_core(act, wgt, ascales, wscales, act_unsigned=False, fp4=False) -> torch.Tensor:
    """
    ``acc[m,n] = sum_g as[g,m] * ws[g,n] * (A_g . W_g^T)`` in fp32
    (int4: nunchaku/ops/triton/native/w4a4.py:713-720; NVFP4: nunchaku/ops/triton/gemm_w4a4.py:302-350
    with the dequantisation of tests/triton/test_w4a4.py:32-42).
    """
    if fp4:
        a = e2m1_decode(unpack_nibbles(act))
        w = e2m1_decode(unpack_nibbles(wgt))
        G = 16
    else:
        a = int4_values(act, not act_unsigned).float()
        w = int4_values(wgt, True).float()
        G = 64
    M, K = a.shape
    N = w.shape[0]
    asf = ascales.float()[:, :M]
    wsf = wscales.float()[:, :N]
    if fp4:
        # every 16-wide partial dot is exact in fp32, so scaling the operands first is the same sum
        grp = torch.arange(K) // G
        return (a * asf[grp].t()) @ (w * wsf[grp].t()).t()
    out = torch.zeros(M, N)
    for g in range(K // G):
        sl = slice(G * g, G * g + G)
        out += (a[:, sl] @ w[:, sl].T) * asf[g][:, None] * wsf[g][None, :]
    return out


def gemm_w4a4(
    act,
    wgt,
    ascales,
    wscales,
    bias=None,
    lora_act=None,
    lora_up=None,
    act_unsigned=False,
    fp4=False,
    alpha=1.0,
    wcscales=None,
    fuse_silu=False,
) -> torch.Tensor:
    """
    fp32 tile after ``_w4a4_epilogue`` (nunchaku/ops/triton/gemm_w4a4.py:155-209): wcscale, alpha,
    LoRA-up with ``lora_act`` rounded to ``lora_up``'s dtype, bias, optional SiLU.  With the default
    flags this is ``reference()`` of nunchaku/ops/triton/native/w4a4.py:713-726.
    """
    out = gemm_core(act, wgt, ascales, wscales, act_unsigned, fp4)
    M, N = out.shape
    if wcscales is not None:
        out = out * wcscales.float()[None, :N]
    if alpha is not None and alpha != 1.0:
        out = out * alpha
    if lora_up is not None and lora_up.shape[1]:
        R = lora_up.shape[1]
        out = out + lora_act[:M, :R].to(lora_up.dtype).float() @ lora_up[:N].float().T
    if bias is not None:
        out = out + bias[:N].float()
    if fuse_silu:
        out = silu(out)
    return out


# ----------------------------------------------------------------------------------------------
# fused epilogues (A.4, A.5, SwiGLU)
# ----------------------------------------------------------------------------------------------
def qk_norm_rope(lin: torch.Tensor, norm_q, norm_k, rot, eps: float = 1e-6) -> torch.Tensor:
    """
    Per-head RMSNorm + RoPE on the Q and K thirds of ``lin`` (rows, N), V untouched
    (nunchaku/ops/triton/native/w4a4.py:729-740; kernel form nunchaku/ops/triton/gemm_w4a4.py:498-521).
    ``rot`` is ``(rows, 128)`` fp32 of ``(sin, cos)`` pairs.
    """
    M, N = lin.shape
    x = lin.float().clone().view(M, 3, N // 3 // HEAD_DIM, HEAD_DIM)
    sc = rot.float().reshape(M, 1, HEAD_DIM // 2, 2)
    sin, cos = sc[..., 0], sc[..., 1]
    for part, w in ((0, norm_q), (1, norm_k)):
        h = x[:, part]
        h = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * w.float()
        xe, xo = h[..., 0::2], h[..., 1::2]
        x[:, part] = torch.stack([xe * cos - xo * sin, xe * sin + xo * cos], -1).flatten(-2)
    return x.view(M, N)


def _requant(v: torch.Tensor, unsigned: bool):
    M, N = v.shape
    vg = v.view(M, N // 64, 64)
    if unsigned:
        scale = vg.amax(-1).clamp_min(0) / 15
    else:
        scale = vg.abs().amax(-1) / 7
    # the kernels multiply by the reciprocal of the unrounded scale (gemm_w4a4.py:771)
    q = vg * (1.0 / torch.where(scale == 0, torch.ones_like(scale), scale))[..., None]
    r = torch.round(q)
    codes = (r.clamp(0, 15) if unsigned else r.clamp(-8, 7)).to(torch.int32).view(M, N)
    return codes, scale.T.contiguous()


def gelu_quant(lin: torch.Tensor, smooth, lora_down, dtype, shift: float = GELU_SHIFT):
    """
    GELU + next-layer LoRA-down + unsigned int4 quantisation of the fp32 tile ``lin`` (M, N):
    ``(codes int32 [M,N], scales fp32 [N/64, M], lora_act fp32 [M,R2] | None)``
    (kernel: nunchaku/ops/triton/gemm_w4a4.py:723-778; torch form nunchaku/ops/triton/native/w4a4.py:743-753).
    """
    x = gelu_tanh(lin)
    lora = x.to(dtype).float() @ lora_down.float() if lora_down is not None else None
    v = x + shift
    if smooth is not None:
        v = v * (1.0 / smooth.float())[None, :]
    codes, scale = _requant(v, unsigned=True)
    return codes, scale, lora


def swiglu_quant(lin: torch.Tensor, smooth, lora_down, dtype):
    """
    ``silu(gate) * up`` of ``lin = [gate | up]`` + LoRA-down + signed int4 quantisation
    (nunchaku/ops/triton/native/w4a4.py:756-766).
    """
    H = lin.shape[1] // 2
    y = silu(lin[:, :H]) * lin[:, H:].float()
    lora = y.to(dtype).float() @ lora_down.float() if lora_down is not None else None
    v = y * (1.0 / smooth.float())[None, :] if smooth is not None else y
    codes, scale = _requant(v, unsigned=False)
    return codes, scale, lora


def interleave_swiglu(n: int) -> torch.Tensor:
    """Row order ``[gate | up]`` -> 16-row blocks of (gate, up) (nunchaku/ops/triton/native/w4a4.py:349-359)."""
    h, b = n // 2, 16
    g = torch.arange(h).view(h // b, b)
    return torch.stack([g, g + h], dim=1).reshape(-1)


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    """Relative Frobenius error ``|a - b| / |b|`` in fp64."""
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))

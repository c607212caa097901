"""
CPU restatement of the AWQ W4A16 path, the attention op and the FLUX rotary table of
nunchaku-rocm (test infrastructure, not product code; only tests, the smoke check and the
benchmark's CPU-baseline leg import it).

Parity status: pinned for the AWQ packing (``tests/golden/make_golden.py`` runs the reference's
``pack_w4`` of nunchaku/models/text_encoders/tinychat_utils.py:76-106, which loads standalone on a
CPU); the GEMV/attention arithmetic exists in the reference only as Triton kernels and is pinned
through the reference tests' own definitions (tests/triton/test_gemm.py:128-159,
tests/triton/test_w4a4.py:241-254).
"""

from __future__ import annotations

import math

import torch


# ----------------------------------------------------------------------------------------------
# AWQ W4A16 (A.6)
# ----------------------------------------------------------------------------------------------
def awq_pack(q: torch.Tensor) -> torch.Tensor:
    """
    Logical uint4 ``q[n, k]`` (int32, values 0..15) -> TinyChat int16 ``[n/4, k]``, returned viewed as
    int32 ``[n/4, k/2]`` like ``AWQW4A16Linear.qweight`` (layout: nunchaku/ops/triton/awq.py:8-18).
    Written from the element formula, not from the reference's view/permute chain:
    nibble ``(n, k)`` sits in ``B[n // 4, e]`` at bit ``4 * ((k % 32) // 8)`` with
    ``t = (k // 32) * 8 + k % 8``, ``e = (t // 16) * 64 + (n % 4) * 16 + t % 16`` (awq.py:28-46).
    """
    n, k = q.shape
    nn_, kk = torch.meshgrid(torch.arange(n), torch.arange(k), indexing="ij")
    t = (kk // 32) * 8 + kk % 8
    e = (t // 16) * 64 + (nn_ % 4) * 16 + t % 16
    sh = 4 * ((kk % 32) // 8)
    flat = torch.zeros(n // 4 * k, dtype=torch.int32)
    flat.index_add_(0, ((nn_ // 4) * k + e).reshape(-1), (q.to(torch.int32) << sh.to(torch.int32)).reshape(-1))
    b16 = flat.view(n // 4, k)
    b16 = torch.where(b16 >= 32768, b16 - 65536, b16).to(torch.int16)
    return b16.view(torch.int32)


def awq_unpack(kernel: torch.Tensor, n: int, k: int) -> torch.Tensor:
    """Inverse of :func:`awq_pack`: int32 ``[n/4, k/2]`` -> uint4 codes ``[n, k]`` int32."""
    b = kernel.view(torch.int16).to(torch.int32) & 0xFFFF
    nn_, kk = torch.meshgrid(torch.arange(n), torch.arange(k), indexing="ij")
    t = (kk // 32) * 8 + kk % 8
    e = (t // 16) * 64 + (nn_ % 4) * 16 + t % 16
    sh = 4 * ((kk % 32) // 8)
    return (b[nn_ // 4, e] >> sh) & 0xF


def awq_dequant(kernel, scales, zeros, n: int, k: int, group: int = 64) -> torch.Tensor:
    """``W[n,k] = q[n,k] * s[k/g, n] + z[k/g, n]`` in fp32 (nunchaku/ops/triton/awq.py:49-80)."""
    q = awq_unpack(kernel, n, k).float()
    grp = torch.arange(k) // group
    return q * scales.float()[grp].t() + zeros.float()[grp].t()


def awq_gemv(x, kernel, scales, zeros, n: int, k: int, group: int = 64) -> torch.Tensor:
    """
    ``out[row, n] = sum_c ( s[c,n] * sum_{k in c} x[k] q[n,k] + z[c,n] * sum_{k in c} x[k] )`` in fp32
    (nunchaku/ops/triton/awq.py:121-183); the caller rounds to the 16-bit dtype.
    """
    xf = x.reshape(-1, k).float()
    q = awq_unpack(kernel, n, k).float()
    out = torch.zeros(xf.shape[0], n)
    for c in range(k // group):
        sl = slice(c * group, (c + 1) * group)
        out += (xf[:, sl] @ q[:, sl].T) * scales[c].float()[None, :] + xf[:, sl].sum(1, keepdim=True) * zeros[
            c
        ].float()[None, :]
    return out


# ----------------------------------------------------------------------------------------------
# attention (A.7)
# ----------------------------------------------------------------------------------------------
def attention(q, k, v, scale: float | None = None) -> torch.Tensor:
    """
    Unmasked attention on ``(B, H, T, D)`` -> ``(B, Tq, H * D)`` fp32, with the kernel's rounding
    points (nunchaku/ops/triton/attention.py:61-117): ``q * scale * log2(e)`` is rounded to the
    input dtype, the probabilities are rounded to the input dtype before ``P @ V``.
    """
    B, H, Tq, D = q.shape
    T = q.dtype
    if scale is None:
        scale = D**-0.5
    qs = (q.float() * (scale * 1.4426950408889634)).to(T).float()
    s = qs @ k.float().transpose(-1, -2)
    m = s.amax(-1, keepdim=True)
    p = torch.exp2(s - m)
    l = p.sum(-1, keepdim=True)
    o = (p.to(T).float() @ v.float()) / l
    return o.transpose(1, 2).reshape(B, Tq, H * D)


def attention_exact(q, k, v, scale: float | None = None) -> torch.Tensor:
    """fp32 softmax attention without the kernel's roundings (tests/triton/test_w4a4.py:252-254)."""
    B, H, Tq, D = q.shape
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), scale=scale)
    return ref.transpose(1, 2).reshape(B, Tq, H * D)


# ----------------------------------------------------------------------------------------------
# FLUX rotary table
# ----------------------------------------------------------------------------------------------
def rope(pos: torch.Tensor, dim: int, theta: int = 10000) -> torch.Tensor:
    """``(B, S)`` positions -> ``(B, S, dim/2, 1, 2)`` fp32 of (sin, cos) (nunchaku/models/embeddings.py:11-50)."""
    scale = torch.arange(0, dim, 2, dtype=torch.float64) / dim
    omega = 1.0 / (theta**scale)
    out = pos.double()[..., None] * omega
    return torch.stack([torch.sin(out), torch.cos(out)], dim=-1).view(pos.shape[0], -1, dim // 2, 1, 2).float()


def flux_rotary_table(txt_tokens: int = 512, height: int = 64, width: int = 64, axes=(16, 56, 56)) -> torch.Tensor:
    """
    The ``(S, 64, 1, 2)`` fp32 table FLUX feeds the fused QKV epilogue for ``txt_tokens`` text rows
    (ids 0,0,0) followed by a ``height x width`` grid (ids 0,y,x): per-axis :func:`rope` concatenated
    along the pair dimension (nunchaku/models/embeddings.py:74-97, axes and theta from
    nunchaku/models/transformers/transformer_flux_v2.py:366).
    """
    ids = torch.zeros(txt_tokens + height * width, 3)
    yy, xx = torch.meshgrid(torch.arange(height), torch.arange(width), indexing="ij")
    ids[txt_tokens:, 1] = yy.reshape(-1)
    ids[txt_tokens:, 2] = xx.reshape(-1)
    parts = [rope(ids[None, :, i], axes[i]) for i in range(3)]
    return torch.cat(parts, dim=2)[0].contiguous()


def log2e() -> float:
    return math.log2(math.e)

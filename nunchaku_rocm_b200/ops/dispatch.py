"""
Operator wrappers with the names and signatures of nunchaku/ops/dispatch.py:19-99.  There is a single
set of kernels behind them, so nothing is dispatched; the module keeps the call sites' import path.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .triton.attention import attention_fp16 as _attn
from .triton.awq import awq_gemm_w4a16, awq_gemv_w4a16

__all__ = ["gemm_awq", "gemv_awq", "attention_fp16", "scaled_dot_product_attention"]


def gemv_awq(in_feats, kernel, scaling_factors, zeros, m: int, n: int, k: int, group_size: int) -> torch.Tensor:
    """AWQ W4A16 GEMV. See :func:`nunchaku_rocm_b200.ops.gemv.awq_gemv_w4a16_cuda`."""
    return awq_gemv_w4a16(in_feats, kernel, scaling_factors, zeros, m, n, k, group_size)


def gemm_awq(in_feats, kernel, scaling_factors, zeros) -> torch.Tensor:
    """AWQ W4A16 GEMM."""
    return awq_gemm_w4a16(in_feats, kernel, scaling_factors, zeros)


def attention_fp16(q, k, v, o, scale: float) -> None:
    """Unmasked attention, fp32 accumulation, written into ``o``."""
    _attn(q, k, v, o, scale)


def scaled_dot_product_attention(query, key, value, attn_mask: torch.Tensor | None = None) -> torch.Tensor:
    """
    Drop-in for ``F.scaled_dot_product_attention`` on ``(B, H, T, D)`` inputs (no dropout, not causal).
    Unmasked 16-bit attention with a head dimension of 64 or 128 and unit last stride runs on the CUDA kernel
    of this package; anything else (a mask, fp32, another head dimension) goes to torch, as in the reference
    (nunchaku/ops/dispatch.py:67-99).
    """
    head_dim = query.shape[-1]
    if (
        attn_mask is not None
        or query.device.type != "cuda"
        or query.dtype not in (torch.float16, torch.bfloat16)
        or not (key.dtype == value.dtype == query.dtype)
        or head_dim not in (64, 128)
        or any(t.stride(-1) != 1 for t in (query, key, value))
        or any(s % 8 for t in (query, key, value) for s in t.stride()[:-1])
        or any(t.data_ptr() % 16 for t in (query, key, value))
    ):
        return F.scaled_dot_product_attention(query, key, value, attn_mask=attn_mask, dropout_p=0.0, is_causal=False)
    batch_size, heads, tokens, _ = query.shape
    out = torch.empty(batch_size, tokens, heads * head_dim, dtype=query.dtype, device=query.device)
    _attn(query, key, value, out, head_dim**-0.5)
    return out.view(batch_size, tokens, heads, head_dim).transpose(1, 2)

"""AWQ W4A16 GEMV op with the signature of nunchaku/ops/gemv.py:10-56."""

from __future__ import annotations

import torch

from .dispatch import gemv_awq as _gemv_awq


def awq_gemv_w4a16_cuda(
    in_feats: torch.Tensor,
    kernel: torch.Tensor,
    scaling_factors: torch.Tensor,
    zeros: torch.Tensor,
    m: int,
    n: int,
    k: int,
    group_size: int = 64,
) -> torch.Tensor:
    """
    ``out (m, n) = in_feats (m, k) @ W^T`` with ``W[n, k] = q[n, k] * scaling_factors[k // group, n] + zeros[k // group, n]``,
    ``kernel`` the TinyChat-packed ``(n // 4, k // 2)`` int32 weight.
    """
    return _gemv_awq(in_feats, kernel, scaling_factors, zeros, m, n, k, group_size)

"""Host helpers the reference exposes from ``nunchaku.ops.triton.native.w4a4`` that callers outside the kernels use."""

from __future__ import annotations

import torch

SWIGLU_BLOCK = 16
HEAD_DIM = 128
GELU_SHIFT = 0.171875


def interleave_swiglu(n: int, device=None) -> torch.Tensor:
    """
    Row order the SwiGLU epilogue reads for a projection whose output is ``[gate (n/2) | up (n/2)]``: blocks of 16
    gate rows followed by the matching 16 up rows (nunchaku/ops/triton/native/w4a4.py:349-359).
    ``weight[idx]`` applies it; ``out.view(M, n // 32, 2, 16)`` splits an output back into gate and up.
    """
    h, b = n // 2, SWIGLU_BLOCK
    g = torch.arange(h, device=device).view(h // b, b)
    return torch.stack([g, g + h], dim=1).reshape(-1)

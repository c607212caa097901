"""
Rotary table in the natural layout the fused QKV epilogue reads: ``(rows, head_dim / 2, 1, 2)`` fp32
with ``(sin, cos)`` last (the reference's ``rope`` / ``NunchakuFluxPosEmbed``,
nunchaku/models/embeddings.py:11-50, 74-97).
"""

from __future__ import annotations

import torch


def rope(pos: torch.Tensor, dim: int, theta: int) -> torch.Tensor:
    """``pos (B, S)`` -> ``(B, S, dim // 2, 1, 2)`` fp32; angles computed in fp64."""
    assert dim % 2 == 0, "The dimension must be even."
    scale = torch.arange(0, dim, 2, dtype=torch.float64, device=pos.device) / dim
    omega = 1.0 / (theta**scale)
    out = pos.to(torch.float64)[..., None] * omega
    stacked = torch.stack([torch.sin(out), torch.cos(out)], dim=-1)
    return stacked.view(pos.shape[0], -1, dim // 2, 1, 2).float()


def flux_pos_embed(ids: torch.Tensor, axes_dim=(16, 56, 56), theta: int = 10000) -> torch.Tensor:
    """``ids (S, 3)`` -> ``(S, sum(axes_dim) / 2, 1, 2)``: one :func:`rope` per axis, concatenated along the pairs."""
    parts = [rope(ids[None, :, i], axes_dim[i], theta) for i in range(ids.shape[-1])]
    return torch.cat(parts, dim=2)[0].contiguous()


def flux_image_ids(txt_tokens: int, height: int, width: int, device=None) -> torch.Tensor:
    """Position ids of ``txt_tokens`` text rows (0, 0, 0) followed by a ``height x width`` latent grid (0, y, x)."""
    ids = torch.zeros(txt_tokens + height * width, 3, device=device)
    yy, xx = torch.meshgrid(torch.arange(height, device=device), torch.arange(width, device=device), indexing="ij")
    ids[txt_tokens:, 1] = yy.reshape(-1)
    ids[txt_tokens:, 2] = xx.reshape(-1)
    return ids

"""Activation quantizer op with the signature of nunchaku/ops/quantize.py:11-88."""

from __future__ import annotations

import torch

from .triton.gemm_w4a4 import quantize_w4a4_act_fuse_lora as _quantize


def ceil_divide(a: int, b: int) -> int:
    return (a + b - 1) // b


def svdq_quantize_w4a4_act_fuse_lora_cuda(
    input: torch.Tensor,
    output: torch.Tensor | None = None,
    oscales: torch.Tensor | None = None,
    lora_down: torch.Tensor | None = None,
    lora_act_out: torch.Tensor | None = None,
    smooth: torch.Tensor | None = None,
    fuse_glu: bool = False,
    fp4: bool = False,
    pad_size: int = 256,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """
    Quantize ``input (M, K)`` to packed 4-bit rows and compute the LoRA-down hidden state.

    Outputs are padded to ``M_pad = ceil(M / pad_size) * pad_size`` rows when allocated here:
    ``output (M_pad, K // 2)`` uint8, ``oscales (K // G, M_pad)`` (input dtype, or float8_e4m3fn for NVFP4),
    ``lora_act_out (M_pad, R)`` fp32.  Rows ``>= M`` are left uninitialised, as in the reference
    (nunchaku/ops/quantize.py:65-78).
    """
    batch_size, channels = input.shape
    rank = lora_down.shape[1]
    batch_size_pad = ceil_divide(batch_size, pad_size) * pad_size
    if output is None:
        output = torch.empty(batch_size_pad, channels // 2, dtype=torch.uint8, device=input.device)
    if oscales is None:
        if fp4:
            assert channels % 16 == 0
            oscales = torch.empty(channels // 16, batch_size_pad, dtype=torch.float8_e4m3fn, device=input.device)
        else:
            assert channels % 64 == 0
            oscales = torch.empty(channels // 64, batch_size_pad, dtype=input.dtype, device=input.device)
    if lora_act_out is None:
        lora_act_out = torch.empty(batch_size_pad, rank, dtype=torch.float32, device=input.device)
    _quantize(input, output, oscales, lora_down, lora_act_out, smooth, fuse_glu, fp4)
    return output, oscales, lora_act_out

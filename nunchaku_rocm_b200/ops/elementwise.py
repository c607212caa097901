"""
The element-wise steps around the quantised linears of a DiT block, fused to one pass over HBM each
(``csrc/elementwise.cu``).  The reference runs them as torch operators: ``NunchakuAdaLayerNormZero``
(nunchaku/models/normalization.py:60-159) and the gated residuals of the transformer blocks
(nunchaku/models/transformers/transformer_flux_v2.py:174-343).
"""

from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L

__all__ = ["layernorm_modulate", "gated_residual"]


def _bind():
    lib = L.lib()
    if not getattr(lib, "_ew_bound", False):
        lib.nb_layernorm_modulate.argtypes = [C.c_void_p] * 4 + [C.c_int32] * 3 + [C.c_int64] * 4 + [C.c_float, C.c_float, C.c_int32, C.c_void_p]
        lib.nb_gated_residual.argtypes = [C.c_void_p] * 5 + [C.c_int32] * 3 + [C.c_int64] * 6 + [C.c_int32, C.c_void_p]
        lib._ew_bound = True
    return lib


def _rows(x: torch.Tensor) -> torch.Tensor:
    """``(B, T, dim)`` as a view whose rows are evenly strided (a copy only if they are not)."""
    B, T, D = x.shape
    if x.stride(2) != 1 or (B > 1 and x.stride(0) != T * x.stride(1)) or x.stride(1) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    return x


def layernorm_modulate(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, scale_add: float = 0.0,
                       eps: float = 1e-6) -> torch.Tensor:
    """``LayerNorm(x) * (scale[:, None] + scale_add) + shift[:, None]`` for ``x (B, T, dim)``, ``scale / shift (B, dim)``
    (any strides), no affine; rounded to the dtype where ``layer_norm``, ``+``, ``*``, ``+`` of the reference round."""
    B, T, D = x.shape
    if D % 1024 or D > 4096:
        return torch.nn.functional.layer_norm(x, (D,), eps=eps) * (scale + scale_add)[:, None] + shift[:, None]
    dev = L.require_cuda(x, scale, shift)
    x = _rows(x)
    assert scale.shape == (B, D) and shift.shape == (B, D) and scale.stride() == shift.stride() and scale.dtype == x.dtype == shift.dtype
    out = torch.empty(B, T, D, dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        L.check(
            _bind().nb_layernorm_modulate(L.ptr(x), L.ptr(scale), L.ptr(shift), L.ptr(out), B * T, T, D, x.stride(1), D,
                                          scale.stride(0), scale.stride(1), float(scale_add), float(eps), L.DTYPE_CODE[x.dtype],
                                          L.stream_of(out)),
            "layernorm_modulate",
        )
    return out


def gated_residual(x: torch.Tensor, gate: torch.Tensor, y: torch.Tensor, y2: torch.Tensor | None = None) -> torch.Tensor:
    """``x + gate[:, None] * (y [+ y2])`` for ``x, y, y2 (B, T, dim)``, ``gate (B, dim)`` (any strides); rounded to the dtype where the reference's ``+``, ``*``, ``+`` round."""
    B, T, D = x.shape
    dev = L.require_cuda(x, gate, y)
    assert D % 8 == 0 and y.shape == x.shape and gate.shape == (B, D) and gate.dtype == x.dtype == y.dtype
    x, y = _rows(x), _rows(y)
    if y2 is not None:
        assert y2.shape == x.shape and y2.dtype == x.dtype
        y2 = _rows(y2)
    out = torch.empty(B, T, D, dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        L.check(
            _bind().nb_gated_residual(L.ptr(x), L.ptr(gate), L.ptr(y), L.ptr(y2) if y2 is not None else None, L.ptr(out), B * T, T,
                                      D, x.stride(1), y.stride(1), y2.stride(1) if y2 is not None else 0, D, gate.stride(0),
                                      gate.stride(1), L.DTYPE_CODE[x.dtype], L.stream_of(out)),
            "gated_residual",
        )
    return out

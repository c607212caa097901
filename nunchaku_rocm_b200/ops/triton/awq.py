"""
AWQ W4A16 operators with the signatures of ``nunchaku.ops.triton.awq`` (nunchaku/ops/triton/awq.py:83-251).
``kernel`` is the TinyChat packing ``[n // 4, k // 2]`` int32 (viewed int16 ``[n // 4, k]``).
"""

from __future__ import annotations

import ctypes as C

import torch

from ... import _lib as L

__all__ = ["awq_dequantize", "awq_gemv_w4a16", "awq_gemm_w4a16"]


def _bind():
    lib = L.lib()
    if not getattr(lib, "_awq_bound", False):
        lib.nb_awq_gemv.argtypes = [C.c_void_p] * 5 + [C.c_int32] * 3 + [C.c_int64] * 4 + [C.c_int32, C.c_void_p]
        lib.nb_awq_dequant.argtypes = [C.c_void_p] * 4 + [C.c_int32] * 3 + [C.c_int64] * 3 + [C.c_int32, C.c_void_p]
        lib.nb_awq_gemm.argtypes = [C.c_void_p] * 5 + [C.c_int32] * 4 + [C.c_int64] * 4 + [C.c_int32, C.c_void_p]
        lib._awq_bound = True
    return lib


def awq_dequantize(kernel, scaling_factors, zeros, n: int, k: int, group_size: int, dtype: torch.dtype) -> torch.Tensor:
    """Unpack an AWQ W4 weight to dense ``[n, k]``: ``q * s + z`` (nunchaku/ops/triton/awq.py:83-118)."""
    dev = L.require_cuda(kernel, scaling_factors, zeros)
    packed = kernel.view(torch.int16)
    assert packed.shape == (n // 4, k), f"unexpected packed AWQ weight shape {tuple(packed.shape)}"
    assert scaling_factors.dtype == dtype and zeros.dtype == dtype
    assert scaling_factors.stride(1) == 1 and zeros.stride() == scaling_factors.stride() and packed.stride(1) == 1
    out = torch.empty(n, k, dtype=dtype, device=dev)
    with torch.cuda.device(dev):
        L.check(
            _bind().nb_awq_dequant(L.ptr(packed), L.ptr(scaling_factors), L.ptr(zeros), L.ptr(out), n, k, group_size,
                                   packed.stride(0), scaling_factors.stride(0), out.stride(0), L.DTYPE_CODE[dtype],
                                   L.stream_of(out)),
            "awq_dequantize",
        )
    return out


def awq_gemv_w4a16(in_feats, kernel, scaling_factors, zeros, m: int, n: int, k: int, group_size: int = 64) -> torch.Tensor:
    """
    AWQ W4A16 GEMV for small batches; same contract as the reference (nunchaku/ops/triton/awq.py:186-229):
    group 64 streams the packed weight once, other group sizes dequantise and multiply.
    """
    x = in_feats.reshape(m, k)
    if group_size == 64 and k % 64 == 0 and n % 4 == 0 and k * 32 <= 200 * 1024:
        dev = L.require_cuda(x, kernel, scaling_factors, zeros)
        x = x.contiguous()
        packed = kernel.view(torch.int16)
        assert packed.shape == (n // 4, k), f"unexpected packed AWQ weight shape {tuple(packed.shape)}"
        assert scaling_factors.stride(1) == 1 and zeros.stride() == scaling_factors.stride()
        assert scaling_factors.dtype == x.dtype and zeros.dtype == x.dtype
        out = torch.empty(m, n, dtype=x.dtype, device=dev)
        with torch.cuda.device(dev):
            L.check(
                _bind().nb_awq_gemv(L.ptr(x), L.ptr(packed), L.ptr(scaling_factors), L.ptr(zeros), L.ptr(out), m, n, k,
                                    x.stride(0), packed.stride(0), scaling_factors.stride(0), out.stride(0),
                                    L.DTYPE_CODE[x.dtype], L.stream_of(out)),
                "awq_gemv_w4a16",
            )
        return out.reshape(*in_feats.shape[:-1], n)
    return awq_gemm_w4a16(in_feats, kernel, scaling_factors, zeros, group_size)


def _gemm_kernel_takes(x: torch.Tensor, n: int, k: int, group_size: int) -> bool:
    return (k % 64 == 0 and n % 4 == 0 and group_size % 32 == 0 and k % group_size == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)


def awq_gemm_w4a16(in_feats, kernel, scaling_factors, zeros, group_size: int = 128) -> torch.Tensor:
    """
    AWQ W4A16 GEMM (nunchaku/ops/triton/awq.py:232-251: dequantise, then a dense matmul).  One kernel here
    (``awq_gemm_kernel``: the weight tile is widened to ``q * s + z`` in the 16-bit dtype in shared memory and multiplied
    on the tensor cores with fp32 accumulation); shapes it does not take (k % 64, group % 32, unaligned rows) go through
    :func:`awq_dequantize` and ``torch.matmul``.
    """
    shape = in_feats.shape
    k = shape[-1]
    x = in_feats.reshape(-1, k)
    n = scaling_factors.shape[-1]
    if not _gemm_kernel_takes(x, n, k, group_size):
        x = x.contiguous()
    if _gemm_kernel_takes(x, n, k, group_size):
        dev = L.require_cuda(x, kernel, scaling_factors, zeros)
        packed = kernel.view(torch.int16)
        assert packed.shape == (n // 4, k), f"unexpected packed AWQ weight shape {tuple(packed.shape)}"
        assert scaling_factors.dtype == x.dtype and zeros.dtype == x.dtype
        assert scaling_factors.stride(1) == 1 and zeros.stride() == scaling_factors.stride() and packed.stride(1) == 1
        out = torch.empty(x.shape[0], n, dtype=x.dtype, device=dev)
        with torch.cuda.device(dev):
            L.check(
                _bind().nb_awq_gemm(L.ptr(x), L.ptr(packed), L.ptr(scaling_factors), L.ptr(zeros), L.ptr(out), x.shape[0], n, k,
                                    group_size, x.stride(0), packed.stride(0), scaling_factors.stride(0), out.stride(0),
                                    L.DTYPE_CODE[x.dtype], L.stream_of(out)),
                "awq_gemm_w4a16",
            )
        return out.reshape(*shape[:-1], n)
    w = awq_dequantize(kernel, scaling_factors, zeros, n, k, group_size, x.dtype)
    return torch.matmul(x, w.t()).reshape(*shape[:-1], n)

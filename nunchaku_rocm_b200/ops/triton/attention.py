"""Unmasked flash attention with the signature of ``nunchaku.ops.triton.attention`` (attention.py:120-169)."""

from __future__ import annotations

import ctypes as C

import torch

from ... import _lib as L

__all__ = ["attention_fp16"]


def attention_fp16(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, scale: float,
                   _impl: int = L.IMPL_AUTO) -> None:
    """
    ``o[b, t, h * D:(h + 1) * D] = softmax(q k^T * scale) v`` for ``q (B, H, Tq, D)``, ``k, v (B, H, Tkv, D)``,
    written in place into ``o (B, Tq, H * D)``.  Inputs may be strided views with unit last stride.  ``_impl`` selects
    the kernel (tests only): head dimension 128 runs on the tcgen05 kernel, the rest on the mma.sync kernel.
    """
    B, H, Tq, D = q.shape
    Tkv = k.shape[2]
    assert k.shape[3] == D and v.shape[3] == D
    assert o.shape == (B, Tq, H * D), f"unexpected output shape {tuple(o.shape)}"
    dev = L.require_cuda(q, k, v, o)
    if q.dtype not in L.DTYPE_CODE or not (k.dtype == v.dtype == o.dtype == q.dtype):
        raise NotImplementedError("attention_fp16 takes float16 or bfloat16 tensors of one dtype")
    if any(t.stride(-1) != 1 for t in (q, k, v, o)):
        raise ValueError("q, k, v, o need unit stride in the last dimension")
    lib = L.lib()
    a = L.AttnArgs()
    a.q, a.k, a.v, a.o = L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o)
    a.B, a.H, a.Tq, a.Tkv, a.D, a.dtype = B, H, Tq, Tkv, D, L.DTYPE_CODE[q.dtype]
    a.scale = float(scale)
    a.stride_qb, a.stride_qh, a.stride_qm = q.stride(0), q.stride(1), q.stride(2)
    a.stride_kb, a.stride_kh, a.stride_kn = k.stride(0), k.stride(1), k.stride(2)
    a.stride_vb, a.stride_vh, a.stride_vn = v.stride(0), v.stride(1), v.stride(2)
    a.stride_ob, a.stride_om = o.stride(0), o.stride(1)
    a.impl = _impl
    a.status = L.ptr(L.status_word(dev))
    need = lib.nb_attention_scratch_bytes(C.byref(a))
    scratch = None
    if need > 0:
        scratch = torch.empty(need, dtype=torch.uint8, device=dev)
        a.scratch, a.scratch_bytes = L.ptr(scratch), need
    with torch.cuda.device(dev):
        L.check(lib.nb_attention(C.byref(a), L.stream_of(q)), "attention_fp16")

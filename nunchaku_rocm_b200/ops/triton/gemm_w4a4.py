"""
W4A4 GEMM and activation quantizer: the kernel-level entry points the reference's models and tests
import from ``nunchaku.ops.triton.gemm_w4a4`` (same names, arguments and error behaviour), here
launching the sm_100a CUDA kernels of ``libnunchaku_b200.so``.  The module path keeps the
reference's name only so that imports written against it resolve; nothing here uses Triton and
there is no other backend to fall back to.

Layouts are the natural ones of nunchaku/ops/triton/gemm_w4a4.py:4-19: ``act`` ``[M, K//2]`` uint8
(element ``k`` = low nibble of byte ``k//2`` for even ``k``), ``wgt`` ``[N, K//2]``, scales
``[K//group, rows]``, ``rotary_emb`` ``[rows, 64, 1, 2]`` fp32 of (sin, cos).
"""

from __future__ import annotations

import collections
import ctypes as C
import os
import threading

import torch

from ... import _lib as L

__all__ = [
    "gemm_w4a4",
    "gemm_w4a4_group_sums",
    "quantize_w4a4_act",
    "quantize_w4a4_act_fuse_lora",
    "quantize_w4a4_wgt",
]

HEAD_DIM = 128
GELU_SHIFT = 0.171875


def _dtype_code(dt: torch.dtype) -> int:
    try:
        return L.DTYPE_CODE[dt]
    except KeyError:
        raise NotImplementedError(f"16-bit dtype must be bfloat16 or float16, got {dt}") from None


# ------------------------------------------------------------------------------------------------
# quantizer
# ------------------------------------------------------------------------------------------------
def _launch_quantize(
    input: torch.Tensor,
    output: torch.Tensor,
    oscales: torch.Tensor,
    lora_down: torch.Tensor | None,
    lora_act_out: torch.Tensor | None,
    smooth: torch.Tensor | None,
    fuse_glu: bool,
    fp4: bool,
    fuse_gelu: bool = False,
    shift_value: float = 0.0,
    unsigned: bool = False,
) -> None:
    """Argument handling of the reference's ``_launch_quantize`` (nunchaku/ops/triton/gemm_w4a4.py:1465-1518)."""
    input = input.reshape(-1, input.shape[-1])
    M = input.shape[0]
    K = input.shape[1] // 2 if fuse_glu else input.shape[1]
    group = 16 if fp4 else 64
    assert K % group == 0, f"K={K} must be a multiple of the group size {group}"
    if K % 64:
        raise NotImplementedError(f"K={K}: the quantizer works on 64-column blocks")
    dev = L.require_cuda(input, output, oscales, lora_down, lora_act_out, smooth)
    if input.stride(-1) != 1:
        input = input.contiguous()
    has_lora = lora_down is not None and lora_act_out is not None
    if has_lora and lora_down.stride(-1) != 1:
        lora_down = lora_down.contiguous()
    if smooth is not None:
        smooth = smooth.contiguous()
    assert output.stride(-1) == 1 and oscales.stride(-1) == 1
    a = L.QuantArgs()
    a.input, a.output, a.oscales = L.ptr(input), L.ptr(output), L.ptr(oscales)
    a.lora_down, a.lora_act_out = (L.ptr(lora_down), L.ptr(lora_act_out)) if has_lora else (None, None)
    a.smooth = L.ptr(smooth)
    a.M, a.K, a.R = M, K, lora_down.shape[1] if has_lora else 0
    a.dtype = _dtype_code(input.dtype)
    a.fuse_glu, a.fuse_gelu, a.fp4, a.is_unsigned = int(fuse_glu), int(fuse_gelu), int(fp4), int(unsigned)
    a.shift = float(shift_value)
    a.stride_im, a.stride_om, a.stride_sg = input.stride(0), output.stride(0), oscales.stride(0)
    a.stride_ld = lora_down.stride(0) if has_lora else 0
    a.stride_lam = lora_act_out.stride(0) if has_lora else 0
    with torch.cuda.device(dev):
        L.check(L.lib().nb_quantize_w4a4(C.byref(a), L.stream_of(input)), "quantize_w4a4")


def quantize_w4a4_act_fuse_lora(
    input: torch.Tensor,
    output: torch.Tensor | None = None,
    oscales: torch.Tensor | None = None,
    lora_down: torch.Tensor | None = None,
    lora_act_out: torch.Tensor | None = None,
    smooth: torch.Tensor | None = None,
    fuse_glu: bool = False,
    fp4: bool = False,
    fuse_gelu: bool = False,
    shift_value: float = 0.0,
    unsigned: bool = False,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """
    Quantize activations to 4 bits and compute the LoRA down-projection; signature and allocation
    rules of nunchaku/ops/triton/gemm_w4a4.py:1521-1565.  Returns ``(output, oscales, lora_act_out)``.
    """
    inp = input.reshape(-1, input.shape[-1])
    M = inp.shape[0]
    K = inp.shape[1] // 2 if fuse_glu else inp.shape[1]
    group = 16 if fp4 else 64
    if output is None:
        output = torch.empty(M, K // 2, dtype=torch.uint8, device=input.device)
    if oscales is None:
        sdtype = torch.float8_e4m3fn if fp4 else input.dtype
        oscales = torch.empty(K // group, M, dtype=sdtype, device=input.device)
    if lora_act_out is None and lora_down is not None:
        lora_act_out = torch.empty(M, lora_down.shape[1], dtype=torch.float32, device=input.device)
    _launch_quantize(
        inp, output, oscales, lora_down, lora_act_out, smooth, fuse_glu, fp4, fuse_gelu, shift_value, unsigned
    )
    return output, oscales, lora_act_out


def quantize_w4a4_act(input, output=None, oscales=None, fp4: bool = False):
    """Per-group symmetric 4-bit activation quantisation (nunchaku/ops/triton/gemm_w4a4.py:1568-1576)."""
    out, scales, _ = quantize_w4a4_act_fuse_lora(input, output, oscales, fp4=fp4)
    return out, scales


def quantize_w4a4_wgt(input, output=None, oscales=None, fp4: bool = False):
    """Same maths applied to a weight matrix (nunchaku/ops/triton/gemm_w4a4.py:1579-1592)."""
    out, scales, _ = quantize_w4a4_act_fuse_lora(input, output, oscales, fp4=fp4)
    return out, scales


# ------------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------------
def _apply_rmsnorm_rope_qk(out, norm_q, norm_k, rotary_emb, epsilon: float = 1e-6) -> None:
    """In-place per-head RMSNorm + RoPE on the Q/K thirds of a stored tile (gemm_w4a4.py:834-866)."""
    M, N = out.shape
    third = N // 3
    assert third % HEAD_DIM == 0, f"Q/K/V third ({third}) must be a multiple of HEAD_DIM ({HEAD_DIM})"
    dev = L.require_cuda(out, norm_q, norm_k, rotary_emb)
    rot = rotary_emb.reshape(-1, HEAD_DIM)
    assert rot.dtype == torch.float32 and rot.stride(1) == 1 and M % rot.shape[0] == 0
    q = L.QKArgs(L.ptr(norm_q.contiguous()), L.ptr(norm_k.contiguous()), L.ptr(rot), rot.stride(0), rot.shape[0], epsilon)
    with torch.cuda.device(dev):
        L.check(
            L.lib().nb_qk_norm_rope(L.ptr(out), M, N, out.stride(0), _dtype_code(out.dtype), C.byref(q), L.stream_of(out)),
            "qk_norm_rope",
        )


def _gemm_args(act, wgt, out2d, ascales, wscales, bias, lora_act_in, lora_up, wcscales, act_unsigned, fuse_silu, fp4,
               alpha, dtype, impl):
    M, K, N = act.shape[0], act.shape[1] * 2, wgt.shape[0]
    has_lora = lora_act_in is not None and lora_up is not None and lora_up.shape[1] > 0
    a = L.GemmArgs()
    a.act, a.wgt, a.out = L.ptr(act), L.ptr(wgt), L.ptr(out2d)
    a.ascales, a.wscales, a.bias = L.ptr(ascales), L.ptr(wscales), L.ptr(bias)
    a.lora_act, a.lora_up = (L.ptr(lora_act_in), L.ptr(lora_up)) if has_lora else (None, None)
    a.wcscales = L.ptr(wcscales)
    a.M, a.N, a.K = M, N, K
    a.actual_m = out2d.shape[0] if out2d is not None else M
    a.R = lora_up.shape[1] if has_lora else 0
    a.dtype = _dtype_code(dtype)
    a.act_unsigned, a.fp4, a.fuse_silu, a.impl = int(act_unsigned), int(fp4), int(fuse_silu), impl
    a.alpha = 1.0 if alpha is None else float(alpha)
    a.stride_am, a.stride_wn = act.stride(0), wgt.stride(0)
    a.stride_asg, a.stride_wsg = ascales.stride(0), wscales.stride(0)
    a.stride_om = out2d.stride(0) if out2d is not None else 0
    a.stride_lam = lora_act_in.stride(0) if has_lora else 0
    a.stride_lun = lora_up.stride(0) if has_lora else 0
    a.status = L.ptr(L.status_word(act.device))
    return a


def _checks(act, wgt, out2d, ascales, wscales, bias, lora_act_in, lora_up, wcscales, fp4, dtype):
    M, K, N = act.shape[0], act.shape[1] * 2, wgt.shape[0]
    G = K // (16 if fp4 else 64)
    sdt = torch.float8_e4m3fn if fp4 else dtype
    for name, s, rows in (("ascales", ascales, M), ("wscales", wscales, N)):
        if s.dtype != sdt:
            raise ValueError(f"{name} dtype {s.dtype} != {sdt}")
        if s.dim() != 2 or s.shape[0] < G or s.shape[1] < rows or s.stride(-1) != 1:
            raise ValueError(f"{name} shape {tuple(s.shape)} for M/N={rows}, groups={G}")
    if act.stride(-1) != 1 or wgt.stride(-1) != 1 or act.element_size() != 1 or wgt.element_size() != 1:
        raise ValueError("act/wgt must be packed byte tensors with unit inner stride")
    if out2d is not None and (out2d.stride(-1) != 1 or out2d.shape[1] != N or out2d.dtype != dtype):
        raise ValueError("out must be row-major (rows, N) of the output dtype")
    if bias is not None and (bias.dtype != dtype or bias.numel() < N or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous (N,) tensor of the output dtype")
    if wcscales is not None and (wcscales.dtype != dtype or wcscales.numel() < N or not wcscales.is_contiguous()):
        raise ValueError("wcscales must be a contiguous (N,) tensor of the output dtype")
    if (lora_act_in is None) != (lora_up is None):
        pass  # the reference treats a lone half as "no low-rank branch" (gemm_w4a4.py:1148)
    elif lora_up is not None and lora_up.shape[1]:
        R = lora_up.shape[1]
        if lora_act_in.dtype != torch.float32 or lora_up.dtype != dtype:
            raise ValueError(f"LoRA dtypes {lora_act_in.dtype}/{lora_up.dtype}")
        if lora_up.shape[0] < N or lora_act_in.shape[0] < M or lora_act_in.shape[1] < R:
            raise ValueError("LoRA shapes")
        if lora_act_in.stride(-1) != 1 or lora_up.stride(-1) != 1:
            raise ValueError("LoRA tensors need unit inner stride")


# ------------------------------------------------------------------------------------------------
# Load-time form of the weights for the int4 tensor-core kernel
# ------------------------------------------------------------------------------------------------
# A layer's weights do not change between calls, so the form the kernel's TMA loads read (one e4m3 byte per int4 value,
# column scales in the drain's order) is written once per weight and kept: the counterpart of the reference's load-time
# weight packing.  An entry keeps the weight and scale tensors alive (so their addresses cannot be handed to other
# tensors while it exists; their bytes count against the budget together with the prepared buffer) and is dropped when
# either has been modified in place (torch's version counter) or when the budget is exceeded (least recently used
# first).  NUNCHAKU_B200_PREPARED_WEIGHTS_MB=0 turns it off.
#
# CUDA graphs: a call made while the current stream is capturing bakes the buffer's address into the graph.  Such an
# entry is PINNED: it is never evicted, and if it has to be replaced (weights updated in place) the old buffer is parked
# in `_PINNED_BUFFERS`, so a replay never reads freed memory -- it reads the weights as they were at capture time.
# Re-capture after changing weights; `clear_prepared_weights(release_pinned=True)` frees everything once no graph that
# used the buffers will be replayed again.
_PREPARED: "collections.OrderedDict[tuple, list]" = collections.OrderedDict()
_PREPARED_BYTES = 0
_PINNED_BUFFERS: list = []
_PREPARED_LOCK = threading.RLock()
# entry fields
_E_WGT, _E_WVER, _E_WSC, _E_SVER, _E_BUF, _E_EVENT, _E_STREAM, _E_PINNED, _E_BYTES = range(9)


def _prepared_budget(device) -> int:
    mb = os.environ.get("NUNCHAKU_B200_PREPARED_WEIGHTS_MB")
    if mb is not None:
        return int(mb) << 20
    return torch.cuda.get_device_properties(device).total_memory // 4


def clear_prepared_weights(release_pinned: bool = False) -> None:
    """
    Drop the prepared weight buffers (and the references to the weights they were made from).  Buffers that a CUDA
    graph capture has used stay alive unless ``release_pinned`` is set: only pass it when no such graph will run again.
    """
    global _PREPARED_BYTES
    with _PREPARED_LOCK:
        for key in list(_PREPARED):
            e = _PREPARED[key]
            if e[_E_PINNED] and not release_pinned:
                _PINNED_BUFFERS.append(e[_E_BUF])
            del _PREPARED[key]
        _PREPARED_BYTES = 0
        if release_pinned:
            _PINNED_BUFFERS.clear()


def _drop_entry(key) -> None:
    global _PREPARED_BYTES
    e = _PREPARED.pop(key)
    _PREPARED_BYTES -= e[_E_BYTES]
    if e[_E_PINNED]:
        _PINNED_BUFFERS.append(e[_E_BUF])  # a captured graph may still read it


def _attach_prepared(a, wgt, wscales) -> None:
    global _PREPARED_BYTES
    budget = _prepared_budget(wgt.device)
    if budget <= 0:
        return
    try:
        wver, sver = wgt._version, wscales._version
    except RuntimeError:
        return  # inference-mode tensors carry no version counter: an in-place update could not be seen, so no cache
    capturing = torch.cuda.is_current_stream_capturing()
    key = (wgt.device.index, wgt.data_ptr(), wscales.data_ptr(), a.N, a.K, a.stride_wn, a.stride_wsg, a.dtype)
    stream = torch.cuda.current_stream(wgt.device)
    with _PREPARED_LOCK:
        e = _PREPARED.get(key)
        if e is not None and (e[_E_WVER] != wver or e[_E_SVER] != sver):
            _drop_entry(key)
            e = None
        if e is None:
            if capturing:
                return  # no allocation that outlives a graph capture: this call runs the whole pre-pass
            lib = L.lib()
            nbytes = lib.nb_gemm_w4a4_prepared_bytes(C.byref(a))
            held = nbytes + wgt.numel() * wgt.element_size() + wscales.numel() * wscales.element_size()
            if nbytes <= 0 or held > budget:
                return
            for old_key in list(_PREPARED):
                if _PREPARED_BYTES + held <= budget:
                    break
                if not _PREPARED[old_key][_E_PINNED]:
                    _drop_entry(old_key)
            if _PREPARED_BYTES + held > budget:
                return  # what is left is pinned by graph captures
            buf = torch.empty(nbytes, dtype=torch.uint8, device=wgt.device)
            with torch.cuda.device(wgt.device):
                L.check(lib.nb_gemm_w4a4_prepare_weights(C.byref(a), L.ptr(buf), nbytes, L.stream_of(wgt)), "prepare_weights")
            done = torch.cuda.Event()
            done.record(stream)
            e = [wgt, wver, wscales, sver, buf, done, stream, False, held]
            _PREPARED[key] = e
            _PREPARED_BYTES += held
        else:
            _PREPARED.move_to_end(key)
            if capturing:
                e[_E_PINNED] = True
            # Another stream must not read the buffer before the kernel that wrote it has run.  (Inside a graph capture no
            # dependency on outside work can be recorded; a capture starts after the capturing stream has joined the
            # streams whose results it uses, which covers a buffer prepared before.)
            elif e[_E_STREAM] != stream and not e[_E_EVENT].query():
                stream.wait_event(e[_E_EVENT])
        a.wgt_prepared, a.wgt_prepared_bytes = L.ptr(e[_E_BUF]), e[_E_BUF].numel()


def _run(a, epi, epi_kind, act, wgt=None, wscales=None, keep=None):
    """Launch one GEMM call.  ``keep``: tensors whose pointers sit in ``a`` / ``epi`` and that nothing else references
    (contiguous copies); holding them here keeps their memory from being handed to the scratch allocation below."""
    lib = L.lib()
    if wgt is not None and lib.nb_gemm_w4a4_uses_tcgen05(C.byref(a), epi, epi_kind) == 1:
        _attach_prepared(a, wgt, wscales)
    need = lib.nb_gemm_w4a4_scratch_bytes(C.byref(a), epi, epi_kind)
    scratch = None
    if need > 0:
        scratch = torch.empty(need, dtype=torch.uint8, device=act.device)
        a.scratch, a.scratch_bytes = L.ptr(scratch), need
    with torch.cuda.device(act.device):
        L.check(lib.nb_gemm_w4a4(C.byref(a), epi, epi_kind, L.stream_of(act)), "gemm_w4a4")
    return scratch


def gemm_w4a4(
    act: torch.Tensor,
    wgt: torch.Tensor,
    out: torch.Tensor | None = None,
    ascales: torch.Tensor | None = None,
    wscales: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    lora_act_in: torch.Tensor | None = None,
    lora_up: torch.Tensor | None = None,
    wcscales: torch.Tensor | None = None,
    norm_q: torch.Tensor | None = None,
    norm_k: torch.Tensor | None = None,
    rotary_emb: torch.Tensor | None = None,
    qout: torch.Tensor | None = None,
    oscales: torch.Tensor | None = None,
    smooth_factor: torch.Tensor | None = None,
    lora_down: torch.Tensor | None = None,
    lora_act_out: torch.Tensor | None = None,
    act_unsigned: bool = False,
    fuse_silu: bool = False,
    fp4: bool = False,
    alpha: float = 1.0,
    out_dtype: torch.dtype = torch.bfloat16,
    fuse_swiglu: bool = False,
    _impl: int = L.IMPL_AUTO,
) -> torch.Tensor | None:
    """
    ``out = alpha * wcscale * (deq(act) @ deq(wgt).T) + lora_act @ lora_up.T + bias`` with the optional
    fused epilogues; arguments, allocation rules and assertion behaviour follow the reference's
    ``gemm_w4a4`` (nunchaku/ops/triton/gemm_w4a4.py:1003-1314):

    * ``norm_q / norm_k / rotary_emb``: per-head RMSNorm + RoPE on the Q and K thirds.  One table of
      ``S`` rows may serve ``B * S`` activation rows (row ``m`` reads ``rotary_emb[m % S]``).
    * ``qout / oscales`` (+ ``smooth_factor, lora_down, lora_act_out``): GELU, ``+0.171875``, next-layer
      unsigned int4 quantisation and LoRA-down; ``out`` then is optional (pre-GELU tile).
    * ``fuse_swiglu``: ``silu(gate) * up`` on 16-row interleaved rows, signed re-quantisation.
    ``_impl`` selects the kernel (tests only).
    """
    assert ascales is not None and wscales is not None, "W4A4 GEMM requires both scale tensors"
    act = act.reshape(-1, act.shape[-1])
    M, K, N = act.shape[0], act.shape[1] * 2, wgt.shape[0]
    assert wgt.shape[1] * 2 == K, f"weight K mismatch: {wgt.shape[1] * 2} vs {K}"
    group_size = 16 if fp4 else 64
    assert K % group_size == 0
    L.require_cuda(act, wgt, out, ascales, wscales, bias, lora_act_in, lora_up, wcscales, norm_q, norm_k, rotary_emb,
                   qout, oscales, smooth_factor, lora_down, lora_act_out)
    has_lora = lora_act_in is not None and lora_up is not None
    la, lu = (lora_act_in, lora_up) if has_lora else (None, None)

    if fuse_swiglu:
        assert out is None and qout is not None and oscales is not None, "fuse_swiglu writes qout/oscales, not out"
        assert not (
            fp4 or fuse_silu or wcscales is not None or norm_q is not None or rotary_emb is not None
        ), "fuse_swiglu is int4-only and excludes the other epilogues"
        assert alpha is None or alpha == 1.0
        assert (lora_down is None) == (lora_act_out is None), "lora_down and lora_act_out must be given together"
        dtype = oscales.dtype
        _checks(act, wgt, None, ascales, wscales, bias, la, lu, None, False, dtype)
        qout2d = qout.reshape(-1, qout.shape[-1])
        a = _gemm_args(act, wgt, None, ascales, wscales, bias, la, lu, None, act_unsigned, False, False, 1.0, dtype, _impl)
        q, keep = _requant_args(qout2d, oscales, smooth_factor, lora_down, lora_act_out, 0.0, N // 2, M, dtype)
        _run(a, C.byref(q), L.EPI_SWIGLU_QUANT, act, wgt, wscales, keep)
        return None

    want_quant = qout is not None or oscales is not None
    if want_quant:
        assert qout is not None and oscales is not None, "qout and oscales must be given together"
    fuse_quant = (
        want_quant
        and not fp4
        and norm_q is None
        and rotary_emb is None
        and not fuse_silu
        and wcscales is None
        and (alpha is None or alpha == 1.0)
        and N % 128 == 0
        and qout.stride(-1) == 1
        and (lora_down is None) == (lora_act_out is None)
    )
    if out is None and not fuse_quant:
        out = torch.empty(M, N, dtype=out_dtype, device=act.device)
    out2d = out.reshape(-1, N) if out is not None else None
    actual_m = out2d.shape[0] if out2d is not None else M
    assert actual_m <= M, f"out has more rows ({actual_m}) than act ({M})"
    dtype = out2d.dtype if out2d is not None else oscales.dtype
    _checks(act, wgt, out2d, ascales, wscales, bias, la, lu, wcscales, fp4, dtype)

    want_qk = norm_q is not None or norm_k is not None or rotary_emb is not None
    if want_qk:
        assert (
            norm_q is not None and norm_k is not None and rotary_emb is not None
        ), "norm_q, norm_k, and rotary_emb must all be given together"

    if fuse_quant:
        a = _gemm_args(act, wgt, out2d, ascales, wscales, bias, la, lu, None, act_unsigned, False, False, 1.0, dtype, _impl)
        qout2d = qout.reshape(-1, qout.shape[-1])
        q, keep = _requant_args(qout2d, oscales, smooth_factor, lora_down, lora_act_out, GELU_SHIFT, N, M, dtype)
        fused_fast = L.lib().nb_gemm_w4a4_uses_tcgen05(C.byref(a), C.byref(q), L.EPI_GELU_QUANT) == 1
        if fused_fast or _impl == L.IMPL_GENERIC:
            _run(a, C.byref(q), L.EPI_GELU_QUANT, act, wgt, wscales, keep)
            return out
        # no fused tensor-core kernel for this call: GEMM to a 16-bit tile, then the quantizer with the
        # GELU fused in, as the reference does for calls its fused kernel does not take (gemm_w4a4.py:1298-1312)
        if out2d is None:
            out2d = torch.empty(M, N, dtype=dtype, device=act.device)

    fuse_qk = want_qk and N % 3 == 0 and (N // 3) % HEAD_DIM == 0 and rotary_emb.dtype == torch.float32
    a = _gemm_args(act, wgt, out2d, ascales, wscales, bias, la, lu, wcscales, act_unsigned, fuse_silu, fp4, alpha, dtype, _impl)
    if fuse_qk:
        assert rotary_emb.numel() % HEAD_DIM == 0
        rot = rotary_emb.reshape(-1, HEAD_DIM)
        assert rot.stride(1) == 1
        S = rot.shape[0]
        if not (S == actual_m or (S < actual_m and actual_m % S == 0)):
            raise ValueError(f"rotary_emb has {S} rows for {actual_m} output rows")
        nq, nk = norm_q.contiguous(), norm_k.contiguous()
        if nq.dtype != dtype or nk.dtype != dtype or nq.numel() != HEAD_DIM or nk.numel() != HEAD_DIM:
            raise ValueError(f"norm_q/norm_k must be ({HEAD_DIM},) tensors of the output dtype")
        q = L.QKArgs(L.ptr(nq), L.ptr(nk), L.ptr(rot), rot.stride(0), S, 1e-6)
        _run(a, C.byref(q), L.EPI_QK, act, wgt, wscales, (nq, nk))
    else:
        _run(a, None, L.EPI_STORE, act, wgt, wscales)
        if want_qk:
            _apply_rmsnorm_rope_qk(out2d, norm_q, norm_k, rotary_emb)

    if want_quant:
        shift_value = 0.0 if fp4 else GELU_SHIFT
        _launch_quantize(
            out2d, qout, oscales, lora_down, lora_act_out, smooth_factor, fuse_glu=False, fp4=fp4, fuse_gelu=True,
            shift_value=shift_value, unsigned=not fp4,
        )
    return out


def _requant_args(qout2d, oscales, smooth, lora_down, lora_act_out, shift, Nq, M, dtype):
    if qout2d.dtype != torch.uint8 or qout2d.shape[0] < M or qout2d.shape[1] != Nq // 2 or qout2d.stride(-1) != 1:
        raise ValueError(f"qout shape/dtype {tuple(qout2d.shape)} {qout2d.dtype}")
    if oscales.dtype != dtype or oscales.dim() != 2 or oscales.shape[0] != Nq // 64 or oscales.shape[1] < M:
        raise ValueError(f"oscales shape {tuple(oscales.shape)}")
    if smooth is not None and (smooth.dtype != dtype or smooth.numel() != Nq):
        raise ValueError("smooth_factor must be a (N,) tensor of the output dtype")
    q = L.RequantArgs()
    q.qout, q.oscales = L.ptr(qout2d), L.ptr(oscales)
    smooth = smooth.contiguous() if smooth is not None else None  # returned: the caller keeps a copy alive over the launch
    q.smooth = L.ptr(smooth)
    if lora_down is not None:
        R2 = lora_down.shape[1]
        if lora_down.dtype != dtype or lora_down.shape[0] != Nq or lora_down.stride(-1) != 1:
            raise ValueError(f"lora_down shape/dtype {tuple(lora_down.shape)} {lora_down.dtype}")
        if lora_act_out.dtype != torch.float32 or lora_act_out.shape[0] < M or lora_act_out.shape[1] != R2:
            raise ValueError("lora_act_out must be (>= M, R2) fp32")
        q.lora_down, q.lora_act_out, q.R2 = L.ptr(lora_down), L.ptr(lora_act_out), R2
        q.stride_ld, q.stride_lom = lora_down.stride(0), lora_act_out.stride(0)
    q.shift = shift
    q.stride_qm, q.stride_osg = qout2d.stride(0), oscales.stride(0)
    return q, (smooth,)


def gemm_w4a4_group_sums(act, wgt, act_unsigned: bool = False, _impl: int = L.IMPL_AUTO) -> torch.Tensor:
    """
    Debug: the exact int32 ``p_g[m, n]`` of every 64-group as the selected kernel accumulates them,
    ``(K/64, M, N)`` int32 -- the integer contract of nunchaku/ops/triton/gemm_w4a4.py:477-483.
    """
    act = act.reshape(-1, act.shape[-1])
    M, K, N = act.shape[0], act.shape[1] * 2, wgt.shape[0]
    dev = L.require_cuda(act, wgt)
    ones_a = torch.ones(K // 64, M, dtype=torch.bfloat16, device=dev)
    ones_w = torch.ones(K // 64, N, dtype=torch.bfloat16, device=dev)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    p = torch.empty(K // 64, M, N, dtype=torch.int32, device=dev)
    a = _gemm_args(act, wgt, out, ones_a, ones_w, None, None, None, None, act_unsigned, False, False, 1.0,
                   torch.bfloat16, _impl)
    need = L.lib().nb_gemm_w4a4_scratch_bytes(C.byref(a), None, L.EPI_STORE)
    scratch = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
    a.scratch, a.scratch_bytes = L.ptr(scratch), need
    with torch.cuda.device(dev):
        L.check(L.lib().nb_gemm_w4a4_group_sums(C.byref(a), L.ptr(p), L.stream_of(act)), "gemm_w4a4_group_sums")
    return p

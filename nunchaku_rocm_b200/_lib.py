"""
ctypes binding of ``libnunchaku_b200.so`` (declarations: ``include/nunchaku_b200.h``).

Mirrors the reference's way of reaching its native kernels: raw ``data_ptr()``s and strides in C
structs, launched on torch's current stream with a device guard
(nunchaku/ops/triton/native/hip.py:129-167, nunchaku/ops/triton/native/w4a4.py:80-124).
There is no fallback: a missing library or a non-zero status raises.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("NUNCHAKU_B200_LIB") or os.path.join(_HERE, "libnunchaku_b200.so")

NB_OK, NB_ERR_INVALID, NB_ERR_UNSUPPORTED, NB_ERR_LAUNCH, NB_ERR_DEVICE, NB_ERR_TOO_LARGE = range(6)
DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1}
EPI_STORE, EPI_QK, EPI_GELU_QUANT, EPI_SWIGLU_QUANT = range(4)
IMPL_AUTO, IMPL_TCGEN05, IMPL_GENERIC, IMPL_TCGEN05_PAIR, IMPL_TCGEN05_SINGLE = range(5)
NOALLOC_SCRATCH_BYTES = 16 << 20  # NB_NOALLOC_SCRATCH_BYTES


class GemmArgs(C.Structure):
    _fields_ = (
        [(n, C.c_void_p) for n in ("act", "wgt", "out", "ascales", "wscales", "bias", "lora_act", "lora_up", "wcscales")]
        + [
            (n, C.c_int32)
            for n in ("M", "N", "K", "actual_m", "R", "dtype", "act_unsigned", "fp4", "fuse_silu", "impl")
        ]
        + [("alpha", C.c_float)]
        + [
            (n, C.c_int64)
            for n in ("stride_am", "stride_wn", "stride_asg", "stride_wsg", "stride_om", "stride_lam", "stride_lun")
        ]
        + [("status", C.c_void_p), ("scratch", C.c_void_p), ("scratch_bytes", C.c_int64)]
        + [("wgt_prepared", C.c_void_p), ("wgt_prepared_bytes", C.c_int64)]
    )


class QKArgs(C.Structure):
    _fields_ = [
        ("norm_q", C.c_void_p),
        ("norm_k", C.c_void_p),
        ("rot", C.c_void_p),
        ("stride_rm", C.c_int64),
        ("rot_rows", C.c_int32),
        ("eps", C.c_float),
    ]


class RequantArgs(C.Structure):
    _fields_ = (
        [(n, C.c_void_p) for n in ("qout", "oscales", "smooth", "lora_down", "lora_act_out")]
        + [("R2", C.c_int32), ("shift", C.c_float)]
        + [(n, C.c_int64) for n in ("stride_qm", "stride_osg", "stride_ld", "stride_lom")]
    )


class QuantArgs(C.Structure):
    _fields_ = (
        [(n, C.c_void_p) for n in ("input", "output", "oscales", "lora_down", "lora_act_out", "smooth")]
        + [(n, C.c_int32) for n in ("M", "K", "R", "dtype", "fuse_glu", "fuse_gelu", "fp4", "is_unsigned")]
        + [("shift", C.c_float)]
        + [(n, C.c_int64) for n in ("stride_im", "stride_om", "stride_sg", "stride_ld", "stride_lam")]
    )


class AttnArgs(C.Structure):
    _fields_ = (
        [(n, C.c_void_p) for n in ("q", "k", "v", "o")]
        + [(n, C.c_int32) for n in ("B", "H", "Tq", "Tkv", "D", "dtype")]
        + [("scale", C.c_float)]
        + [
            (n, C.c_int64)
            for n in (
                "stride_qb", "stride_qh", "stride_qm",
                "stride_kb", "stride_kh", "stride_kn",
                "stride_vb", "stride_vh", "stride_vn",
                "stride_ob", "stride_om",
            )
        ]
        + [("scratch", C.c_void_p), ("scratch_bytes", C.c_int64), ("status", C.c_void_p), ("impl", C.c_int32)]
    )


_lock = threading.RLock()
_lib = None


class NativeLibraryError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """The loaded library; raises when it has not been built (no CPU or eager fallback exists)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise NativeLibraryError(
                        f"{LIB_PATH} is missing: build it with `python -m nunchaku_rocm_b200.build` "
                        "(nvcc, sm_100a). There is no fallback path."
                    )
                l = C.CDLL(LIB_PATH)
                l.nb_strerror.restype = C.c_char_p
                l.nb_last_cuda_error_string.restype = C.c_char_p
                l.nb_last_error_detail.restype = C.c_char_p
                l.nb_gemm_w4a4_scratch_bytes.restype = C.c_int64
                l.nb_gemm_w4a4.argtypes = [C.POINTER(GemmArgs), C.c_void_p, C.c_int, C.c_void_p]
                l.nb_gemm_w4a4_scratch_bytes.argtypes = [C.POINTER(GemmArgs), C.c_void_p, C.c_int]
                l.nb_gemm_w4a4_noalloc.argtypes = [C.POINTER(GemmArgs), C.c_void_p, C.c_int, C.c_void_p]
                l.nb_gemm_w4a4_uses_tcgen05.restype = C.c_int64
                l.nb_gemm_w4a4_uses_tcgen05.argtypes = [C.POINTER(GemmArgs), C.c_void_p, C.c_int]
                l.nb_gemm_w4a4_prepared_bytes.restype = C.c_int64
                l.nb_gemm_w4a4_prepared_bytes.argtypes = [C.POINTER(GemmArgs)]
                l.nb_gemm_w4a4_prepare_weights.restype = C.c_int
                l.nb_gemm_w4a4_prepare_weights.argtypes = [C.POINTER(GemmArgs), C.c_void_p, C.c_int64, C.c_void_p]
                l.nb_gemm_w4a4_group_sums.argtypes = [C.POINTER(GemmArgs), C.c_void_p, C.c_void_p]
                l.nb_quantize_w4a4.argtypes = [C.POINTER(QuantArgs), C.c_void_p]
                l.nb_attention.argtypes = [C.POINTER(AttnArgs), C.c_void_p]
                l.nb_attention_scratch_bytes.argtypes = [C.POINTER(AttnArgs)]
                l.nb_attention_scratch_bytes.restype = C.c_int64
                l.nb_debug_expire_wait.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
                l.nb_qk_norm_rope.argtypes = [
                    C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.POINTER(QKArgs), C.c_void_p,
                ]
                _lib = l
    return _lib


def check(status: int, what: str) -> None:
    """Raise for a non-zero status (error convention of nunchaku/ops/triton/native/hip.py:110-116)."""
    if status == NB_OK:
        return
    l = lib()
    msg = l.nb_strerror(status).decode()
    detail = l.nb_last_error_detail().decode()
    if detail:
        msg += f" ({detail})"
    if status == NB_ERR_LAUNCH:
        msg += ": " + l.nb_last_cuda_error_string().decode()
        l.nb_last_cuda_error()
    if status == NB_ERR_INVALID:
        raise ValueError(f"{what}: {msg}")
    if status == NB_ERR_UNSUPPORTED:
        raise NotImplementedError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg}")


def ptr(t: torch.Tensor | None):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_of(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


_selftested: set[int] = set()


def ensure_selftest(dev: torch.device) -> None:
    """
    Run the library's self-test once per device before the first kernel call on it, as the reference does when its
    native module is first loaded (nunchaku/ops/triton/native/w4a4.py:371-389, 533-704): small seeded problems on the
    tensor-core kernels against the CUDA-core kernel.  A mismatch raises; nothing is silently switched off.
    The test allocates and synchronises, so a first call that happens inside a stream capture postpones it to the next
    call outside one.  ``NUNCHAKU_B200_SELFTEST=0`` skips it.
    """
    i = dev.index if dev.index is not None else torch.cuda.current_device()
    if i in _selftested:
        return
    if os.environ.get("NUNCHAKU_B200_SELFTEST", "1") == "0":
        _selftested.add(i)
        return
    if torch.cuda.is_current_stream_capturing():
        return
    with _lock:
        if i in _selftested:
            return
        with torch.cuda.device(i):
            rc = lib().nb_selftest()
        if rc != NB_OK:
            raise RuntimeError(
                f"libnunchaku_b200 self-test failed on cuda:{i} ({lib().nb_strerror(rc).decode()}): the tensor-core "
                "kernels disagree with the CUDA-core kernel on this device"
            )
        _selftested.add(i)


def require_cuda(*tensors: torch.Tensor | None) -> torch.device:
    """All given tensors must live on one CUDA device; there is no CPU path.  First use of a device runs the self-test."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if t.device.type != "cuda":
            raise RuntimeError("nunchaku_rocm_b200 kernels need CUDA tensors (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("tensors on different devices")
    if dev is not None:
        ensure_selftest(dev)
    return dev


_status_words: dict[int, torch.Tensor] = {}


def status_word(dev: torch.device) -> torch.Tensor:
    """One int32 per device that kernels set when a bounded wait expires; read by :func:`device_status`."""
    i = dev.index if dev.index is not None else torch.cuda.current_device()
    w = _status_words.get(i)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=dev)
        _status_words[i] = w
    return w


def device_status(dev: torch.device | None = None) -> int:
    """Synchronising read of the device status word (0 = no kernel ever gave up on a wait)."""
    if dev is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    return int(status_word(dev).item())


class KernelWaitExpired(RuntimeError):
    """A kernel gave up on a bounded wait: its results are void (nb_status NB_ERR_DEVICE)."""


def check_device_status(dev: torch.device | None = None, reset: bool = True) -> None:
    """
    Synchronise and raise :class:`KernelWaitExpired` if any kernel since the last check set the device's status word
    (the error convention of nunchaku/ops/triton/native/hip.py:110-116: a runtime failure becomes an exception and the
    stored error is cleared).  ``reset`` zeroes the word so that later work starts clean.
    """
    if dev is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    code = device_status(dev)
    if code:
        if reset:
            status_word(dev).zero_()
        raise KernelWaitExpired(
            f"{lib().nb_strerror(NB_ERR_DEVICE).decode()} on {dev}: status {code:#x} (role/barrier code of the kernel)"
        )

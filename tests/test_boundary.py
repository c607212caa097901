"""CPU-only checks of the drop-in boundary: the library loads, exports what the header declares, and the
Python operators keep the reference's signatures and refuse to run without CUDA tensors."""

import inspect
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from nunchaku_rocm_b200 import _lib

    lib = _lib.lib()
    header = open(os.path.join(ROOT, "include", "nunchaku_b200.h")).read()
    declared = sorted(set(re.findall(r"^(?:int|int64_t|const char\*)\s+(nb_[a-z0-9_]+)\s*\(", header, re.M)))
    assert len(declared) >= 10
    for sym in declared:
        assert hasattr(lib, sym), f"{sym} is declared in the header but not exported"
    assert lib.nb_version() >= 100
    assert lib.nb_strerror(0) == b"ok" and b"unsupported" in lib.nb_strerror(2)


def test_struct_sizes_match_the_header():
    # natural alignment, no packing pragmas: sizes computed from the header's field lists
    from nunchaku_rocm_b200 import _lib

    assert ctypes_size(_lib.GemmArgs) == 9 * 8 + 10 * 4 + 4 + 4 + 7 * 8 + 3 * 8 + 2 * 8  # pad after alpha to 8
    assert ctypes_size(_lib.QKArgs) == 3 * 8 + 8 + 4 + 4
    assert ctypes_size(_lib.RequantArgs) == 5 * 8 + 4 + 4 + 4 * 8
    assert ctypes_size(_lib.QuantArgs) == 6 * 8 + 8 * 4 + 4 + 4 + 5 * 8


def _header_struct_fields(name: str) -> list[str]:
    """Field names of `typedef struct <name> {...}` in the header, in declaration order."""
    header = open(os.path.join(ROOT, "include", "nunchaku_b200.h")).read()
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), header, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        # "const void* a"  /  "int32_t M, N, K"  /  "int64_t stride_am, stride_wn"
        first, *rest = decl.split(",")
        names.append(re.search(r"([A-Za-z_][A-Za-z0-9_]*)\s*$", first).group(1))
        names += [r.strip().lstrip("*").strip() for r in rest]
    return names


def _integration_snippet_fields() -> list[str]:
    """Field names of the `GemmArgs` ctypes structure shown in INTEGRATION.md, by evaluating that snippet."""
    import ctypes

    md = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    code = re.search(r"class GemmArgs\(C\.Structure\):.*?\n\n", md, re.S).group(0)
    ns = {"C": ctypes}
    exec(code, ns)
    return [f[0] for f in ns["GemmArgs"]._fields_], ctypes.sizeof(ns["GemmArgs"])


def test_struct_fields_match_the_header_and_the_integration_snippet():
    # a binding that is one field short makes the library read past the caller's struct
    from nunchaku_rocm_b200 import _lib

    for cname, ctype in (("nb_gemm_args", _lib.GemmArgs), ("nb_qk_args", _lib.QKArgs),
                         ("nb_requant_args", _lib.RequantArgs), ("nb_quant_args", _lib.QuantArgs),
                         ("nb_attn_args", _lib.AttnArgs)):
        assert _header_struct_fields(cname) == [f[0] for f in ctype._fields_], cname
    names, size = _integration_snippet_fields()
    assert names == _header_struct_fields("nb_gemm_args")
    assert size == ctypes_size(_lib.GemmArgs)


def ctypes_size(t):
    import ctypes

    return ctypes.sizeof(t)


def test_op_signatures_match_reference():
    # parameter names and order of nunchaku/ops/gemm.py:12-42, quantize.py:11-21, gemm_w4a4.py:1003-1027
    from nunchaku_rocm_b200.ops.gemm import svdq_gemm_w4a4_cuda
    from nunchaku_rocm_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import gemm_w4a4, quantize_w4a4_act_fuse_lora

    assert list(inspect.signature(svdq_gemm_w4a4_cuda).parameters) == [
        "act", "wgt", "out", "qout", "ascales", "wscales", "oscales", "poolout", "lora_act_in", "lora_up",
        "lora_down", "lora_act_out", "norm_q", "norm_k", "rotary_emb", "bias", "smooth_factor", "out_vk",
        "out_linearattn", "act_unsigned", "lora_scales", "fuse_silu", "fp4", "alpha", "wcscales", "out_q", "out_k",
        "out_v", "attn_tokens",
    ]
    assert list(inspect.signature(svdq_quantize_w4a4_act_fuse_lora_cuda).parameters) == [
        "input", "output", "oscales", "lora_down", "lora_act_out", "smooth", "fuse_glu", "fp4", "pad_size",
    ]
    assert list(inspect.signature(gemm_w4a4).parameters)[:23] == [
        "act", "wgt", "out", "ascales", "wscales", "bias", "lora_act_in", "lora_up", "wcscales", "norm_q", "norm_k",
        "rotary_emb", "qout", "oscales", "smooth_factor", "lora_down", "lora_act_out", "act_unsigned", "fuse_silu",
        "fp4", "alpha", "out_dtype", "fuse_swiglu",
    ]
    assert list(inspect.signature(quantize_w4a4_act_fuse_lora).parameters) == [
        "input", "output", "oscales", "lora_down", "lora_act_out", "smooth", "fuse_glu", "fp4", "fuse_gelu",
        "shift_value", "unsigned",
    ]


def test_backend_is_the_natural_layout_seam(monkeypatch):
    from nunchaku_rocm_b200.ops import backend

    assert backend.get_backend() == "triton" and not backend.has_cuda_extension()
    monkeypatch.setenv("NUNCHAKU_BACKEND", "bogus")
    with pytest.raises(ValueError):
        backend.get_backend()
    monkeypatch.delenv("NUNCHAKU_BACKEND")
    backend.set_backend("triton")
    backend.set_backend(None)
    with pytest.raises(ValueError):
        backend.set_backend("rocm")
    with pytest.raises(RuntimeError):
        backend.set_backend("cuda")
    with pytest.raises(RuntimeError):
        backend.load_cuda_ops()


def test_no_cpu_fallback():
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import gemm_w4a4, quantize_w4a4_act_fuse_lora

    x = torch.randn(8, 64).to(torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        quantize_w4a4_act_fuse_lora(x)
    act = torch.zeros(8, 32, dtype=torch.uint8)
    s = torch.ones(1, 8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        gemm_w4a4(act, act, None, s, s)


def test_unsupported_epilogues_raise_like_the_reference():
    from nunchaku_rocm_b200.ops.gemm import svdq_gemm_w4a4_cuda

    act = torch.zeros(8, 32, dtype=torch.uint8)
    s = torch.ones(1, 8, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError, match="out_q"):
        svdq_gemm_w4a4_cuda(act, act, ascales=s, wscales=s, lora_up=torch.zeros(8, 16), out_q=torch.zeros(1))


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "nunchaku_rocm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, re.M), f"{f} imports the oracle"


def test_a_failing_self_test_raises_on_first_use(monkeypatch):
    # the reference refuses to use its native module when the load-time self-test fails
    # (nunchaku/ops/triton/native/w4a4.py:371-389); here the first op on a device raises
    import contextlib

    from nunchaku_rocm_b200 import _lib

    class FakeLib:
        calls = 0

        def nb_selftest(self):
            FakeLib.calls += 1
            return _lib.NB_ERR_DEVICE

        def nb_strerror(self, rc):
            return b"a kernel gave up on a bounded wait"

    monkeypatch.setattr(_lib, "lib", lambda: FakeLib())
    monkeypatch.setattr(_lib, "_selftested", set())
    monkeypatch.setattr(torch.cuda, "device", lambda i: contextlib.nullcontext())
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    monkeypatch.delenv("NUNCHAKU_B200_SELFTEST", raising=False)
    with pytest.raises(RuntimeError, match="self-test failed on cuda:3"):
        _lib.ensure_selftest(torch.device("cuda", 3))
    assert FakeLib.calls == 1 and 3 not in _lib._selftested
    # a passing test is remembered per device and not repeated
    FakeLib.nb_selftest = lambda self: 0
    _lib.ensure_selftest(torch.device("cuda", 3))
    _lib.ensure_selftest(torch.device("cuda", 3))
    assert 3 in _lib._selftested
    # inside a stream capture the test is postponed, not skipped for good
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: True)
    _lib.ensure_selftest(torch.device("cuda", 4))
    assert 4 not in _lib._selftested

"""
"The reference's model classes run unchanged": the import alias of INTEGRATION.md (section 1) is installed exactly as
written there, the reference's own ``nunchaku/models/linear.py`` (from the unmodified install under ``baseline/_ref``) is
loaded on top of it, and its layers are run through this library's operators.
"""

import importlib.util
import os
import re
import sys
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LINEAR = os.path.join(ROOT, "baseline", "_ref", "nunchaku", "models", "linear.py")


def _alias_snippet() -> str:
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    m = re.search(r"import alias installed before the model classes are imported:\s*```python\n(.*?)```", text, re.S)
    assert m, "the alias snippet is missing from INTEGRATION.md"
    return m.group(1)


@pytest.fixture()
def aliased():
    """Install the alias (with an empty stand-in for the parent package) and undo it afterwards."""
    before = dict(sys.modules)
    for name in ("nunchaku", "nunchaku.models"):
        pkg = types.ModuleType(name)
        pkg.__path__ = []
        sys.modules[name] = pkg
    exec(compile(_alias_snippet(), "INTEGRATION.md:alias", "exec"), {})
    yield
    for k in list(sys.modules):
        if k not in before:
            del sys.modules[k]
    sys.modules.update(before)


def _load_reference_linear():
    if not os.path.exists(REF_LINEAR):
        pytest.skip("the reference install (baseline/_ref) is not present")
    spec = importlib.util.spec_from_file_location("nunchaku.models.linear", REF_LINEAR)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["nunchaku.models.linear"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_alias_covers_every_module_and_resolves_to_this_library(aliased):
    import nunchaku_rocm_b200.ops as ours

    names = re.findall(r'"(ops[\w.]*)"', _alias_snippet())
    assert len(names) >= 14
    for n in names:
        assert sys.modules["nunchaku." + n] is importlib.import_module("nunchaku_rocm_b200." + n)
    from nunchaku.ops.gemm import svdq_gemm_w4a4_cuda  # noqa: E402  (resolved through the alias)
    from nunchaku.ops.backend import get_backend  # noqa: E402

    assert svdq_gemm_w4a4_cuda is ours.gemm.svdq_gemm_w4a4_cuda
    assert get_backend() == "triton"


def test_reference_linear_classes_import_and_bind_to_this_library(aliased):
    ref = _load_reference_linear()
    import nunchaku_rocm_b200.ops.gemm as g
    import nunchaku_rocm_b200.ops.gemv as v
    import nunchaku_rocm_b200.ops.quantize as q

    assert ref.svdq_gemm_w4a4_cuda is g.svdq_gemm_w4a4_cuda
    assert ref.awq_gemv_w4a16_cuda is v.awq_gemv_w4a16_cuda
    assert ref.svdq_quantize_w4a4_act_fuse_lora_cuda is q.svdq_quantize_w4a4_act_fuse_lora_cuda
    lin = ref.SVDQW4A4Linear(256, 384, rank=16)
    assert lin.qweight.shape == (384, 128) and lin.wscales.shape == (4, 384)
    awq = ref.AWQW4A16Linear(256, 384, group_size=64)
    assert awq.qweight.shape == (96, 128)


@pytest.mark.gpu
@pytest.mark.parametrize("precision", ["int4", "nvfp4"])
def test_reference_linear_forward_runs_on_this_library(aliased, precision):
    """The unmodified reference layer class, driven by this library's operators, against this package's mirror of the
    class (bit for bit: same operators, same order) and against the oracle chain."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    ref = _load_reference_linear()
    from nunchaku_rocm_b200.models.linear import SVDQW4A4Linear as Mirror
    from oracle import w4a4

    dev = torch.device("cuda", 0)
    T = torch.bfloat16
    cin, cout, rank, tokens = 512, 768, 32, 200
    g = torch.Generator().manual_seed(11)
    a = ref.SVDQW4A4Linear(cin, cout, rank=rank, precision=precision, torch_dtype=T, device=dev)
    b = Mirror(cin, cout, rank=rank, precision=precision, torch_dtype=T, device=dev)
    params = dict(
        qweight=torch.randint(-128, 128, a.qweight.shape, dtype=torch.int8, generator=g),
        bias=(torch.randn(cout, generator=g) * 0.1).to(T),
        smooth_factor=(torch.rand(cin, generator=g) + 0.5).to(T),
        proj_down=(torch.randn(cin, rank, generator=g) * 0.05).to(T),
        proj_up=(torch.randn(cout, rank, generator=g) * 0.05).to(T),
    )
    if precision == "int4":
        params["wscales"] = (torch.rand(a.wscales.shape, generator=g) * 0.02 + 0.005).to(T)
    else:
        params["wscales"] = (torch.rand(a.wscales.shape, generator=g) * 0.05 + 0.01).to(torch.float8_e4m3fn)
        params["wcscales"] = (torch.rand(cout, generator=g) * 0.5 + 0.5).to(T)
    with torch.no_grad():
        for layer in (a, b):
            for k, v in params.items():
                getattr(layer, k).copy_(v.to(dev))
            if precision == "nvfp4":
                layer.wtscale = 0.75
    x = torch.randn(1, tokens, cin, generator=g).to(T)
    with torch.no_grad():
        ya, yb = a(x.to(dev)), b(x.to(dev))
    assert ya.shape == (1, tokens, cout)
    assert torch.equal(ya, yb)
    fp4 = precision == "nvfp4"
    q, s, la, _ = w4a4.quantize_act(x[0], lora_down=params["proj_down"], smooth=params["smooth_factor"], fp4=fp4)
    want = w4a4.gemm_w4a4(q, params["qweight"].view(torch.uint8), s, params["wscales"], bias=params["bias"], lora_act=la,
                          lora_up=params["proj_up"], fp4=fp4, alpha=0.75 if fp4 else 1.0, wcscales=params.get("wcscales"))
    err = w4a4.rel_fro(ya[0].float().cpu(), want.float())
    assert err <= 5e-3, err

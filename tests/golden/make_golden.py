"""
Generate ``tests/golden/*.npz`` by running the reference's own CPU-runnable code on seeded inputs.

Run once, in a container that has the reference checkout (read-only) available:

    python tests/golden/make_golden.py /path/to/nunchaku-rocm

The reference's package ``__init__`` imports diffusers, which is not installed, and its Triton
modules need a GPU driver at import, so the pure-PyTorch modules are loaded by file path under
stub packages, the way the reference's own tests do (tests/triton/conftest.py:22-35).
Loaded: nunchaku/ops/triton/native/w4a4.py (``reference*``, ``_unpack``, ``interleave_swiglu``),
nunchaku/lora/flux/packer.py, nunchaku/ops/triton/layout.py,
nunchaku/models/text_encoders/tinychat_utils.py (``pack_w4``), and the ``rope`` function cut out of
nunchaku/models/embeddings.py (the module itself imports diffusers).

bf16 tensors are stored as their uint16 bit patterns (key suffix ``__bf16``).
"""

from __future__ import annotations

import ast
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _stub(name: str, path: str) -> None:
    m = types.ModuleType(name)
    m.__path__ = [path]
    sys.modules[name] = m


def _load(name: str, file: str):
    spec = importlib.util.spec_from_file_location(name, file)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_reference(root: str):
    n = os.path.join(root, "nunchaku")
    _stub("nunchaku", n)
    _stub("nunchaku.lora", os.path.join(n, "lora"))
    _stub("nunchaku.lora.flux", os.path.join(n, "lora", "flux"))
    _stub("nunchaku.ops", os.path.join(n, "ops"))
    _stub("nunchaku.ops.triton", os.path.join(n, "ops", "triton"))
    _stub("nunchaku.ops.triton.native", os.path.join(n, "ops", "triton", "native"))
    _stub("nunchaku.models", os.path.join(n, "models"))
    _stub("nunchaku.models.text_encoders", os.path.join(n, "models", "text_encoders"))
    _load("nunchaku.utils", os.path.join(n, "utils.py"))
    _load("nunchaku.lora.flux.utils", os.path.join(n, "lora", "flux", "utils.py"))
    packer = _load("nunchaku.lora.flux.packer", os.path.join(n, "lora", "flux", "packer.py"))
    layout = _load("nunchaku.ops.triton.layout", os.path.join(n, "ops", "triton", "layout.py"))
    _load("nunchaku.ops.triton.native.build", os.path.join(n, "ops", "triton", "native", "build.py"))
    native = _load("nunchaku.ops.triton.native.w4a4", os.path.join(n, "ops", "triton", "native", "w4a4.py"))
    tiny = _load(
        "nunchaku.models.text_encoders.tinychat_utils", os.path.join(n, "models", "text_encoders", "tinychat_utils.py")
    )
    # rope(): cut the function out of embeddings.py
    src = open(os.path.join(n, "models", "embeddings.py")).read()
    fn = next(x for x in ast.parse(src).body if isinstance(x, ast.FunctionDef) and x.name == "rope")
    ns = {"torch": torch}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "embeddings.rope", "exec"), ns)
    return native, packer, layout, tiny, ns["rope"]


def _np(t: torch.Tensor):
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def save(name: str, **tensors):
    out = {}
    for k, v in tensors.items():
        if isinstance(v, torch.Tensor):
            if v.dtype == torch.bfloat16:
                k += "__bf16"
            elif v.dtype == torch.float8_e4m3fn:
                k += "__e4m3"
            out[k] = _np(v)
        else:
            out[k] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, {k: v.shape for k, v in out.items()})


def main(root: str) -> None:
    native, packer_mod, layout, tiny, rope = load_reference(root)
    T = torch.bfloat16
    g = torch.Generator().manual_seed(1234)

    def rnd(*shape):
        return torch.rand(*shape, generator=g)

    def nrm(*shape):
        return torch.randn(*shape, generator=g)

    # ---- 1. reference(): the self-test shape of native/w4a4.py:537 and a second shape -------------
    for tag, (M, N, K, R) in {"a": (136, 264, 256, 16), "b": (64, 128, 384, 32)}.items():
        act = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
        wgt = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
        asc = (rnd(K // 64, M) * 0.02 + 0.01).to(T)
        wsc = (rnd(K // 64, N) * 0.02 + 0.01).to(T)
        bias = nrm(N).to(T)
        la = nrm(M, R)
        lu = (nrm(N, R) * 0.1).to(T)
        outs = {}
        for uns in (False, True):
            outs[f"out_{'u' if uns else 's'}"] = native.reference(act, wgt, asc, wsc, bias, la, lu, uns)
        outs["out_nolora_s"] = native.reference(act, wgt, asc, wsc, None, None, None, False)
        save(f"gemm_{tag}", act=act, wgt=wgt, ascales=asc, wscales=wsc, bias=bias, lora_act=la, lora_up=lu, **outs)

    # ---- 2. reference_qk ------------------------------------------------------------------------
    M, N = 40, 3 * 2 * 128
    lin = nrm(M, N) * 3
    nq = (rnd(128) + 0.5).to(T)
    nk = (rnd(128) + 0.5).to(T)
    rot = nrm(M, 128)
    save("qk", lin=lin, norm_q=nq, norm_k=nk, rot=rot, out=native.reference_qk(lin, nq, nk, rot))

    # ---- 3. reference_gelu_quant / reference_swiglu_quant ------------------------------------------
    M, N, R2 = 48, 256, 48
    lin = nrm(M, N) * 2
    smooth = (rnd(N) + 0.5).to(T)
    ld = (nrm(N, R2) * 0.1).to(T)
    q, s, l = native.reference_gelu_quant(lin, smooth, ld, T)
    save("gelu_quant", lin=lin, smooth=smooth, lora_down=ld, codes=q, scales=s, lora=l)
    H = N // 2
    smooth_h = (rnd(H) + 0.5).to(T)
    ld_h = (nrm(H, R2) * 0.1).to(T)
    q, s, l = native.reference_swiglu_quant(lin, smooth_h, ld_h, T)
    save(
        "swiglu_quant",
        lin=lin,
        smooth=smooth_h,
        lora_down=ld_h,
        codes=q,
        scales=s,
        lora=l,
        interleave=native.interleave_swiglu(N),
    )

    # ---- 4. AWQ TinyChat packing ------------------------------------------------------------------
    n, k = 64, 128
    q = torch.randint(0, 16, (n, k), dtype=torch.int32, generator=g)
    save("awq_pack", q=q, packed_i16=tiny.pack_w4(q))

    # ---- 5. checkpoint (mma-fragment) layout: packer outputs and the converter's inverses -----------
    P = packer_mod.NunchakuWeightPacker(bits=4)
    n, k, r = 256, 256, 32
    codes = torch.randint(-8, 8, (n, k), dtype=torch.int32, generator=g)
    packed_w = P.pack_weight(codes)
    scale = (rnd(n, k // 64) * 0.02 + 0.01).to(T)  # (n, groups) as the packer takes it
    packed_s = P.pack_scale(scale, group_size=64)
    chan = nrm(n).to(T)
    packed_c = P.pack_scale(chan, group_size=-1)
    micro = (rnd(n, k // 16) * 2 + 0.1).to(T)
    packed_m = P.pack_micro_scale(micro, group_size=16)
    up = (nrm(n, r) * 0.1).to(T)
    down_t = (nrm(r, k) * 0.1).to(T)  # (rank, in): what pack_lowrank_weight(down=True) takes
    packed_up = P.pack_lowrank_weight(up, down=False)
    packed_down = P.pack_lowrank_weight(down_t, down=True)
    save(
        "layout",
        codes=codes,
        packed_w=packed_w,
        unpacked_w=layout.unpack_weight(packed_w, n, k),
        scale=scale,
        packed_s=packed_s,
        unpacked_s=layout.unpack_scale(packed_s, n, 64),
        chan=chan,
        packed_c=packed_c,
        unpacked_c=layout.unpack_scale(packed_c.reshape(1, -1), n, -1),
        micro=micro,
        packed_m=packed_m,
        unpacked_m=layout.unpack_scale(packed_m, n, 16),
        up=up,
        packed_up=packed_up,
        unpacked_up=P.unpack_lowrank_weight(packed_up, down=False),
        down_t=down_t,
        packed_down=packed_down,
        unpacked_down=P.unpack_lowrank_weight(packed_down, down=True),
    )

    # ---- 6. rope() ---------------------------------------------------------------------------------
    pos = torch.tensor([[0.0, 1.0, 2.0, 17.0, 63.0]])
    save("rope", pos=pos, out16=rope(pos, 16, 10000), out56=rope(pos, 56, 10000))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of the reference repository>")
    main(sys.argv[1])

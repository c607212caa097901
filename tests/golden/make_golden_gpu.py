"""
Run the reference's own Triton kernels on an NVIDIA GPU (they are arch-generic; Triton's NVIDIA backend compiles them)
and store their outputs as fixtures, plus their run times as a speed bar on the same device.

    python tests/golden/make_golden_gpu.py <copy of the reference checkout> <output directory>

The modules under ``nunchaku/ops/triton`` are loaded by file path inside a private package, exactly as the reference's
test suite does (tests/triton/conftest.py:22-35), so neither ``nunchaku/__init__`` nor diffusers is needed.  Its native
hipRTC module reports itself unavailable off gfx11 and the Triton kernels run.

Fixtures pin the oracle pieces that exist only as Triton kernels in the reference: the plain activation quantizer
(signed, unsigned+GELU, NVFP4), the generic NVFP4 GEMM, the int4 GEMM with the fused GELU re-quantisation, the AWQ GEMV
and the attention kernel.  Each ``.npz`` holds the seeded inputs and the reference's outputs; ``tests/test_oracle.py``
compares the oracle with them on the CPU and ``tests/test_reference_gpu_vectors.py`` the CUDA kernels on the GPU.
bf16 tensors are stored as uint16 bit patterns (``__bf16``), e4m3 as bytes (``__e4m3``).
"""

from __future__ import annotations

import importlib.util
import json
import os
import sys
import time

import numpy as np
import torch

T = torch.bfloat16
PKG = "_nunchaku_triton"


def load_kernels(root: str, name: str):
    d = os.path.join(root, "nunchaku", "ops", "triton")
    if PKG not in sys.modules:
        pkg = importlib.util.module_from_spec(importlib.util.spec_from_loader(PKG, loader=None, is_package=True))
        pkg.__path__ = [d]
        sys.modules[PKG] = pkg
    full = f"{PKG}.{name}"
    if full not in sys.modules:
        spec = importlib.util.spec_from_file_location(full, os.path.join(d, f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[full] = mod
        spec.loader.exec_module(mod)
    return sys.modules[full]


def _np(t: torch.Tensor):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def save(outdir: str, name: str, **tensors) -> None:
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
    np.savez_compressed(os.path.join(outdir, name + ".npz"), **out)
    print("saved", name, {k: tuple(v.shape) for k, v in out.items()}, flush=True)


def timed(fn, iters: int = 20, warm: int = 5) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main(root: str, outdir: str) -> None:
    os.makedirs(outdir, exist_ok=True)
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(4321)
    W = load_kernels(root, "gemm_w4a4")
    A = load_kernels(root, "attention")
    Q = load_kernels(root, "awq")
    times: dict[str, float | str] = {"device": torch.cuda.get_device_name(0)}
    import triton

    times["triton"] = triton.__version__

    def rnd(*s):
        return torch.rand(*s, generator=g)

    def nrm(*s):
        return torch.randn(*s, generator=g)

    def d(t):
        return None if t is None else t.to(dev)

    # ---- 1. activation quantizer: signed + smooth + LoRA-down, unsigned + GELU + shift, NVFP4 ------------------------
    M, K, R = 72, 512, 32
    x = nrm(M, K)
    x[:, ::61] *= 20
    x = x.to(T)
    ld = (nrm(K, R) * 0.1).to(T)
    sm = (rnd(K) + 0.5).to(T)
    q, s, l = W.quantize_w4a4_act_fuse_lora(d(x), lora_down=d(ld), smooth=d(sm))
    qu, su, lu_ = W.quantize_w4a4_act_fuse_lora(d(x), lora_down=d(ld), smooth=d(sm), fuse_gelu=True, shift_value=0.171875,
                                                unsigned=True)
    qf, sf, _ = W.quantize_w4a4_act_fuse_lora(d(x), fp4=True)
    x2 = nrm(M, 2 * K).to(T)
    qg, sg, lg = W.quantize_w4a4_act_fuse_lora(d(x2), lora_down=d(ld), fuse_glu=True)
    save(outdir, "triton_quantize", x=x, x_glu=x2, lora_down=ld, smooth=sm, q_signed=q[:M], s_signed=s[:, :M], l_signed=l[:M],
         q_gelu_u=qu[:M], s_gelu_u=su[:, :M], l_gelu_u=lu_[:M], q_fp4=qf[:M], s_fp4=sf[:, :M], q_glu=qg[:M],
         s_glu=sg[:, :M], l_glu=lg[:M])

    # ---- 2. NVFP4 GEMM (generic kernel of the reference): wcscales, alpha, LoRA-up, bias ------------------------------
    M, N, K, R = 136, 264, 512, 16
    act = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    wgt = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    asc = (rnd(K // 16, M) * 0.05 + 0.01).to(torch.float8_e4m3fn)
    wsc = (rnd(K // 16, N) * 0.05 + 0.01).to(torch.float8_e4m3fn)
    wcs = (rnd(N) * 0.5 + 0.5).to(T)
    bias = nrm(N).to(T)
    la = nrm(M, R) * 0.5
    lu = (nrm(N, R) * 0.1).to(T)
    out = W.gemm_w4a4(d(act), d(wgt), None, d(asc), d(wsc), d(bias), d(la), d(lu), wcscales=d(wcs), alpha=0.75, fp4=True,
                      out_dtype=T)
    save(outdir, "triton_gemm_fp4", act=act, wgt=wgt, ascales=asc, wscales=wsc, wcscales=wcs, bias=bias, lora_act=la,
         lora_up=lu, alpha=0.75, out=out)

    # ---- 3. int4 GEMM: plain, fused Q/K RMSNorm + RoPE, fused GELU re-quantisation ---------------------------------------
    M, N, K, R, R2 = 144, 768, 256, 16, 48
    act = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    wgt = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    asc = (rnd(K // 64, M) * 0.02 + 0.01).to(T)
    wsc = (rnd(K // 64, N) * 0.02 + 0.01).to(T)
    bias = nrm(N).to(T)
    la = nrm(M, R)
    lu = (nrm(N, R) * 0.1).to(T)
    nq = (1 + nrm(128) * 0.05).to(T)
    nk = (1 + nrm(128) * 0.05).to(T)
    th = rnd(M, 64) * 6.28
    rot = torch.stack([torch.sin(th), torch.cos(th)], -1).reshape(M, 64, 1, 2).float().contiguous()
    smq = (rnd(N) + 0.5).to(T)
    ldq = (nrm(N, R2) * 0.1).to(T)
    plain = W.gemm_w4a4(d(act), d(wgt), None, d(asc), d(wsc), d(bias), d(la), d(lu))
    qk = W.gemm_w4a4(d(act), d(wgt), None, d(asc), d(wsc), d(bias), d(la), d(lu), norm_q=d(nq), norm_k=d(nk),
                     rotary_emb=d(rot))
    res = {}
    for uns in (False, True):
        qout = torch.zeros(M, N // 2, dtype=torch.uint8, device=dev)
        osc = torch.zeros(N // 64, M, dtype=T, device=dev)
        lao = torch.zeros(M, R2, dtype=torch.float32, device=dev)
        W.gemm_w4a4(d(act), d(wgt), None, d(asc), d(wsc), d(bias), d(la), d(lu), qout=qout, oscales=osc,
                    smooth_factor=d(smq), lora_down=d(ldq), lora_act_out=lao, act_unsigned=uns)
        tag = "u" if uns else "s"
        res.update({f"gq_q_{tag}": qout, f"gq_s_{tag}": osc, f"gq_l_{tag}": lao})
    save(outdir, "triton_gemm_int4", act=act, wgt=wgt, ascales=asc, wscales=wsc, bias=bias, lora_act=la, lora_up=lu,
         norm_q=nq, norm_k=nk, rot=rot, smooth=smq, lora_down=ldq, out_plain=plain, out_qk=qk, **res)

    # ---- 4. attention (tail in both directions), AWQ GEMV --------------------------------------------------------------
    B, H, TQ, TKV, D = 1, 3, 200, 333, 128
    qa, ka, va = (nrm(B, H, TQ if i == 0 else TKV, D).to(T) for i in range(3))
    qa[:, :, ::7] *= 4.0
    o = torch.empty(B, TQ, H * D, dtype=T, device=dev)
    A.attention_fp16(d(qa), d(ka), d(va), o, D**-0.5)
    save(outdir, "triton_attention", q=qa, k=ka, v=va, o=o)

    n, k = 256, 512
    packed = torch.randint(-(2**31), 2**31 - 1, (n // 4, k // 2), dtype=torch.int32, generator=g)
    sc = (rnd(k // 64, n) * 0.1 + 0.01).to(T)
    zr = (nrm(k // 64, n) * 0.1).to(T)
    xv = nrm(3, k).to(T)
    og = Q.awq_gemv_w4a16(d(xv), d(packed), d(sc), d(zr), 3, n, k, 64)
    save(outdir, "triton_awq_gemv", x=xv, kernel=packed, scales=sc, zeros=zr, out=og)

    # ---- 5. the reference's kernels timed on this device at the benchmark shapes (speed bar; CUDA events, 20 iterations) --
    def big(M, N, K, R=32):
        a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device=dev)
        w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev)
        return (a, w, (torch.rand(K // 64, M, device=dev) * 0.02 + 0.01).to(T),
                (torch.rand(K // 64, N, device=dev) * 0.02 + 0.01).to(T), torch.randn(N, device=dev).to(T),
                torch.randn(M, R, device=dev), (torch.randn(N, R, device=dev) * 0.1).to(T))

    try:
        M = 4608
        a, w, as_, ws_, b_, la_, lu_ = big(M, 3072, 3072)
        o_ = torch.empty(M, 3072, dtype=T, device=dev)
        times["gemm_int4_4608x3072x3072_ms"] = timed(lambda: W.gemm_w4a4(a, w, o_, as_, ws_, b_, la_, lu_))
        a, w, as_, ws_, b_, la_, lu_ = big(M, 9216, 3072)
        o_ = torch.empty(M, 9216, dtype=T, device=dev)
        th = torch.rand(M, 64, device=dev) * 6.28
        rot_ = torch.stack([torch.sin(th), torch.cos(th)], -1).reshape(M, 64, 1, 2).float().contiguous()
        nq_, nk_ = torch.ones(128, dtype=T, device=dev), torch.ones(128, dtype=T, device=dev)
        times["gemm_int4_qk_4608x9216x3072_ms"] = timed(
            lambda: W.gemm_w4a4(a, w, o_, as_, ws_, b_, la_, lu_, norm_q=nq_, norm_k=nk_, rotary_emb=rot_))
        a, w, as_, ws_, b_, la_, lu_ = big(M, 12288, 3072)
        qo = torch.empty(M, 6144, dtype=torch.uint8, device=dev)
        os_ = torch.empty(192, M, dtype=T, device=dev)
        lo_ = torch.empty(M, 32, dtype=torch.float32, device=dev)
        sm_ = torch.ones(12288, dtype=T, device=dev)
        ld_ = (torch.randn(12288, 32, device=dev) * 0.1).to(T)
        times["gemm_int4_gelu_quant_4608x12288x3072_ms"] = timed(
            lambda: W.gemm_w4a4(a, w, None, as_, ws_, b_, la_, lu_, qout=qo, oscales=os_, smooth_factor=sm_, lora_down=ld_,
                                lora_act_out=lo_))
        xq = torch.randn(M, 3072, device=dev).to(T)
        ldq_ = (torch.randn(3072, 32, device=dev) * 0.1).to(T)
        times["quantize_4608x3072_rank32_ms"] = timed(lambda: W.quantize_w4a4_act_fuse_lora(xq, lora_down=ldq_, smooth=sm_[:3072]))
        qa_, ka_, va_ = (torch.randn(1, 24, 4608, 128, device=dev).to(T) for _ in range(3))
        oa_ = torch.empty(1, 4608, 3072, dtype=T, device=dev)
        times["attention_b1_h24_t4608_d128_ms"] = timed(lambda: A.attention_fp16(qa_, ka_, va_, oa_, 128**-0.5), iters=10)
        Mq = 7168
        af = torch.randint(0, 256, (Mq, 1536), dtype=torch.uint8, device=dev)
        wf = torch.randint(0, 256, (9216, 1536), dtype=torch.uint8, device=dev)
        asf = (torch.rand(192, Mq, device=dev) * 0.05 + 0.01).to(torch.float8_e4m3fn)
        wsf = (torch.rand(192, 9216, device=dev) * 0.05 + 0.01).to(torch.float8_e4m3fn)
        of = torch.empty(Mq, 9216, dtype=T, device=dev)
        times["gemm_nvfp4_7168x9216x3072_ms"] = timed(lambda: W.gemm_w4a4(af, wf, of, asf, wsf, fp4=True), iters=5, warm=2)
        kp = torch.randint(-(2**31), 2**31 - 1, (18432 // 4, 3072 // 2), dtype=torch.int32, device=dev)
        sc_ = (torch.rand(48, 18432, device=dev) * 0.1 + 0.01).to(T)
        zr_ = (torch.randn(48, 18432, device=dev) * 0.1).to(T)
        xv_ = torch.randn(1, 3072, device=dev).to(T)
        times["awq_gemv_18432x3072_m1_ms"] = timed(lambda: Q.awq_gemv_w4a16(xv_, kp, sc_, zr_, 1, 18432, 3072, 64))
    except Exception as e:  # a fixture run is still useful when a timing case fails
        times["timing_error"] = f"{type(e).__name__}: {e}"
    with open(os.path.join(outdir, "triton_reference_times.json"), "w") as f:
        json.dump(times, f, indent=1)
    print(json.dumps(times), flush=True)


if __name__ == "__main__":
    t0 = time.time()
    main(sys.argv[1], sys.argv[2])
    print(f"done in {time.time() - t0:.0f} s")

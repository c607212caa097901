"""
Per-kernel timings of the hot path on one GPU, after the reference's
``tests/triton/bench_kernels.py`` (:36-44: warm-up, timed iterations, TFLOP/s = 2MNK/t for GEMMs, 4BHT^2D/t for
attention, GB/s for the quantizer).  Differences: CUDA events around a CUDA graph of the launches instead of wall clock, inputs
rotated over several buffer sets so that HBM-bound kernels do not run out of L2, and every line carries the roofline
that bounds the kernel and the fraction of the measured peak (``MEASURED_PEAKS.json`` beside the repository root, else
the stated fallback).

    python -m nunchaku_rocm_b200.bench_kernels [--iters 50] [--warmup 10] [--only quantize,gemm,mlp,fp4,awq,layout,attention]

Prints one JSON object per kernel and shape.  Synthetic seeded inputs with the benchmark configurations' shapes.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from bench import make_cfg_inputs, measured_peaks  # noqa: E402  (bench.py sits at the repository root)


def time_ms(fn, sets, iters, warmup):
    """
    Per-launch device time of ``fn(set)``, rotating through ``sets``.  The ``iters`` launches are captured into one CUDA
    graph and the graph is timed with CUDA events (median and best of five replays, divided by ``iters``): a kernel of a
    few microseconds would otherwise be timed together with the host's launch overhead.
    """
    for i in range(warmup):
        fn(sets[i % len(sets)])
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(iters):
                fn(sets[i % len(sets)])
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    t = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        t.append(a.elapsed_time(b) / iters)
    return statistics.median(t), min(t)


def emit(kernel, shape, ms, best, work, unit, bound, peak, src, extra=None):
    achieved = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
    line = {
        "kernel": kernel, "shape": shape, "ms_median": round(ms, 5), "ms_best": round(best, 5),
        "bound": bound, "achieved": round(achieved, 2), "unit": unit, "peak": peak, "frac": round(achieved / peak, 4),
        "peak_source": src,
    }
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--only", default="quantize,gemm,mlp,fp4,awq,layout,attention")
    args = ap.parse_args()
    only = set(args.only.split(","))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, src = measured_peaks()
    hbm = float(peaks["hbm_gbs"])
    bf16 = float(peaks["bf16_tflops"])
    i8 = 2.0 * bf16  # the 8-bit tensor pipe runs at twice the bf16 rate; the driver measures bf16 only

    from nunchaku_rocm_b200.ops.quantize import svdq_quantize_w4a4_act_fuse_lora_cuda as quantize
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import gemm_w4a4
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import quantize_w4a4_act_fuse_lora as quantize_kernel_level
    from nunchaku_rocm_b200.ops.triton.awq import awq_gemv_w4a16
    from nunchaku_rocm_b200.ops.triton.attention import attention_fp16

    M, R = 4608, 32
    T = torch.bfloat16

    # ---------------------------------------------------------------- activation quantizer (HBM)
    if "quantize" in only:
        for K in (3072, 12288):
            n_sets = max(2, math.ceil(400e6 / (M * K * 2)))
            sets = []
            for i in range(n_sets):
                p = make_cfg_inputs(M, K, 128, R, dev, seed=i)
                mp = (M + 255) // 256 * 256
                p["q"] = torch.empty(mp, K // 2, dtype=torch.uint8, device=dev)
                p["s"] = torch.empty(K // 64, mp, dtype=T, device=dev)
                p["l"] = torch.empty(mp, R, dtype=torch.float32, device=dev)
                sets.append(p)
            ms, best = time_ms(lambda p: quantize(p["x"], p["q"], p["s"], p["proj_down"], p["l"], p["smooth"]), sets,
                               args.iters, args.warmup)
            work = 2 * M * K + M * K // 2 + 2 * (K // 64) * M + 4 * M * R + 2 * K * R
            emit("quantize_kernel", f"M={M} K={K} R={R} signed int4", ms, best, work, "GB/s", "hbm", hbm, src)
            if K == 12288:  # the GELU + shift + unsigned re-quantisation between fc1 and fc2 of an MLP
                ms, best = time_ms(lambda p: quantize_kernel_level(p["x"], p["q"][:M], p["s"][:, :M], p["proj_down"], p["l"][:M],
                                                                   p["smooth"], fuse_gelu=True, shift_value=0.171875,
                                                                   unsigned=True), sets, args.iters, args.warmup)
                emit("quantize_kernel", f"M={M} K={K} R={R} GELU + shift, unsigned int4", ms, best, work, "GB/s", "hbm", hbm, src)
            del sets

    # ---------------------------------------------------------------- W4A4 GEMM (tensor pipe)
    if "gemm" in only:
        cases = [("plain", 3072, 3072, False), ("qk_norm_rope", 3072, 9216, False), ("fc2 unsigned acts", 12288, 3072, True)]
        for name, K, N, uns in cases:
            sets = []
            for i in range(3):
                p = make_cfg_inputs(M, K, N, R, dev, seed=10 + i)
                if uns:
                    xx = p["x"].float().abs().to(T)
                    p["q"], p["s"], p["l"] = quantize_kernel_level(xx, lora_down=p["proj_down"], smooth=p["smooth"], unsigned=True)
                else:
                    p["q"], p["s"], p["l"] = quantize(p["x"], lora_down=p["proj_down"], smooth=p["smooth"])
                p["out"] = torch.empty(M, N, dtype=T, device=dev)
                sets.append(p)
            kw = (lambda p: dict(norm_q=p["norm_q"], norm_k=p["norm_k"], rotary_emb=p["rotary_emb"])) if name == "qk_norm_rope" else (lambda p: {})
            ms, best = time_ms(lambda p: gemm_w4a4(p["q"], p["qweight"], p["out"], p["s"], p["wscales"], p["bias"], p["l"],
                                                   p["proj_up"], act_unsigned=uns, **kw(p)), sets, args.iters, args.warmup)
            emit("activation pre-pass + tcgen05 int4 GEMM", f"{name}: M={M} K={K} N={N} R={R}", ms, best, 2.0 * M * N * K, "TFLOP/s",
                 "tensor", i8, src + " x2 (8-bit pipe)")
            del sets

    # ---------------------------------------------------------------- transformer MLP pair through the layer API
    if "mlp" in only:
        from nunchaku_rocm_b200.models.linear import SVDQW4A4Linear
        from nunchaku_rocm_b200.ops.fused import fused_gelu_mlp

        def rand_layer(cin, cout, unsigned, seed):
            g = torch.Generator(device=dev).manual_seed(seed)
            lin = SVDQW4A4Linear(cin, cout, rank=R, bias=True, precision="int4", act_unsigned=unsigned, torch_dtype=T, device=dev)
            with torch.no_grad():
                lin.qweight.copy_(torch.randint(-128, 128, lin.qweight.shape, dtype=torch.int8, generator=g, device=dev))
                lin.wscales.copy_((torch.rand(lin.wscales.shape, generator=g, device=dev) * 0.015 + 0.005).to(T))
                lin.bias.copy_((torch.randn(cout, generator=g, device=dev) * 0.1).to(T))
                lin.smooth_factor.copy_((torch.rand(cin, generator=g, device=dev) + 0.5).to(T))
                lin.proj_down.copy_((torch.randn(cin, R, generator=g, device=dev) * 0.02).to(T))
                lin.proj_up.copy_((torch.randn(cout, R, generator=g, device=dev) * 0.02).to(T))
            return lin

        fc1, fc2 = rand_layer(3072, 12288, False, 1), rand_layer(12288, 3072, True, 2)
        for Mm in (256, 1024, 4608, 8192):
            g = torch.Generator(device=dev).manual_seed(Mm)
            sets = [dict(x=torch.randn(1, Mm, 3072, generator=g, device=dev).to(T)) for _ in range(3)]
            ms, best = time_ms(lambda p: fused_gelu_mlp(p["x"], fc1, fc2), sets, max(10, args.iters // 2), args.warmup)
            emit("fused_gelu_mlp (quantize, fc1 GEMM, GELU + requant, fc2 GEMM)", f"M={Mm} 3072->12288->3072 R={R}", ms, best,
                 2.0 * Mm * 12288 * 3072 * 2, "TFLOP/s", "tensor", i8, src + " x2 (8-bit pipe)")

    # ---------------------------------------------------------------- NVFP4 GEMM (block-scaled tensor pipe)
    if "fp4" in only:
        fp4_peak = 4.0 * bf16  # e2m1 operands run at four times the bf16 rate; the driver measures bf16 only
        for name, Mq, K, N in [("qwen qkv", 7168, 3072, 9216), ("qwen mlp fc1", 7168, 3072, 12288), ("qwen mlp fc2", 7168, 12288, 3072)]:
            sets = []
            for i in range(3):
                g = torch.Generator(device=dev).manual_seed(20 + i)
                p = dict(
                    act=torch.randint(0, 256, (Mq, K // 2), dtype=torch.uint8, generator=g, device=dev),
                    wgt=torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g, device=dev),
                    asc=(torch.rand(K // 16, Mq, generator=g, device=dev) * 0.05 + 0.01).to(torch.float8_e4m3fn),
                    wsc=(torch.rand(K // 16, N, generator=g, device=dev) * 0.05 + 0.01).to(torch.float8_e4m3fn),
                    wcs=(torch.rand(N, generator=g, device=dev) * 0.5 + 0.5).to(T),
                    bias=torch.randn(N, generator=g, device=dev).to(T),
                    la=torch.randn(Mq, R, generator=g, device=dev),
                    lu=(torch.randn(N, R, generator=g, device=dev) * 0.02).to(T),
                    out=torch.empty(Mq, N, dtype=T, device=dev))
                sets.append(p)
            ms, best = time_ms(lambda p: gemm_w4a4(p["act"], p["wgt"], p["out"], p["asc"], p["wsc"], p["bias"], p["la"], p["lu"],
                                                   wcscales=p["wcs"], alpha=0.9, fp4=True), sets, args.iters, args.warmup)
            emit("prepack_fp4_kernel + gemm_fp4_kernel", f"{name}: M={Mq} K={K} N={N} R={R}", ms, best, 2.0 * Mq * N * K, "TFLOP/s",
                 "tensor", fp4_peak, src + " x4 (4-bit pipe)")
            del sets

    # ---------------------------------------------------------------- AWQ W4A16 GEMV (HBM)
    if "awq" in only:
        n, k = 18432, 3072
        g = torch.Generator().manual_seed(0)
        sets = []
        for i in range(8):  # 8 x 32 MB of weights > L2
            sets.append(dict(  # every 4-bit pattern is a valid code, so random words are a valid packed weight
                w=torch.randint(-(2**31), 2**31 - 1, (n // 4, k // 2), dtype=torch.int32, generator=g).to(dev),
                s=(torch.rand(k // 64, n, generator=g) * 0.1 + 0.01).to(T).to(dev),
                z=(torch.randn(k // 64, n, generator=g) * 0.1).to(T).to(dev)))
        for m in (1, 2, 4, 8):
            x = torch.randn(m, k, generator=g).to(T).to(dev)
            ms, best = time_ms(lambda p: awq_gemv_w4a16(x, p["w"], p["s"], p["z"], m, n, k, 64), sets, args.iters, args.warmup)
            work = n * k // 2 + 2 * 2 * (k // 64) * n + 2 * m * k + 2 * m * n
            emit("awq_gemv_kernel", f"m={m} n={n} k={k} g=64", ms, best, work, "GB/s", "hbm", hbm, src)
        # the one-kernel W4A16 GEMM for larger batches (legacy mma.sync tensor path: about a third of the bf16 peak at best)
        from nunchaku_rocm_b200.ops.triton.awq import awq_gemm_w4a16
        for m in (512, 4608):
            x = torch.randn(m, k, generator=g).to(T).to(dev)
            ms, best = time_ms(lambda p: awq_gemm_w4a16(x, p["w"], p["s"], p["z"], 64), sets, max(5, args.iters // 5), 3)
            emit("awq_gemm_kernel", f"m={m} n={n} k={k} g=64", ms, best, 2.0 * m * n * k, "TFLOP/s", "tensor", bf16, src)
        del sets

    # ---------------------------------------------------------------- checkpoint layout converter (HBM)
    if "layout" in only:
        from nunchaku_rocm_b200.ops.triton.layout import unpack_weight_packed_nibbles
        n, k = 12288, 3072
        g = torch.Generator().manual_seed(3)
        sets = [dict(w=torch.randint(-128, 128, (n, k // 2), dtype=torch.int8, generator=g).to(dev)) for _ in range(12)]  # 12 x 18.9 MB > L2 with the outputs
        ms, best = time_ms(lambda p: unpack_weight_packed_nibbles(p["w"], n, k), sets, args.iters, args.warmup)
        emit("layout_unpack_weight_kernel", f"n={n} k={k} (stored fragment order -> natural nibbles)", ms, best, n * k, "GB/s", "hbm", hbm, src)
        del sets

    # ---------------------------------------------------------------- attention (tensor pipe, bf16)
    if "attention" in only:
        B, H, D = 1, 24, 128
        for Tn in (4608, 7168):
            g = torch.Generator(device=dev).manual_seed(1)
            sets = []
            for i in range(2):
                qkv = torch.randn(B, Tn, 3, H, D, generator=g, device=dev).to(T)
                q, k, v = (qkv[:, :, j].permute(0, 2, 1, 3) for j in range(3))  # (B, H, T, D) strided views
                sets.append(dict(q=q, k=k, v=v, o=torch.empty(B, Tn, H * D, dtype=T, device=dev)))
            ms, best = time_ms(lambda p: attention_fp16(p["q"], p["k"], p["v"], p["o"], D ** -0.5), sets, args.iters, args.warmup)
            emit("attention_tc_kernel", f"B={B} H={H} T={Tn} D={D} bf16", ms, best, 4.0 * B * H * Tn * Tn * D, "TFLOP/s", "tensor",
                 bf16, src)


if __name__ == "__main__":
    main()

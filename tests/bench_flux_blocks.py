"""
FLUX.1-architecture transformer blocks assembled from this package's operators (a script, not a pytest file):
one double-stream block and one single-stream block with random-init int4 weights, wired as the reference's
``NunchakuFluxTransformerBlock`` / ``NunchakuFluxSingleTransformerBlock`` (nunchaku/models/transformers/
transformer_flux_v2.py:174-343) are, at the benchmark configuration's shapes (hidden 3072, 24 heads x 128, MLP ratio 4,
rank-32 branches, 4096 image + 512 text tokens).  The quantised linears, the fused QKV / MLP operators, the AWQ adaLN
modulation and the attention kernel are this package's; LayerNorm, modulation arithmetic, gating and residuals are
plain torch, as in the reference (diffusers layers).

It times each block inside a CUDA graph and extrapolates to the 19 + 38 blocks and 4 denoising steps of the
configuration: an estimate of the transformer's share of an image, with embedders, VAE and text encoders excluded.

    python tests/bench_flux_blocks.py [--batch 1] [--iters 10]
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

HID, HEADS, HD, RANK, TXT, IMG = 3072, 24, 128, 32, 512, 4096


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    T = torch.bfloat16

    from nunchaku_rocm_b200.models.embeddings import flux_image_ids, flux_pos_embed
    from nunchaku_rocm_b200.models.linear import AWQW4A16Linear, SVDQW4A4Linear
    from nunchaku_rocm_b200.ops.dispatch import scaled_dot_product_attention
    from nunchaku_rocm_b200.ops.fused import fused_gelu_mlp, fused_qkv_norm_rottary

    g = torch.Generator(device=dev).manual_seed(0)

    def svdq(cin, cout, unsigned=False):
        lin = SVDQW4A4Linear(cin, cout, rank=RANK, bias=True, precision="int4", act_unsigned=unsigned, torch_dtype=T, device=dev)
        with torch.no_grad():
            lin.qweight.copy_(torch.randint(-128, 128, lin.qweight.shape, dtype=torch.int8, generator=g, device=dev))
            lin.wscales.copy_((torch.rand(lin.wscales.shape, generator=g, device=dev) * 0.015 + 0.005).to(T) / (cin / 3072) ** 0.5)
            lin.bias.copy_((torch.randn(cout, generator=g, device=dev) * 0.02).to(T))
            lin.smooth_factor.copy_((torch.rand(cin, generator=g, device=dev) + 0.5).to(T))
            lin.proj_down.copy_((torch.randn(cin, RANK, generator=g, device=dev) * 0.02).to(T))
            lin.proj_up.copy_((torch.randn(cout, RANK, generator=g, device=dev) * 0.02).to(T))
        return lin

    def awq(cin, cout):
        lin = AWQW4A16Linear(cin, cout, bias=True, group_size=64, torch_dtype=T, device=dev)
        with torch.no_grad():
            lin.qweight.copy_(torch.randint(-2**31, 2**31 - 1, lin.qweight.shape, dtype=torch.int32, generator=g, device=dev))
            lin.wscales.copy_((torch.rand(lin.wscales.shape, generator=g, device=dev) * 0.002 + 0.0005).to(T))
            lin.wzeros.copy_((torch.randn(lin.wzeros.shape, generator=g, device=dev) * 0.005).to(T))
            lin.bias.copy_((torch.randn(cout, generator=g, device=dev) * 0.02).to(T))
        return lin

    class RMS(nn.Module):  # per-head RMSNorm weights of the attention (the operator only needs `.weight`)
        def __init__(self):
            super().__init__()
            self.weight = nn.Parameter((1 + torch.randn(HD, generator=g, device=dev) * 0.05).to(T), requires_grad=False)
            self.eps = 1e-6

    class Stream:  # the quantised layers of one stream of a double block
        def __init__(self):
            self.mod = awq(HID, 6 * HID)
            self.qkv, self.out = svdq(HID, 3 * HID), svdq(HID, HID)
            self.nq, self.nk = RMS(), RMS()
            self.fc1, self.fc2 = svdq(HID, 4 * HID), svdq(4 * HID, HID, unsigned=True)

    img, txt = Stream(), Stream()
    single_mod = awq(HID, 3 * HID)
    single_qkv, single_out = svdq(HID, 3 * HID), svdq(HID, HID)
    single_nq, single_nk = RMS(), RMS()
    single_fc1, single_fc2 = svdq(HID, 4 * HID), svdq(4 * HID, HID, unsigned=True)

    B = args.batch
    rot = flux_pos_embed(flux_image_ids(TXT, 64, 64, device=dev))  # (4608, 64, 1, 2) fp32, text rows first
    rot_txt, rot_img = rot[:TXT].contiguous(), rot[TXT:].contiguous()
    temb = torch.randn(B, HID, generator=g, device=dev).to(T)
    x_img = torch.randn(B, IMG, HID, generator=g, device=dev).to(T)
    x_txt = torch.randn(B, TXT, HID, generator=g, device=dev).to(T)

    def ada_zero(mod, x):
        e = mod(F.silu(temb))  # (B, 6 * HID) through the AWQ GEMV
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = e.chunk(6, dim=1)
        n = F.layer_norm(x, (HID,), eps=1e-6) * (1 + scale_msa[:, None]) + shift_msa[:, None]
        return n, gate_msa, shift_mlp, scale_mlp, gate_mlp

    qkv_joint = torch.empty(B, TXT + IMG, 3 * HID, dtype=T, device=dev)

    def attention(qkv):
        # joint attention over text + image tokens: (B, S, 3, H, D) views of the buffer both projections wrote
        qkv = qkv.view(B, TXT + IMG, 3, HEADS, HD)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        o = scaled_dot_product_attention(q, k, v)  # (B, H, S, D) view of (B, S, H * D)
        o = o.transpose(1, 2).reshape(B, TXT + IMG, HID)
        return o[:, :TXT], o[:, TXT:]

    def double_block(x_img, x_txt):
        n_img, g_msa, sh_mlp, sc_mlp, g_mlp = ada_zero(img.mod, x_img)
        n_txt, cg_msa, csh_mlp, csc_mlp, cg_mlp = ada_zero(txt.mod, x_txt)
        if B == 1:  # both GEMMs write their rows of the joint buffer (a row slice of one batch element is contiguous)
            fused_qkv_norm_rottary(n_img, img.qkv, img.nq, img.nk, rot_img, output=qkv_joint[0, TXT:])
            fused_qkv_norm_rottary(n_txt, txt.qkv, txt.nq, txt.nk, rot_txt, output=qkv_joint[0, :TXT])
            qkv = qkv_joint
        else:
            qkv = torch.cat([fused_qkv_norm_rottary(n_txt, txt.qkv, txt.nq, txt.nk, rot_txt),
                             fused_qkv_norm_rottary(n_img, img.qkv, img.nq, img.nk, rot_img)], dim=1)
        a_txt, a_img = attention(qkv)
        x_img = x_img + g_msa[:, None] * img.out(a_img.contiguous())
        x_txt = x_txt + cg_msa[:, None] * txt.out(a_txt.contiguous())
        n_img = F.layer_norm(x_img, (HID,), eps=1e-6) * (1 + sc_mlp[:, None]) + sh_mlp[:, None]
        n_txt = F.layer_norm(x_txt, (HID,), eps=1e-6) * (1 + csc_mlp[:, None]) + csh_mlp[:, None]
        x_img = x_img + g_mlp[:, None] * fused_gelu_mlp(n_img, img.fc1, img.fc2)
        x_txt = x_txt + cg_mlp[:, None] * fused_gelu_mlp(n_txt, txt.fc1, txt.fc2)
        return x_img, x_txt

    rot_all = rot.contiguous()

    def single_block(x):
        e = single_mod(F.silu(temb))
        shift, scale, gate = e.chunk(3, dim=1)
        n = F.layer_norm(x, (HID,), eps=1e-6) * (1 + scale[:, None]) + shift[:, None]
        mlp = fused_gelu_mlp(n, single_fc1, single_fc2)
        qkv = fused_qkv_norm_rottary(n, single_qkv, single_nq, single_nk, rot_all).view(B, TXT + IMG, 3, HEADS, HD)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        o = scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, TXT + IMG, HID)
        return x + gate[:, None] * (single_out(o) + mlp)

    x_cat = torch.cat([x_txt, x_img], dim=1)

    def timed(fn, iters):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
            for _ in range(iters):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        ts = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); graph.replay(); b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / iters)
        return statistics.median(ts)

    with torch.no_grad():
        out_img, out_txt = double_block(x_img, x_txt)
        out_single = single_block(x_cat)
        assert torch.isfinite(out_img.float()).all() and torch.isfinite(out_txt.float()).all() and torch.isfinite(out_single.float()).all()
        ms_double = timed(lambda: double_block(x_img, x_txt), args.iters)
        ms_single = timed(lambda: single_block(x_cat), args.iters)

    from nunchaku_rocm_b200 import _lib

    assert _lib.device_status(dev) == 0
    step_ms = 19 * ms_double + 38 * ms_single
    tokens = TXT + IMG
    gemm_ops = 2.0 * B * tokens * HID * (3 * HID + HID + 8 * HID)  # per block: qkv, out, fc1, fc2
    attn_flops = 4.0 * B * HEADS * tokens * tokens * HD
    print(json.dumps({
        "what": "FLUX.1-architecture blocks from this package's operators, random-init int4 weights, 4096 image + 512 text tokens",
        "batch": B,
        "double_block_ms": round(ms_double, 4),
        "single_block_ms": round(ms_single, 4),
        "transformer_step_ms (19 double + 38 single)": round(step_ms, 2),
        "images_per_s_per_gpu (4 steps, transformer only)": round(B / (4 * step_ms * 1e-3), 3),
        "block_tops (GEMM ops + attention flops over block time)": {
            "double": round((gemm_ops + attn_flops) / (ms_double * 1e-3) / 1e12, 1),
            "single": round((gemm_ops + attn_flops) / (ms_single * 1e-3) / 1e12, 1),
        },
        "excluded": "embedders, final layer, VAE, text encoders, scheduler",
    }), flush=True)


if __name__ == "__main__":
    main()

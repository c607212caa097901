"""
Block-level parity of the FLUX.1-architecture harness: one double-stream and one single-stream block on the GPU against
the same wiring (nunchaku/models/transformers/transformer_flux_v2.py:174-343) evaluated on the CPU with the oracle's
functions for every quantised operator and plain fp32 torch for the rest.  The blocks re-quantise activations several
times in a row, where a value on a rounding boundary may take the neighbouring code in one implementation and not in the
other, so the block outputs are compared by relative Frobenius error (reported, bar 3e-2); the width is reduced
(hidden 512, 4 heads of 128) so that the CPU side finishes in seconds, the code path is the one the full model runs.
"""

import pytest
import torch
import torch.nn.functional as F

from oracle import awq_attn, w4a4

pytestmark = pytest.mark.gpu
T = torch.bfloat16


def _svdq_params(lin):
    return {k: getattr(lin, k).detach().cpu() for k in ("qweight", "wscales", "bias", "smooth_factor", "proj_down", "proj_up")}


def _o_linear(x, lin):
    """SVDQW4A4Linear.forward on the CPU: quantizer + GEMM of the oracle; x (rows, C) in T, fp32 result rounded to T."""
    p = _svdq_params(lin)
    q, s, l, _ = w4a4.quantize_act(x, p["proj_down"], p["smooth_factor"])
    return w4a4.gemm_w4a4(q, p["qweight"].view(torch.uint8), s, p["wscales"], p["bias"], l, p["proj_up"],
                          act_unsigned=lin.act_unsigned).to(T)


def _o_qkv(x, lin, nq, nk, rot):
    p = _svdq_params(lin)
    q, s, l, _ = w4a4.quantize_act(x, p["proj_down"], p["smooth_factor"])
    lin32 = w4a4.gemm_w4a4(q, p["qweight"].view(torch.uint8), s, p["wscales"], p["bias"], l, p["proj_up"])
    rows = x.shape[0]
    r = rot.reshape(-1, 128)
    r = r.repeat(rows // r.shape[0], 1)
    return w4a4.qk_norm_rope(lin32, nq.weight.detach().cpu(), nk.weight.detach().cpu(), r).to(T)


def _o_gelu_mlp(x, fc1, fc2):
    p1, p2 = _svdq_params(fc1), _svdq_params(fc2)
    q, s, l, _ = w4a4.quantize_act(x, p1["proj_down"], p1["smooth_factor"])
    lin = w4a4.gemm_w4a4(q, p1["qweight"].view(torch.uint8), s, p1["wscales"], p1["bias"], l, p1["proj_up"])
    codes, scale, lora = w4a4.gelu_quant(lin, p2["smooth_factor"], p2["proj_down"], T)
    return w4a4.gemm_w4a4(w4a4.pack_nibbles(codes), p2["qweight"].view(torch.uint8), scale.to(T), p2["wscales"], p2["bias"],
                          lora, p2["proj_up"], act_unsigned=True).to(T)


def _o_awq(x, lin):
    n, k = lin.out_features, lin.in_features
    y = awq_attn.awq_gemv(x, lin.qweight.detach().cpu(), lin.wscales.detach().cpu(), lin.wzeros.detach().cpu(), n, k).to(T)
    return y + lin.bias.detach().cpu()


def _o_adaln(mod, x, emb):
    e = _o_awq(F.silu(emb), mod.linear)
    parts = e.view(e.shape[0], -1, mod.n).permute(2, 0, 1)
    norm = F.layer_norm(x, (mod.dim,), eps=1e-6) * (parts[1] + mod.scale_shift)[:, None] + parts[0][:, None]
    if mod.n == 3:
        return norm, parts[2]
    return norm, parts[2], parts[3], parts[4] + mod.scale_shift, parts[5]


def _o_attention(qkv, cfg):
    B, S, _ = qkv.shape
    q, k, v = (t.view(B, S, cfg.heads, cfg.head_dim).transpose(1, 2) for t in qkv.chunk(3, dim=-1))
    return awq_attn.attention(q, k, v, cfg.head_dim**-0.5).to(T)  # (B, S, H D)


def _o_double(blk, h, e, temb, rot_img, rot_txt):
    cfg = blk.cfg
    B, S_img, C = h.shape
    S_txt = e.shape[1]
    nh, gate_msa, shift_mlp, scale_mlp, gate_mlp = _o_adaln(blk.norm1, h, temb)
    ne, c_gate_msa, c_shift_mlp, c_scale_mlp, c_gate_mlp = _o_adaln(blk.norm1_context, e, temb)
    qkv = torch.cat([_o_qkv(ne.reshape(-1, C), blk.add_qkv_proj, blk.norm_added_q, blk.norm_added_k, rot_txt).view(B, S_txt, -1),
                     _o_qkv(nh.reshape(-1, C), blk.to_qkv, blk.norm_q, blk.norm_k, rot_img).view(B, S_img, -1)], dim=1)
    attn = _o_attention(qkv, cfg)
    ca, a = attn[:, :S_txt], attn[:, S_txt:]
    a = _o_linear(a.reshape(-1, C), blk.to_out).view(B, S_img, C)
    ca = _o_linear(ca.reshape(-1, C), blk.to_add_out).view(B, S_txt, C)
    h = h + gate_msa[:, None] * a
    nh = F.layer_norm(h, (C,), eps=1e-6) * scale_mlp[:, None] + shift_mlp[:, None]
    h = h + gate_mlp[:, None] * _o_gelu_mlp(nh.reshape(-1, C), blk.ff.fc1, blk.ff.fc2).view(B, S_img, C)
    e = e + c_gate_msa[:, None] * ca
    ne = F.layer_norm(e, (C,), eps=1e-6) * c_scale_mlp[:, None] + c_shift_mlp[:, None]
    e = e + c_gate_mlp[:, None] * _o_gelu_mlp(ne.reshape(-1, C), blk.ff_context.fc1, blk.ff_context.fc2).view(B, S_txt, C)
    return e, h


def _o_single(blk, h, temb, rot):
    B, S, C = h.shape
    nh, gate = _o_adaln(blk.norm, h, temb)
    mlp = _o_gelu_mlp(nh.reshape(-1, C), blk.mlp_fc1, blk.mlp_fc2).view(B, S, C)
    qkv = _o_qkv(nh.reshape(-1, C), blk.to_qkv, blk.norm_q, blk.norm_k, rot).view(B, S, -1)
    attn = _o_linear(_o_attention(qkv, blk.cfg).reshape(-1, C), blk.to_out).view(B, S, C)
    return h + gate[:, None] * (attn + mlp)


@pytest.mark.parametrize("batch", [1, 2])
def test_double_and_single_block_match_the_oracle_chain(cuda_dev, batch):
    from nunchaku_rocm_b200 import _lib
    from nunchaku_rocm_b200.models.embeddings import flux_image_ids
    from nunchaku_rocm_b200.models.flux_dit import FluxDiT, FluxDiTConfig

    cfg = FluxDiTConfig(hidden=512, heads=4, head_dim=128, n_double=1, n_single=1, rank=16, axes_dim=(16, 56, 56))
    model = FluxDiT(cfg, device=cuda_dev).random_init(seed=3)
    n_txt, grid = 64, 12
    ids = flux_image_ids(n_txt, grid, grid, device=cuda_dev)
    rot_txt, rot_img, rot_all = model.rotary_tables(ids[:n_txt], ids[n_txt:])
    g = torch.Generator().manual_seed(batch)
    h = torch.randn(batch, grid * grid, cfg.hidden, generator=g).to(T)
    e = torch.randn(batch, n_txt, cfg.hidden, generator=g).to(T)
    temb = torch.randn(batch, cfg.hidden, generator=g).to(T)
    dbl, sgl = model.transformer_blocks[0], model.single_transformer_blocks[0]
    with torch.no_grad():
        e_gpu, h_gpu = dbl(h.to(cuda_dev), e.to(cuda_dev), temb.to(cuda_dev), rot_img, rot_txt)
        x_cat = torch.cat([e_gpu, h_gpu], dim=1)
        s_gpu = sgl(x_cat, temb.to(cuda_dev), rot_all)
        torch.cuda.synchronize(cuda_dev)
        assert _lib.device_status(cuda_dev) == 0
        e_ref, h_ref = _o_double(dbl, h, e, temb, rot_img.cpu(), rot_txt.cpu())
        s_ref = _o_single(sgl, x_cat.cpu(), temb, rot_all.cpu())  # same input as the GPU block: isolates the single block
    errs = {
        "double/image": w4a4.rel_fro(h_gpu.float().cpu(), h_ref.float()),
        "double/text": w4a4.rel_fro(e_gpu.float().cpu(), e_ref.float()),
        "single": w4a4.rel_fro(s_gpu.float().cpu(), s_ref.float()),
    }
    print("\nFLUX block parity (relative Frobenius error vs the oracle chain), batch", batch, errs)
    for k, v in errs.items():
        assert v <= 3e-2, (k, v)


def test_full_model_forward_is_finite_and_graph_replay_is_deterministic(cuda_dev):
    # two double + two single blocks at the real width, 512 text + 1024 image tokens: eager and graph results agree bit for bit
    from nunchaku_rocm_b200.models.flux_dit import FluxDiT, FluxDiTConfig, GraphedStep, denoise

    cfg = FluxDiTConfig(n_double=2, n_single=2)
    model = FluxDiT(cfg, device=cuda_dev).random_init(seed=5)
    step = GraphedStep(model, batch=1, txt_tokens=512, grid=32, seed=1)
    with torch.no_grad():
        eager = step._forward().clone()
        out = step.step(t=1.0).clone()
        again = step.step(t=1.0).clone()
    assert out.shape == (1, 1024, cfg.in_channels) and torch.isfinite(out.float()).all()
    assert torch.equal(out, again) and torch.equal(out, eager)
    x = denoise(step, step.latents.clone(), num_steps=2)
    assert torch.isfinite(x.float()).all()


# ------------------------------------------------------------------------------------------------
# Qwen-Image-architecture block (NVFP4): nunchaku/models/transformers/transformer_qwenimage.py:220-309
# ------------------------------------------------------------------------------------------------
def _fp4_params(lin):
    p = {k: getattr(lin, k).detach().cpu() for k in ("qweight", "wscales", "bias", "smooth_factor", "proj_down", "proj_up", "wcscales")}
    p["alpha"] = lin.wtscale
    return p


def _o_linear_fp4(x, lin):
    p = _fp4_params(lin)
    q, s, l, _ = w4a4.quantize_act(x, p["proj_down"], p["smooth_factor"], fp4=True)
    return w4a4.gemm_w4a4(q, p["qweight"].view(torch.uint8), s, p["wscales"], p["bias"], l, p["proj_up"], fp4=True,
                          alpha=p["alpha"], wcscales=p["wcscales"]).to(T)


def _o_gelu_mlp_fp4(x, fc1, fc2):
    # NVFP4: GEMM -> 16-bit tile -> quantizer with the GELU fused in (gemm_w4a4.py:1298-1312), then fc2
    p2 = _fp4_params(fc2)
    h = _o_linear_fp4(x, fc1)
    q, s, l, _ = w4a4.quantize_act(h, p2["proj_down"], p2["smooth_factor"], fp4=True, fuse_gelu=True)
    return w4a4.gemm_w4a4(q, p2["qweight"].view(torch.uint8), s, p2["wscales"], p2["bias"], l, p2["proj_up"], fp4=True,
                          alpha=p2["alpha"], wcscales=p2["wcscales"]).to(T)


def _o_qwen_block(blk, h, e, temb, img_f, txt_f):
    from nunchaku_rocm_b200.models.qwen_dit import _rms, _rotate

    cfg = blk.cfg
    B, S_img, C = h.shape
    S_txt = e.shape[1]

    def mod(m):
        x = _o_awq(F.silu(temb), m.linear)
        return x.view(B, -1, 6).transpose(1, 2).reshape(B, -1).chunk(2, dim=-1)

    def modulate(x, mp):
        shift, scale, gate = mp.chunk(3, dim=-1)
        return x * (scale + 1.0)[:, None] + shift[:, None], gate[:, None]

    im1, im2 = mod(blk.img_mod)
    tm1, tm2 = mod(blk.txt_mod)
    img_m, ig1 = modulate(F.layer_norm(h, (C,), eps=1e-6), im1)
    txt_m, tg1 = modulate(F.layer_norm(e, (C,), eps=1e-6), tm1)
    iq, ik, iv = (t.unflatten(-1, (cfg.heads, -1)) for t in _o_linear_fp4(img_m.reshape(-1, C), blk.to_qkv).view(B, S_img, -1).chunk(3, dim=-1))
    tq, tk, tv = (t.unflatten(-1, (cfg.heads, -1)) for t in _o_linear_fp4(txt_m.reshape(-1, C), blk.add_qkv_proj).view(B, S_txt, -1).chunk(3, dim=-1))
    w = lambda n: getattr(blk, n).detach().cpu()
    iq, ik = _rotate(_rms(iq, w("norm_q")), img_f), _rotate(_rms(ik, w("norm_k")), img_f)
    tq, tk = _rotate(_rms(tq, w("norm_added_q")), txt_f), _rotate(_rms(tk, w("norm_added_k")), txt_f)
    q, k, v = torch.cat([tq, iq], 1), torch.cat([tk, ik], 1), torch.cat([tv, iv], 1)
    attn = awq_attn.attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), cfg.head_dim**-0.5).to(T)
    ta = _o_linear_fp4(attn[:, :S_txt].reshape(-1, C), blk.to_add_out).view(B, S_txt, C)
    ia = _o_linear_fp4(attn[:, S_txt:].reshape(-1, C), blk.to_out).view(B, S_img, C)
    h = h + ig1 * ia
    e = e + tg1 * ta
    m2, g2 = modulate(F.layer_norm(h, (C,), eps=1e-6), im2)
    h = h + g2 * _o_gelu_mlp_fp4(m2.reshape(-1, C), blk.img_mlp.fc1, blk.img_mlp.fc2).view(B, S_img, C)
    m2, g2 = modulate(F.layer_norm(e, (C,), eps=1e-6), tm2)
    e = e + g2 * _o_gelu_mlp_fp4(m2.reshape(-1, C), blk.txt_mlp.fc1, blk.txt_mlp.fc2).view(B, S_txt, C)
    return e, h


def test_qwen_image_block_matches_the_oracle_chain(cuda_dev):
    from nunchaku_rocm_b200 import _lib
    from nunchaku_rocm_b200.models.qwen_dit import QwenDiT, QwenDiTConfig

    cfg = QwenDiTConfig(hidden=512, heads=4, head_dim=128, n_blocks=1, rank=16)
    model = QwenDiT(cfg, device=cuda_dev).random_init(seed=9)
    blk = model.blocks[0]
    B, S_img, S_txt = 1, 200, 56
    g = torch.Generator().manual_seed(4)
    h = torch.randn(B, S_img, cfg.hidden, generator=g).to(T)
    e = torch.randn(B, S_txt, cfg.hidden, generator=g).to(T)
    temb = torch.randn(B, cfg.hidden, generator=g).to(T)
    img_f, txt_f = model.rotary_freqs(S_img, cfg.head_dim, cuda_dev), model.rotary_freqs(S_txt, cfg.head_dim, cuda_dev)
    with torch.no_grad():
        e_gpu, h_gpu = blk(h.to(cuda_dev), e.to(cuda_dev), temb.to(cuda_dev), img_f, txt_f)
        torch.cuda.synchronize(cuda_dev)
        assert _lib.device_status(cuda_dev) == 0
        e_ref, h_ref = _o_qwen_block(blk, h, e, temb, img_f.cpu(), txt_f.cpu())
    errs = {"image": w4a4.rel_fro(h_gpu.float().cpu(), h_ref.float()), "text": w4a4.rel_fro(e_gpu.float().cpu(), e_ref.float())}
    print("\nQwen-Image block parity (relative Frobenius error vs the oracle chain)", errs)
    for k, v in errs.items():
        assert v <= 3e-2, (k, v)


def test_text_stream_on_a_second_cuda_stream_changes_nothing(cuda_dev, monkeypatch):
    # the blocks run their text stream on a second CUDA stream and the models compute the modulation vectors ahead on a third:
    # the same forward with everything on one stream must give the same bits (a missing dependency between the streams would show here, or as a run-to-run difference)
    from nunchaku_rocm_b200.models import flux_dit, qwen_dit

    fcfg = flux_dit.FluxDiTConfig(n_double=2, n_single=1)
    fmodel = flux_dit.FluxDiT(fcfg, device=cuda_dev).random_init(seed=6)
    fstep = flux_dit.GraphedStep(fmodel, batch=1, txt_tokens=512, grid=32, seed=2)
    qcfg = qwen_dit.QwenDiTConfig(n_blocks=2)
    qmodel = qwen_dit.QwenDiT(qcfg, device=cuda_dev).random_init(seed=7)
    qstep = qwen_dit.GraphedQwenStep(qmodel, batch=1, img_tokens=1024, txt_tokens=256)
    with torch.no_grad():
        two = [fstep._forward().clone(), qstep._forward().clone()]
        again = [fstep._forward().clone(), qstep._forward().clone()]
        replay = [fstep.step().clone(), qstep.step().clone()]
        one_stream = lambda device, which="text": torch.cuda.current_stream(device)
        monkeypatch.setattr(flux_dit, "_side_stream", one_stream)
        monkeypatch.setattr(qwen_dit, "_side_stream", one_stream)
        one = [fstep._forward().clone(), qstep._forward().clone()]
    torch.cuda.synchronize(cuda_dev)
    for a, b, c, d in zip(two, again, replay, one):
        assert torch.isfinite(a.float()).all()
        assert torch.equal(a, b) and torch.equal(a, c) and torch.equal(a, d)

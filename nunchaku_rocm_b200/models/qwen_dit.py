"""
Qwen-Image-architecture MMDiT assembled from this package's operators with NVFP4 W4A4 layers: the block wiring of the
reference's ``NunchakuQwenImageTransformerBlock`` (nunchaku/models/transformers/transformer_qwenimage.py:220-309) and its
attention processor (nunchaku/models/attention_processors/qwenimage.py:66-148):

* modulation ``SiLU -> AWQ W4A16 linear`` with the interleaved ``[dim, 6]`` output rows, split into two (shift, scale + 1,
  gate) triples per stream;
* ``to_qkv`` / ``add_qkv_proj`` as plain quantised linears (NVFP4: e2m1 codes, e4m3 scale per 16, per-channel scale and a
  per-tensor ``wtscale``), per-head RMSNorm on Q and K and the complex rotary multiply in torch (the reference does
  both outside its GEMM for this model), joint attention over ``[text; image]``, ``to_out`` / ``to_add_out``;
* the MLPs through ``fused_gelu_mlp``: for NVFP4 that is GEMM -> 16-bit tile -> quantizer with the GELU fused in (the
  reference's own sequence for NVFP4, nunchaku/ops/triton/gemm_w4a4.py:1298-1312).

Every quantised layer runs on this package's kernels (the NVFP4 GEMMs on ``tcgen05.mma kind::mxf4nvf4``).  LayerNorms,
RMSNorms, rotary arithmetic, gating and residuals are torch, as in the reference (diffusers layers).  Weights are seeded
random tensors of the benchmark configuration's format; there are no checkpoints offline.
"""

from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.dispatch import scaled_dot_product_attention
from ..ops.elementwise import gated_residual, layernorm_modulate
from ..ops.fused import fused_gelu_mlp, fused_qkv_norm_rottary
from .flux_dit import _side_stream, join_modulations, modulations_ahead
from .linear import AWQW4A16Linear, SVDQW4A4Linear


@dataclass
class QwenDiTConfig:
    hidden: int = 3072
    heads: int = 24
    head_dim: int = 128
    mlp_ratio: int = 4
    n_blocks: int = 60
    rank: int = 32
    in_channels: int = 64
    text_dim: int = 3584       # Qwen2.5-VL hidden size
    dtype: torch.dtype = torch.bfloat16


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rotate(x: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """``apply_rotary_emb_qwen(..., use_real=False)``: channel pairs as complex numbers times ``freqs (S, D/2)`` complex."""
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    return torch.view_as_real(xc * freqs[None, :, None, :]).flatten(3).to(x.dtype)


def rotary_table(freqs: torch.Tensor) -> torch.Tensor:
    """Complex unit rotations ``(S, D / 2)`` as the fp32 ``(S, D / 2, 1, 2)`` table of (sin, cos) pairs that the fused
    Q/K epilogue reads (a table already in that form passes through)."""
    if not freqs.is_complex():
        return freqs
    return torch.stack([freqs.imag, freqs.real], dim=-1)[:, :, None, :].float().contiguous()


class _Modulation(nn.Module):
    def __init__(self, dim: int, dtype, device):
        super().__init__()
        self.linear = AWQW4A16Linear(dim, 6 * dim, bias=True, group_size=64, torch_dtype=dtype, device=device)

    def forward(self, temb):
        m = self.linear(F.silu(temb))
        m = m.view(m.shape[0], -1, 6).transpose(1, 2).reshape(m.shape[0], -1)  # [B, dim * 6] interleaved -> [B, 6 * dim]
        return m.chunk(2, dim=-1)


class _FeedForward(nn.Module):
    def __init__(self, cfg: QwenDiTConfig, device):
        super().__init__()
        h, m = cfg.hidden, cfg.hidden * cfg.mlp_ratio
        kw = dict(rank=cfg.rank, precision="nvfp4", torch_dtype=cfg.dtype, device=device)
        self.fc1, self.fc2 = SVDQW4A4Linear(h, m, **kw), SVDQW4A4Linear(m, h, **kw)

    def forward(self, x):
        return fused_gelu_mlp(x, self.fc1, self.fc2)


class QwenBlock(nn.Module):
    def __init__(self, cfg: QwenDiTConfig, device):
        super().__init__()
        h, T = cfg.hidden, cfg.dtype
        self.cfg = cfg
        kw = dict(rank=cfg.rank, precision="nvfp4", torch_dtype=T, device=device)
        self.img_mod, self.txt_mod = _Modulation(h, T, device), _Modulation(h, T, device)
        self.to_qkv, self.add_qkv_proj = SVDQW4A4Linear(h, 3 * h, **kw), SVDQW4A4Linear(h, 3 * h, **kw)
        self.to_out, self.to_add_out = SVDQW4A4Linear(h, h, **kw), SVDQW4A4Linear(h, h, **kw)
        for name in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            self.register_parameter(name, nn.Parameter(torch.ones(cfg.head_dim, dtype=T, device=device), requires_grad=False))
        self.img_mlp, self.txt_mlp = _FeedForward(cfg, device), _FeedForward(cfg, device)

    @staticmethod
    def _modulate(x, mod):
        """LayerNorm (no affine) of ``x``, ``* (1 + scale) + shift`` in one pass; returns it and the gate ``(B, dim)``."""
        shift, scale, gate = mod.chunk(3, dim=-1)
        return layernorm_modulate(x, scale, shift, scale_add=1.0), gate

    def forward(self, hidden_states, encoder_hidden_states, temb, img_freqs, txt_freqs, mods=None):
        cfg = self.cfg
        B, S_img, C = hidden_states.shape
        S_txt = encoder_hidden_states.shape[1]
        img_freqs, txt_freqs = rotary_table(img_freqs), rotary_table(txt_freqs)  # (no-op when the model already did it)
        # The text stream of a block (256 tokens: small launches that fill a fraction of the GPU) runs on a second CUDA
        # stream beside the image stream; the two meet at the joint attention and at the end of the block.  Every tensor
        # that crosses streams is a local of this function, so it outlives the join that follows its last use.
        main = torch.cuda.current_stream(hidden_states.device)
        side = _side_stream(hidden_states.device)  # (shared with the FLUX blocks)
        nq, nk, naq, nak = (SimpleNamespace(weight=w) for w in (self.norm_q, self.norm_k, self.norm_added_q, self.norm_added_k))
        qkv = txt_qkv = None
        if B == 1:
            qkv = torch.empty(1, S_txt + S_img, 3 * C, dtype=hidden_states.dtype, device=hidden_states.device)

        side.wait_stream(main)
        with torch.cuda.stream(side):
            txt_mod1, txt_mod2 = mods[1] if mods is not None else self.txt_mod(temb)
            txt_m, txt_gate1 = self._modulate(encoder_hidden_states, txt_mod1)
            # joint attention over [text; image]: both projections write their rows of one buffer, per-head RMSNorm + RoPE
            # of Q and K run in the projection's epilogue
            if B == 1:
                fused_qkv_norm_rottary(txt_m, self.add_qkv_proj, naq, nak, txt_freqs, output=qkv[0, :S_txt])
            else:
                txt_qkv = fused_qkv_norm_rottary(txt_m, self.add_qkv_proj, naq, nak, txt_freqs)
        img_mod1, img_mod2 = mods[0] if mods is not None else self.img_mod(temb)
        img_m, img_gate1 = self._modulate(hidden_states, img_mod1)
        if B == 1:
            fused_qkv_norm_rottary(img_m, self.to_qkv, nq, nk, img_freqs, output=qkv[0, S_txt:])
        main.wait_stream(side)
        if B != 1:
            qkv = torch.cat([txt_qkv, fused_qkv_norm_rottary(img_m, self.to_qkv, nq, nk, img_freqs)], dim=1)
        q, k, v = (t.view(B, S_txt + S_img, cfg.heads, cfg.head_dim).transpose(1, 2) for t in qkv.chunk(3, dim=-1))
        attn = scaled_dot_product_attention(q, k, v).transpose(1, 2).flatten(2, 3)  # (B, S, H D)

        side.wait_stream(main)
        with torch.cuda.stream(side):
            txt_attn = self.to_add_out(attn[:, :S_txt])
            txt_states = gated_residual(encoder_hidden_states, txt_gate1, txt_attn)
            txt_m2, txt_gate2 = self._modulate(txt_states, txt_mod2)
            txt_out = gated_residual(txt_states, txt_gate2, self.txt_mlp(txt_m2))
        img_attn = self.to_out(attn[:, S_txt:])
        hidden_states = gated_residual(hidden_states, img_gate1, img_attn)
        img_m2, img_gate2 = self._modulate(hidden_states, img_mod2)
        hidden_states = gated_residual(hidden_states, img_gate2, self.img_mlp(img_m2))
        main.wait_stream(side)
        encoder_hidden_states = txt_out
        return encoder_hidden_states, hidden_states


class QwenDiT(nn.Module):
    def __init__(self, cfg: QwenDiTConfig | None = None, device="cuda"):
        super().__init__()
        cfg = cfg or QwenDiTConfig()
        self.cfg = cfg
        h, T = cfg.hidden, cfg.dtype
        mk = lambda i, o: nn.Linear(i, o, bias=True, dtype=T, device=device)
        self.img_in, self.txt_in = mk(cfg.in_channels, h), mk(cfg.text_dim, h)
        self.time_in = nn.Sequential(mk(256, h), nn.SiLU(), mk(h, h))
        self.blocks = nn.ModuleList(QwenBlock(cfg, device) for _ in range(cfg.n_blocks))
        self.norm_out_linear, self.proj_out = mk(h, 2 * h), mk(h, cfg.in_channels)

    @torch.no_grad()
    def random_init(self, seed: int = 0) -> "QwenDiT":
        """Seeded NVFP4 weights: random e2m1 codes, e4m3 scales per 16 in U(0.01, 0.06) / sqrt(in / 3072), per-channel scales
        U(0.5, 1), ``wtscale`` 0.05, rank-32 branches N(0, 0.02); AWQ modulation with small scales so gates stay O(0.1)."""
        dev = self.proj_out.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        T = self.cfg.dtype
        for m in self.modules():
            if isinstance(m, SVDQW4A4Linear):
                cin = m.in_features
                m.qweight.copy_(torch.randint(-128, 128, m.qweight.shape, dtype=torch.int8, generator=g, device=dev))
                ws = (torch.rand(m.wscales.shape, generator=g, device=dev) * 0.05 + 0.01) / (cin / 3072) ** 0.5
                m.wscales.copy_(ws.to(torch.float8_e4m3fn))
                m.wcscales.copy_((torch.rand(m.out_features, generator=g, device=dev) * 0.5 + 0.5).to(T))
                m.wtscale = 0.05
                m.bias.copy_((torch.randn(m.out_features, generator=g, device=dev) * 0.02).to(T))
                m.smooth_factor.copy_((torch.rand(cin, generator=g, device=dev) + 0.5).to(T))
                m.proj_down.copy_((torch.randn(cin, m.rank, generator=g, device=dev) * 0.02).to(T))
                m.proj_up.copy_((torch.randn(m.out_features, m.rank, generator=g, device=dev) * 0.02).to(T))
            elif isinstance(m, AWQW4A16Linear):
                m.qweight.copy_(torch.randint(-(2**31), 2**31 - 1, m.qweight.shape, dtype=torch.int32, generator=g, device=dev))
                m.wscales.copy_((torch.rand(m.wscales.shape, generator=g, device=dev) * 0.002 + 0.0005).to(T))
                m.wzeros.copy_((torch.randn(m.wzeros.shape, generator=g, device=dev) * 0.005).to(T))
                m.bias.copy_((torch.randn(m.out_features, generator=g, device=dev) * 0.02).to(T))
            elif isinstance(m, nn.Linear):
                m.weight.copy_((torch.randn(m.weight.shape, generator=g, device=dev) / m.in_features**0.5).to(T))
                m.bias.copy_((torch.randn(m.bias.shape, generator=g, device=dev) * 0.02).to(T))
            elif isinstance(m, QwenBlock):
                for name in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
                    getattr(m, name).copy_((1 + torch.randn(m.cfg.head_dim, generator=g, device=dev) * 0.05).to(T))
        return self

    def quantized_bytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.parameters())

    @staticmethod
    def rotary_freqs(n: int, head_dim: int, device, theta: float = 10000.0) -> torch.Tensor:
        """Complex ``(n, head_dim / 2)`` unit rotations for positions 0..n-1 (a 1-D stand-in for the model's 3-axis table)."""
        inv = 1.0 / theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim)
        ang = torch.arange(n, dtype=torch.float32, device=device)[:, None] * inv[None]
        return torch.polar(torch.ones_like(ang), ang)

    def forward(self, hidden_states, encoder_hidden_states, timestep, img_freqs, txt_freqs):
        from .flux_dit import _timestep_embedding

        cfg = self.cfg
        h = self.img_in(hidden_states)
        e = self.txt_in(encoder_hidden_states)
        temb = self.time_in(_timestep_embedding(timestep * 1000.0).to(cfg.dtype))
        img_freqs, txt_freqs = rotary_table(img_freqs), rotary_table(txt_freqs)
        main = torch.cuda.current_stream(temb.device)
        mods = modulations_ahead(temb, [lambda t, b=b: (b.img_mod(t), b.txt_mod(t)) for b in self.blocks])
        for i, blk in enumerate(self.blocks):
            main.wait_event(mods[i][1])
            e, h = blk(h, e, temb, img_freqs, txt_freqs, mods[i][0])
        join_modulations(temb.device)
        scale, shift = self.norm_out_linear(F.silu(temb)).chunk(2, dim=1)
        h = layernorm_modulate(h, scale, shift, scale_add=1.0)
        return self.proj_out(h)


class GraphedQwenStep:
    """One forward of :class:`QwenDiT` captured in a CUDA graph with static buffers (build after one eager run)."""

    def __init__(self, model: QwenDiT, batch: int, img_tokens: int = 6889, txt_tokens: int = 256, seed: int = 0):
        cfg, dev = model.cfg, model.proj_out.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        self.model = model
        self.latents = torch.randn(batch, img_tokens, cfg.in_channels, generator=g, device=dev).to(cfg.dtype)
        self.text = torch.randn(batch, txt_tokens, cfg.text_dim, generator=g, device=dev).to(cfg.dtype)
        self.timestep = torch.ones(batch, device=dev)
        self.img_freqs = model.rotary_freqs(img_tokens, cfg.head_dim, dev)
        self.txt_freqs = model.rotary_freqs(txt_tokens, cfg.head_dim, dev)
        with torch.no_grad():
            for _ in range(2):
                self._forward()
            torch.cuda.synchronize(dev)
            self.graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side), torch.cuda.graph(self.graph, stream=side):
                self.out = self._forward()
            torch.cuda.current_stream(dev).wait_stream(side)

    def _forward(self):
        return self.model(self.latents, self.text, self.timestep, self.img_freqs, self.txt_freqs)

    def step(self, latents=None, t: float | None = None):
        if latents is not None:
            self.latents.copy_(latents, non_blocking=True)
        if t is not None:
            self.timestep.fill_(t)
        self.graph.replay()
        return self.out

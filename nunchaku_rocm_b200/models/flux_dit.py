"""
FLUX.1-architecture DiT assembled from this package's operators: the block wiring of the reference's
``NunchakuFluxTransformer2DModelV2`` (nunchaku/models/transformers/transformer_flux_v2.py) with its quantised layers,

* ``FluxDoubleBlock``  = ``NunchakuFluxTransformerBlock.forward``        (:174-258): adaLN-Zero (AWQ W4A16 modulation,
  interleaved ``[dim, 6]`` output, ``scale + 1``), fused QKV + RMSNorm + RoPE for both streams, joint attention over
  ``[text; image]``, output projections, LayerNorm + modulation, fused GELU MLP, gated residuals;
* ``FluxSingleBlock``  = ``NunchakuFluxSingleTransformerBlock.forward``  (:291-343): adaLN-Zero-single, fused GELU MLP and
  attention on the same normalised input, ``to_out(attn) + mlp``, gated residual;
* ``FluxDiT.forward``  = the model's forward                            (:437-576): embedders, rotary table for
  ``[txt_ids; img_ids]``, 19 double + 38 single blocks, adaLN-continuous + output projection.

Every W4A4 / AWQ layer is a ``SVDQW4A4Linear`` / ``AWQW4A16Linear`` of this package and runs on its CUDA kernels.  What the
reference takes from diffusers (the timestep / pooled-text embedder, ``x_embedder``, ``context_embedder``, the LayerNorms
and the final ``AdaLayerNormContinuous``) are plain torch layers of the same shapes here: diffusers is not a dependency of
this package, and they are outside the quantised path (under 1 % of a step's arithmetic).

There are no checkpoints offline, so :meth:`FluxDiT.random_init` fills all 57 blocks with DISTINCT seeded int4 weights of
the benchmark configuration's distributions.  :class:`GraphedStep` captures one forward in a CUDA graph (the eager
step is bound by launch overhead: about 900 kernel launches) and :func:`denoise` runs the flow-matching Euler loop a
pipeline would run around it.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.dispatch import scaled_dot_product_attention
from ..ops.elementwise import gated_residual, layernorm_modulate
from ..ops.fused import fused_gelu_mlp, fused_qkv_norm_rottary
from .embeddings import flux_image_ids, flux_pos_embed
from .linear import AWQW4A16Linear, SVDQW4A4Linear


@dataclass
class FluxDiTConfig:
    """FLUX.1-schnell transformer shapes (diffusers ``FluxTransformer2DModel`` defaults the reference wraps)."""

    hidden: int = 3072
    heads: int = 24
    head_dim: int = 128
    mlp_ratio: int = 4
    n_double: int = 19
    n_single: int = 38
    rank: int = 32
    in_channels: int = 64       # 16 latent channels packed 2 x 2
    text_dim: int = 4096        # T5 hidden size
    pooled_dim: int = 768       # CLIP pooled embedding
    axes_dim: tuple = (16, 56, 56)
    theta: int = 10000
    dtype: torch.dtype = torch.bfloat16


class _HeadRMSNorm(nn.Module):
    """Per-head RMSNorm weight; the fused QKV epilogue only reads ``.weight`` (eps 1e-6)."""

    def __init__(self, dim: int, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device), requires_grad=False)
        self.eps = 1e-6


class _AdaLayerNormZero(nn.Module):
    """``NunchakuAdaLayerNormZero`` / ``...Single`` (nunchaku/models/normalization.py:60-159): AWQ modulation linear whose
    output rows are interleaved ``[dim, n]``, LayerNorm without affine, ``scale + scale_shift``."""

    def __init__(self, dim: int, n: int, dtype, device, scale_shift: float = 1.0):
        super().__init__()
        self.n, self.dim, self.scale_shift = n, dim, scale_shift
        self.linear = AWQW4A16Linear(dim, n * dim, bias=True, group_size=64, torch_dtype=dtype, device=device)

    def modulation(self, emb: torch.Tensor) -> torch.Tensor:
        """The ``(n, B, dim)`` modulation vectors: they depend on the time embedding only, so a model may compute every
        block's ahead of the blocks (:func:`modulations_ahead`)."""
        e = self.linear(F.silu(emb))
        # (n, B, dim), contiguous along dim: the element-wise kernels then read the vectors 16 bytes at a time
        return e.view(e.shape[0], -1, self.n).permute(2, 0, 1).contiguous()

    def forward(self, x: torch.Tensor, emb: torch.Tensor, parts: torch.Tensor | None = None):
        if parts is None:
            parts = self.modulation(emb)
        # LayerNorm (no affine) * (scale + scale_shift) + shift in one pass; the second modulation's scale comes back without
        # its scale_shift, which the block's own layernorm_modulate call adds
        norm = layernorm_modulate(x, parts[1], parts[0], scale_add=self.scale_shift)
        if self.n == 3:
            return norm, parts[2]
        return norm, parts[2], parts[3], parts[4], parts[5]


class _FeedForward(nn.Module):
    """``NunchakuFeedForward``: fc1 -> GELU(tanh) -> fc2 with fc2's activations unsigned (models/attention.py:99)."""

    def __init__(self, cfg: FluxDiTConfig, device):
        super().__init__()
        h, m = cfg.hidden, cfg.hidden * cfg.mlp_ratio
        self.fc1 = SVDQW4A4Linear(h, m, rank=cfg.rank, torch_dtype=cfg.dtype, device=device)
        self.fc2 = SVDQW4A4Linear(m, h, rank=cfg.rank, act_unsigned=True, torch_dtype=cfg.dtype, device=device)

    def forward(self, x):
        return fused_gelu_mlp(x, self.fc1, self.fc2)


_SIDE_STREAMS: dict = {}


def _side_stream(device, which: str = "text") -> "torch.cuda.Stream":
    """A further stream of a device (one per name, device and process): "text" carries a block's text stream (or a single
    block's MLP branch), "mod" the modulation vectors computed ahead of the blocks."""
    key = (torch.device(device).index, which)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device)
    return _SIDE_STREAMS[key]


def modulations_ahead(temb: torch.Tensor, per_block) -> list:
    """Every block's modulation vectors on a stream of their own, ahead of the blocks: they depend on ``temb`` only, and
    the small AWQ GEMVs and element-wise launches that make them would otherwise sit between the large kernels of each
    block.  ``per_block``: one callable per block, ``temb ->`` that block's modulation tensors.  Returns ``[(tensors,
    event)]``; the caller waits for a block's event before the block and keeps the list alive until it has joined the
    stream again (:func:`join_modulations`)."""
    main = torch.cuda.current_stream(temb.device)
    ms = _side_stream(temb.device, "mod")
    ms.wait_stream(main)
    out = []
    with torch.cuda.stream(ms):
        for fn in per_block:
            t = fn(temb)
            ev = torch.cuda.Event()
            ev.record(ms)
            out.append((t, ev))
    return out


def join_modulations(device) -> None:
    torch.cuda.current_stream(device).wait_stream(_side_stream(device, "mod"))


class FluxDoubleBlock(nn.Module):
    def __init__(self, cfg: FluxDiTConfig, device):
        super().__init__()
        h, T = cfg.hidden, cfg.dtype
        self.cfg = cfg
        self.norm1 = _AdaLayerNormZero(h, 6, T, device)
        self.norm1_context = _AdaLayerNormZero(h, 6, T, device)
        self.to_qkv = SVDQW4A4Linear(h, 3 * h, rank=cfg.rank, torch_dtype=T, device=device)
        self.add_qkv_proj = SVDQW4A4Linear(h, 3 * h, rank=cfg.rank, torch_dtype=T, device=device)
        self.norm_q, self.norm_k = _HeadRMSNorm(cfg.head_dim, T, device), _HeadRMSNorm(cfg.head_dim, T, device)
        self.norm_added_q, self.norm_added_k = _HeadRMSNorm(cfg.head_dim, T, device), _HeadRMSNorm(cfg.head_dim, T, device)
        self.to_out = SVDQW4A4Linear(h, h, rank=cfg.rank, torch_dtype=T, device=device)
        self.to_add_out = SVDQW4A4Linear(h, h, rank=cfg.rank, torch_dtype=T, device=device)
        self.ff, self.ff_context = _FeedForward(cfg, device), _FeedForward(cfg, device)

    def forward(self, hidden_states, encoder_hidden_states, temb, rotary_img, rotary_txt, mods=None):
        cfg = self.cfg
        mod_img, mod_txt = mods if mods is not None else (None, None)
        B, S_img, _ = hidden_states.shape
        S_txt = encoder_hidden_states.shape[1]
        # The text stream of a block (512 tokens per image: launches that fill a fraction of the GPU) runs on a second
        # CUDA stream beside the image stream; the two meet at the joint attention and at the end of the block.  Every
        # tensor that crosses streams is a local of this function, so it outlives the join that follows its last use.
        main = torch.cuda.current_stream(hidden_states.device)
        side = _side_stream(hidden_states.device)
        qkv = txt_qkv = None
        if B == 1:
            # both projections write their rows of one buffer: the concatenation of the reference without the copy
            qkv = torch.empty(1, S_txt + S_img, 3 * cfg.hidden, dtype=hidden_states.dtype, device=hidden_states.device)

        # joint attention over [text; image] (attention_processors/flux.py:71-110)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            norm_e, c_gate_msa, c_shift_mlp, c_scale_mlp, c_gate_mlp = self.norm1_context(encoder_hidden_states, temb, mod_txt)
            if B == 1:
                fused_qkv_norm_rottary(norm_e, self.add_qkv_proj, self.norm_added_q, self.norm_added_k, rotary_txt, output=qkv[0, :S_txt])
            else:
                txt_qkv = fused_qkv_norm_rottary(norm_e, self.add_qkv_proj, self.norm_added_q, self.norm_added_k, rotary_txt)
        norm_h, gate_msa, shift_mlp, scale_mlp, gate_mlp = self.norm1(hidden_states, temb, mod_img)
        if B == 1:
            fused_qkv_norm_rottary(norm_h, self.to_qkv, self.norm_q, self.norm_k, rotary_img, output=qkv[0, S_txt:])
        main.wait_stream(side)
        if B != 1:
            qkv = torch.cat([txt_qkv, fused_qkv_norm_rottary(norm_h, self.to_qkv, self.norm_q, self.norm_k, rotary_img)], dim=1)
        attn_all = _attention(qkv, cfg)

        ss = self.norm1.scale_shift
        side.wait_stream(main)
        with torch.cuda.stream(side):
            context_attn = self.to_add_out(attn_all[:, :S_txt])
            txt_states = gated_residual(encoder_hidden_states, c_gate_msa, context_attn)
            norm_e2 = layernorm_modulate(txt_states, c_scale_mlp, c_shift_mlp, scale_add=ss)
            txt_out = gated_residual(txt_states, c_gate_mlp, self.ff_context(norm_e2))
        attn = self.to_out(attn_all[:, S_txt:])
        hidden_states = gated_residual(hidden_states, gate_msa, attn)
        norm_h = layernorm_modulate(hidden_states, scale_mlp, shift_mlp, scale_add=ss)
        hidden_states = gated_residual(hidden_states, gate_mlp, self.ff(norm_h))
        main.wait_stream(side)
        encoder_hidden_states = txt_out
        return encoder_hidden_states, hidden_states


class FluxSingleBlock(nn.Module):
    def __init__(self, cfg: FluxDiTConfig, device):
        super().__init__()
        h, T = cfg.hidden, cfg.dtype
        self.cfg = cfg
        self.norm = _AdaLayerNormZero(h, 3, T, device)
        self.mlp_fc1 = SVDQW4A4Linear(h, h * cfg.mlp_ratio, rank=cfg.rank, torch_dtype=T, device=device)
        self.mlp_fc2 = SVDQW4A4Linear(h * cfg.mlp_ratio, h, rank=cfg.rank, act_unsigned=True, torch_dtype=T, device=device)
        self.to_qkv = SVDQW4A4Linear(h, 3 * h, rank=cfg.rank, torch_dtype=T, device=device)
        self.norm_q, self.norm_k = _HeadRMSNorm(cfg.head_dim, T, device), _HeadRMSNorm(cfg.head_dim, T, device)
        self.to_out = SVDQW4A4Linear(h, h, rank=cfg.rank, torch_dtype=T, device=device)

    def forward(self, hidden_states, temb, rotary, mods=None):
        residual = hidden_states
        norm_h, gate = self.norm(hidden_states, temb, mods)
        # the MLP branch and the attention branch meet only in the final sum: the MLP runs on the second stream, so the
        # partly filled last waves of one branch's kernels overlap the other's
        main = torch.cuda.current_stream(hidden_states.device)
        side = _side_stream(hidden_states.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            mlp = fused_gelu_mlp(norm_h, self.mlp_fc1, self.mlp_fc2)
        qkv = fused_qkv_norm_rottary(norm_h, self.to_qkv, self.norm_q, self.norm_k, rotary)
        attn = self.to_out(_attention(qkv, self.cfg))
        main.wait_stream(side)
        return gated_residual(residual, gate, attn, mlp)


def _attention(qkv: torch.Tensor, cfg: FluxDiTConfig) -> torch.Tensor:
    """``(B, S, 3 H D)`` fused projection -> ``(B, S, H D)``: q, k, v are strided views, the kernel writes (B, S, H D)."""
    B, S, _ = qkv.shape
    q, k, v = (t.view(B, S, cfg.heads, cfg.head_dim).transpose(1, 2) for t in qkv.chunk(3, dim=-1))
    o = scaled_dot_product_attention(q, k, v)  # (B, H, S, D) view of a (B, S, H D) buffer
    return o.transpose(1, 2).reshape(B, S, cfg.heads * cfg.head_dim)


def _timestep_embedding(t: torch.Tensor, dim: int = 256) -> torch.Tensor:
    """Sinusoidal embedding of ``t (B,)`` (flip_sin_to_cos, max period 10000), fp32."""
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


class FluxDiT(nn.Module):
    def __init__(self, cfg: FluxDiTConfig | None = None, device="cuda"):
        super().__init__()
        cfg = cfg or FluxDiTConfig()
        self.cfg = cfg
        h, T = cfg.hidden, cfg.dtype
        mk = lambda i, o: nn.Linear(i, o, bias=True, dtype=T, device=device)
        self.x_embedder = mk(cfg.in_channels, h)
        self.context_embedder = mk(cfg.text_dim, h)
        self.time_in = nn.Sequential(mk(256, h), nn.SiLU(), mk(h, h))           # timestep embedder
        self.text_in = nn.Sequential(mk(cfg.pooled_dim, h), nn.SiLU(), mk(h, h))  # pooled-text embedder
        self.transformer_blocks = nn.ModuleList(FluxDoubleBlock(cfg, device) for _ in range(cfg.n_double))
        self.single_transformer_blocks = nn.ModuleList(FluxSingleBlock(cfg, device) for _ in range(cfg.n_single))
        self.norm_out_linear = mk(h, 2 * h)  # AdaLayerNormContinuous
        self.proj_out = mk(h, cfg.in_channels)

    # ---- weights ------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def random_init(self, seed: int = 0) -> "FluxDiT":
        """Seeded random weights, different for every layer: int4 codes U[-8, 7], per-64 scales U(0.005, 0.02) scaled by
        1 / sqrt(in / 3072), rank-32 branches N(0, 0.02), smooth U(0.5, 1.5), RMSNorm weights 1 + N(0, 0.05); AWQ modulation
        codes U[0, 15] with small scales so that gates and shifts stay O(0.1) and the residual stream stays finite."""
        dev = self.proj_out.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        T = self.cfg.dtype
        for m in self.modules():
            if isinstance(m, SVDQW4A4Linear):
                cin = m.in_features
                m.qweight.copy_(torch.randint(-128, 128, m.qweight.shape, dtype=torch.int8, generator=g, device=dev))
                m.wscales.copy_(((torch.rand(m.wscales.shape, generator=g, device=dev) * 0.015 + 0.005) / (cin / 3072) ** 0.5).to(T))
                m.bias.copy_((torch.randn(m.out_features, generator=g, device=dev) * 0.02).to(T))
                m.smooth_factor.copy_((torch.rand(cin, generator=g, device=dev) + 0.5).to(T))
                m.smooth_factor_orig.copy_(m.smooth_factor)
                m.proj_down.copy_((torch.randn(cin, m.rank, generator=g, device=dev) * 0.02).to(T))
                m.proj_up.copy_((torch.randn(m.out_features, m.rank, generator=g, device=dev) * 0.02).to(T))
            elif isinstance(m, AWQW4A16Linear):
                m.qweight.copy_(torch.randint(-(2**31), 2**31 - 1, m.qweight.shape, dtype=torch.int32, generator=g, device=dev))
                m.wscales.copy_((torch.rand(m.wscales.shape, generator=g, device=dev) * 0.002 + 0.0005).to(T))
                m.wzeros.copy_((torch.randn(m.wzeros.shape, generator=g, device=dev) * 0.005).to(T))
                m.bias.copy_((torch.randn(m.out_features, generator=g, device=dev) * 0.02).to(T))
            elif isinstance(m, _HeadRMSNorm):
                m.weight.copy_((1 + torch.randn(m.weight.shape, generator=g, device=dev) * 0.05).to(T))
            elif isinstance(m, nn.Linear):
                m.weight.copy_((torch.randn(m.weight.shape, generator=g, device=dev) / m.in_features**0.5).to(T))
                m.bias.copy_((torch.randn(m.bias.shape, generator=g, device=dev) * 0.02).to(T))
        return self

    def quantized_bytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.parameters())

    # ---- forward ------------------------------------------------------------------------------------------------------
    def rotary_tables(self, txt_ids: torch.Tensor, img_ids: torch.Tensor):
        """``image_rotary_emb`` in the natural layout, split as the reference's forward does (:515-537)."""
        ids = torch.cat((txt_ids, img_ids), dim=0)
        rot = flux_pos_embed(ids, self.cfg.axes_dim, self.cfg.theta)  # (S, 64, 1, 2) fp32
        n_txt = txt_ids.shape[0]
        return rot[:n_txt].contiguous(), rot[n_txt:].contiguous(), rot

    def embed_time(self, timestep: torch.Tensor, pooled: torch.Tensor) -> torch.Tensor:
        t = _timestep_embedding(timestep * 1000.0).to(self.cfg.dtype)
        return self.time_in(t) + self.text_in(pooled)

    def forward(self, hidden_states, encoder_hidden_states, pooled_projections, timestep, img_ids, txt_ids, rotary=None):
        """``hidden_states (B, S_img, 64)``, ``encoder_hidden_states (B, S_txt, 4096)``, ``pooled_projections (B, 768)``,
        ``timestep (B,)`` in [0, 1] -> ``(B, S_img, 64)``.  ``rotary`` may carry precomputed :meth:`rotary_tables`."""
        cfg = self.cfg
        hidden_states = self.x_embedder(hidden_states)
        temb = self.embed_time(timestep, pooled_projections)
        encoder_hidden_states = self.context_embedder(encoder_hidden_states)
        rot_txt, rot_img, rot_all = rotary if rotary is not None else self.rotary_tables(txt_ids, img_ids)
        n_txt = encoder_hidden_states.shape[1]
        main = torch.cuda.current_stream(temb.device)
        mods = modulations_ahead(
            temb,
            [lambda t, b=b: (b.norm1.modulation(t), b.norm1_context.modulation(t)) for b in self.transformer_blocks]
            + [lambda t, b=b: b.norm.modulation(t) for b in self.single_transformer_blocks])
        nd = len(self.transformer_blocks)
        for i, block in enumerate(self.transformer_blocks):
            main.wait_event(mods[i][1])
            encoder_hidden_states, hidden_states = block(hidden_states, encoder_hidden_states, temb, rot_img, rot_txt, mods[i][0])
        hidden_states = torch.cat([encoder_hidden_states, hidden_states], dim=1)
        for i, block in enumerate(self.single_transformer_blocks):
            main.wait_event(mods[nd + i][1])
            hidden_states = block(hidden_states, temb, rot_all, mods[nd + i][0])
        join_modulations(temb.device)
        hidden_states = hidden_states[:, n_txt:]
        scale, shift = self.norm_out_linear(F.silu(temb)).chunk(2, dim=1)
        hidden_states = layernorm_modulate(hidden_states, scale, shift, scale_add=1.0)
        return self.proj_out(hidden_states)


class GraphedStep:
    """
    One transformer forward captured in a CUDA graph with static input / output buffers.  ``step(latents, t)`` copies
    the latents and the timestep in, replays, and returns the static output (valid until the next call).
    Build it after the model has run once eagerly (weight preparation and the library self-test happen there).
    """

    def __init__(self, model: FluxDiT, batch: int, txt_tokens: int = 512, grid: int = 64, seed: int = 0):
        cfg, dev = model.cfg, model.proj_out.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        T = cfg.dtype
        self.model = model
        self.latents = torch.randn(batch, grid * grid, cfg.in_channels, generator=g, device=dev).to(T)
        self.text = torch.randn(batch, txt_tokens, cfg.text_dim, generator=g, device=dev).to(T)
        self.pooled = torch.randn(batch, cfg.pooled_dim, generator=g, device=dev).to(T)
        self.timestep = torch.ones(batch, device=dev)
        ids = flux_image_ids(txt_tokens, grid, grid, device=dev)
        self.txt_ids, self.img_ids = ids[:txt_tokens], ids[txt_tokens:]
        self.rotary = model.rotary_tables(self.txt_ids, self.img_ids)
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
        return self.model(self.latents, self.text, self.pooled, self.timestep, self.img_ids, self.txt_ids, rotary=self.rotary)

    def step(self, latents: torch.Tensor | None = None, t: float | None = None) -> torch.Tensor:
        if latents is not None:
            self.latents.copy_(latents, non_blocking=True)
        if t is not None:
            self.timestep.fill_(t)
        self.graph.replay()
        return self.out


def denoise(step: GraphedStep, latents: torch.Tensor, num_steps: int = 4) -> torch.Tensor:
    """Flow-matching Euler loop of a FLUX.1-schnell pipeline around the transformer: ``x += (t_next - t) * v(x, t)``."""
    ts = torch.linspace(1.0, 0.0, num_steps + 1).tolist()
    x = latents
    for i in range(num_steps):
        v = step.step(x, ts[i])
        x = x + (ts[i + 1] - ts[i]) * v
    return x

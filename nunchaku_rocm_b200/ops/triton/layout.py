"""
Checkpoint layout converter: SVDQuant checkpoints store ``qweight / wscales / bias / smooth_factor / wcscales /
proj_down / proj_up`` in the register-fragment order of the upstream CUDA kernel's ``mma.m16n8k32``; the kernels
here read natural row-major tensors.  This module maps one to the other, once, on the host, with the function
names of the reference's ``nunchaku/ops/triton/layout.py`` (:36-292) and, for the forward direction, of
``NunchakuWeightPacker`` (nunchaku/lora/flux/packer.py:187-398).

Every mapping is written as an index formula -- "logical element (n, k) lives at flat position f(n, k) of the
stored tensor" -- and applied with one gather (unpack) or scatter (pack):

* weight, 4-bit (packer.py:187-239): word ``((((nt*KT + kt)*8 + npk)*8 + nl)*4 + kl)*2 + nps)*2 + kps`` of the
  int32 view, nibble ``rk``, holds ``n = ((nt*8 + npk)*2 + nps)*8 + nl``, ``k = kt*64 + kps*32 + kl*8 + rk``.
* 16-bit scale per 128 channels (packer.py:241-301): channel ``((l8*2 + p2)*4 + l4)*2 + e2`` sits at position
  ``((l8*4 + l4)*2 + p2)*2 + e2`` of its (block, group) row.
* NVFP4 micro scale (packer.py:303-360): channel ``(ps*4 + a4)*8 + b8``, group ``4*x + kg`` sits at
  ``((b8*4 + a4)*4 + ps)*4 + kg`` of its (block, x) row of 512.
* low-rank factors in 16 x 16 blocks (packer.py:362-398): element ``(i = nps*8 + nl, j = kps*8 + kl*2 + rk)`` sits
  at ``((((nl*4 + kl)*2 + nps)*2 + kps)*2 + rk``.
"""

from __future__ import annotations

import torch

__all__ = [
    "unpack_weight",
    "unpack_weight_packed_nibbles",
    "unpack_scale",
    "unpack_lowrank_weight",
    "pack_weight",
    "pack_scale",
    "pack_lowrank_weight",
    "convert_svdq_linear_to_natural_layout",
]

WARP_N = 128


# ------------------------------------------------------------------------------------------------
# index maps
# ------------------------------------------------------------------------------------------------
def _weight_map(n: int, k: int, device):
    """(word index, nibble) of every logical (n, k) in the int32 view of the stored weight."""
    assert n % 128 == 0 and k % 128 == 0, f"n ({n}) and k ({k}) must be multiples of 128"
    nn = torch.arange(n, device=device)[:, None]
    kk = torch.arange(k, device=device)[None, :]
    nt, npk, nps, nl = nn // 128, (nn // 16) % 8, (nn // 8) % 2, nn % 8
    kt, kps, kl, rk = kk // 64, (kk // 32) % 2, (kk // 8) % 4, kk % 8
    word = (((((nt * (k // 64) + kt) * 8 + npk) * 8 + nl) * 4 + kl) * 2 + nps) * 2 + kps
    return word, rk.expand(n, k)


def _scale_pos(n: int, device):
    """Stored position inside its 128-block of every channel, for 16-bit scales / bias / smooth / wcscales."""
    c = torch.arange(n, device=device) % 128
    l8, p2, l4, e2 = c // 16, (c // 8) % 2, (c // 2) % 4, c % 2
    return ((l8 * 4 + l4) * 2 + p2) * 2 + e2


def _micro_map(n: int, groups: int, device):
    """Flat stored index of every (channel, 16-group) of an NVFP4 micro-scale tensor."""
    assert groups % 4 == 0
    c = torch.arange(n, device=device)[:, None]
    g = torch.arange(groups, device=device)[None, :]
    blk, cl = c // 128, c % 128
    ps, a4, b8 = cl // 32, (cl // 8) % 4, cl % 8
    x, kg = g // 4, g % 4
    return (blk * (groups // 4) + x) * 512 + ((b8 * 4 + a4) * 4 + ps) * 4 + kg


def _lowrank_map(rows_n: int, cols_k: int, block_major_k: bool, device):
    """
    Flat stored index of element (i, j) of a matrix whose rows play the "n" role and columns the "k" role of the
    16 x 16 fragment blocks.  Blocks are ordered (k-block outer, n-block inner) for the down projection and
    (n-block outer, k-block inner) for the up projection.
    """
    i = torch.arange(rows_n, device=device)[:, None]
    j = torch.arange(cols_k, device=device)[None, :]
    ib, il, jb, jl = i // 16, i % 16, j // 16, j % 16
    nps, nl = il // 8, il % 8
    kps, kl, rk = jl // 8, (jl // 2) % 4, jl % 2
    off = ((((nl * 4 + kl) * 2 + nps) * 2 + kps) * 2) + rk
    nb, kb = rows_n // 16, cols_k // 16
    blk = jb * nb + ib if block_major_k else ib * kb + jb
    return blk * 256 + off


# ------------------------------------------------------------------------------------------------
# unpack (checkpoint -> natural)
# ------------------------------------------------------------------------------------------------
def unpack_weight(packed: torch.Tensor, n: int, k: int, bits: int = 4) -> torch.Tensor:
    """Stored ``(n, k // 2)`` int8 -> logical codes ``(n, k)`` int32 in ``[0, 16)``."""
    assert bits == 4, "SVDQuant checkpoints are 4-bit"
    words = packed.contiguous().view(torch.int32).reshape(-1)
    word, nib = _weight_map(n, k, packed.device)
    return (words[word] >> (4 * nib).to(torch.int32)) & 0xF


def unpack_weight_packed_nibbles(packed: torch.Tensor, n: int, k: int, bits: int = 4) -> torch.Tensor:
    """
    As :func:`unpack_weight`, returned in the natural packed form ``(n, k // 2)`` uint8, even ``k`` in the low nibble.
    A tensor that sits on a CUDA device is converted there by ``layout_unpack_weight_kernel`` (a permutation of 32-bit
    words at HBM speed); on the host the index formula runs in torch.
    """
    assert bits == 4, "SVDQuant checkpoints are 4-bit"
    if packed.is_cuda:
        import ctypes as C

        from ... import _lib as L

        lib = L.lib()
        lib.nb_layout_unpack_weight.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_void_p]
        assert n % 128 == 0 and k % 128 == 0, f"n ({n}) and k ({k}) must be multiples of 128"
        src = packed.contiguous()
        assert src.numel() * src.element_size() == n * k // 2
        out = torch.empty(n, k // 2, dtype=torch.uint8, device=packed.device)
        with torch.cuda.device(packed.device):
            L.check(lib.nb_layout_unpack_weight(L.ptr(src), L.ptr(out), n, k, out.stride(0), L.stream_of(out)),
                    "unpack_weight_packed_nibbles")
        return out
    codes = unpack_weight(packed, n, k, bits)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8)


def unpack_scale(packed: torch.Tensor, n: int, group_size: int, bits: int = 4, warp_n: int = WARP_N) -> torch.Tensor:
    """
    Stored scales -> ``(k // group_size, n)`` (or ``(n,)`` for ``group_size == -1``: bias, smooth factor, per-channel
    scale).  ``group_size == 16`` with 4 bits is the NVFP4 micro-scale layout.
    """
    assert warp_n == WARP_N and n % 128 == 0
    flat = packed.contiguous().reshape(-1)
    if bits == 4 and group_size == 16:
        groups = flat.numel() // n
        return flat[_micro_map(n, groups, packed.device)].t().contiguous()
    groups = 1 if group_size == -1 else flat.numel() // n
    c = torch.arange(n, device=packed.device)
    pos = _scale_pos(n, packed.device)
    g = torch.arange(groups, device=packed.device)[:, None]
    out = flat[((c // 128)[None, :] * groups + g) * 128 + pos[None, :]]
    return out.reshape(n) if group_size == -1 else out.contiguous()


def unpack_lowrank_weight(weight: torch.Tensor, down: bool) -> torch.Tensor:
    """Stored low-rank factor ``(c, r)`` -> ``(rank, in)`` for ``down`` or ``(out, rank)`` for up."""
    c, r = weight.shape
    flat = weight.contiguous().reshape(-1)
    if down:
        return flat[_lowrank_map(r, c, True, weight.device)]  # rows = rank ("n" role), columns = in ("k" role)
    return flat[_lowrank_map(c, r, False, weight.device)]


# ------------------------------------------------------------------------------------------------
# pack (natural -> checkpoint): the forward direction, used to build synthetic checkpoints
# ------------------------------------------------------------------------------------------------
def pack_weight(codes: torch.Tensor) -> torch.Tensor:
    """Logical codes ``(n, k)`` int32 (any sign, low 4 bits kept) -> stored ``(n, k // 2)`` int8."""
    n, k = codes.shape
    word, nib = _weight_map(n, k, codes.device)
    words = torch.zeros(n * k // 8, dtype=torch.int64, device=codes.device)
    words.index_add_(0, word.reshape(-1), ((codes.to(torch.int64) & 0xF) << (4 * nib).to(torch.int64)).reshape(-1))
    words = torch.where(words >= 2**31, words - 2**32, words).to(torch.int32)
    return words.view(torch.int8).view(n, k // 2)


def pack_scale(scale: torch.Tensor, group_size: int) -> torch.Tensor:
    """Natural ``(groups, n)`` (or ``(n,)`` with ``group_size == -1``) -> stored order; group 16 casts to e4m3."""
    if group_size == -1:
        n, groups, nat = scale.numel(), 1, scale.reshape(1, -1)
    else:
        groups, n = scale.shape
        nat = scale
    if group_size == 16:
        nat = nat.to(torch.float8_e4m3fn)
        out = torch.empty(n * groups, dtype=nat.dtype, device=scale.device)
        out.view(torch.uint8)[_micro_map(n, groups, scale.device).reshape(-1)] = nat.t().contiguous().view(torch.uint8).reshape(-1)
        return out.view(-1, n)
    c = torch.arange(n, device=scale.device)
    g = torch.arange(groups, device=scale.device)[:, None]
    idx = ((c // 128)[None, :] * groups + g) * 128 + _scale_pos(n, scale.device)[None, :]
    out = torch.empty(n * groups, dtype=scale.dtype, device=scale.device)
    out[idx.reshape(-1)] = nat.reshape(-1)
    return out if group_size == -1 else out.view(-1, n)


def pack_lowrank_weight(weight: torch.Tensor, down: bool) -> torch.Tensor:
    """``(rank, in)`` for ``down`` / ``(out, rank)`` for up -> stored ``(c, r)``."""
    a, b = weight.shape
    idx = _lowrank_map(a, b, down, weight.device)
    out = torch.empty(a * b, dtype=weight.dtype, device=weight.device)
    out[idx.reshape(-1)] = weight.reshape(-1)
    return out.view(b, a) if down else out.view(a, b)


# ------------------------------------------------------------------------------------------------
# module converter
# ------------------------------------------------------------------------------------------------
def convert_svdq_linear_to_natural_layout(linear) -> None:
    """
    Convert one ``SVDQW4A4Linear``'s parameters in place from the checkpoint layout to the natural layout
    (nunchaku/ops/triton/layout.py:226-292): ``qweight``, ``wscales``, ``bias``, ``smooth_factor``, ``wcscales``,
    ``proj_down`` (stored from the transposed ``(rank, in)`` tensor, hence the ``.t()``), ``proj_up``.
    ``smooth_factor_orig`` is unused and left alone.  Call exactly once per loaded layer.
    """
    n, half_k = linear.qweight.shape
    k = half_k * 2
    with torch.no_grad():
        linear.qweight.data = unpack_weight_packed_nibbles(linear.qweight.data, n, k).view(torch.int8)
        linear.wscales.data = unpack_scale(linear.wscales.data, n, group_size=linear.group_size).to(linear.wscales.dtype)
        if linear.bias is not None:
            linear.bias.data = unpack_scale(linear.bias.data.reshape(1, -1), n, group_size=-1).to(linear.bias.dtype)
        linear.smooth_factor.data = unpack_scale(linear.smooth_factor.data.reshape(1, -1), k, group_size=-1).to(
            linear.smooth_factor.dtype
        )
        if linear.wcscales is not None:
            linear.wcscales.data = unpack_scale(linear.wcscales.data.reshape(1, -1), n, group_size=-1).to(
                linear.wcscales.dtype
            )
        if linear.proj_down.numel() > 0:
            linear.proj_down.data = unpack_lowrank_weight(linear.proj_down.data, down=True).t().contiguous()
        if linear.proj_up.numel() > 0:
            linear.proj_up.data = unpack_lowrank_weight(linear.proj_up.data, down=False).contiguous()

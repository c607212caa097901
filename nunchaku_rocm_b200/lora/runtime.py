"""
Runtime LoRA for one layer, with the call signatures of the reference's ``attach_lora`` / ``detach_lora``
(nunchaku/lora/runtime.py:475-535).

An :class:`~nunchaku_rocm_b200.models.linear.SVDQW4A4Linear` already carries a 16-bit low-rank branch
``(x @ proj_down) @ proj_up^T`` that the quantiser and the GEMM kernels evaluate with a run-time rank.  Extra
LoRAs are therefore not a second code path: their factors are concatenated to ``proj_down`` / ``proj_up`` along the
rank axis (zero-padded to a multiple of 16, the rank granularity of the kernels), and the same two launches compute
``W4A4(x) + (x @ [down | lora_downs]) @ [up | lora_ups]^T``.  Layers without such a branch (AWQ modulation layers,
plain ``nn.Linear``) get a forward hook that adds ``(x @ down^T) @ up^T``.

The mapping from a LoRA checkpoint's key names to module paths (the reference's ``set_loras``) belongs to the
model classes, which this package does not contain; it ends in calls of :func:`attach_lora`.
"""

from __future__ import annotations

import torch
from torch import nn

RANK_GRANULARITY = 16  # the low-rank branch of the quantiser and GEMM kernels works on multiples of 16 ranks


def _is_svdq(module: nn.Module) -> bool:
    from ..models.linear import SVDQW4A4Linear

    return isinstance(module, SVDQW4A4Linear)


class _AddLowRank:
    """Forward hook: ``output + sum_i (x @ down_i^T) @ up_i^T`` in the dtype of the factors."""

    def __init__(self, pairs):
        self.pairs = list(pairs)

    def __call__(self, module, args, output):
        x = args[0]
        if self.pairs and self.pairs[0][0].device != x.device:  # the module moved after the attachment
            self.pairs = [(d.to(x.device), u.to(x.device)) for d, u in self.pairs]
        for down, up in self.pairs:
            output = output + ((x.to(down.dtype) @ down.t()) @ up.t()).to(output.dtype)
        return output


def attach_lora(module: nn.Module, pairs: list[tuple[torch.Tensor, torch.Tensor]]) -> None:
    """
    Add ``sum_i (x @ down_i^T) @ up_i^T`` to the layer's output.  ``down_i`` is ``(r_i, in_features)``, ``up_i`` is
    ``(out_features, r_i)`` with the LoRA strength already folded in.  Replaces whatever was attached before;
    :func:`detach_lora` restores the base layer.
    """
    detach_lora(module)
    if not pairs:
        return
    for down, up in pairs:
        if down.dim() != 2 or up.dim() != 2 or down.shape[0] != up.shape[1]:
            raise ValueError(f"LoRA factors must be (r, in) and (out, r); got {tuple(down.shape)} and {tuple(up.shape)}")
    if _is_svdq(module):
        base_down, base_up = module.proj_down.data, module.proj_up.data
        n_in, n_out = base_down.shape[0], base_up.shape[0]
        for down, up in pairs:
            if down.shape[1] != n_in or up.shape[0] != n_out:
                raise ValueError(f"LoRA factors {tuple(down.shape)}, {tuple(up.shape)} do not fit a {n_in} -> {n_out} layer")
        dev, dt = base_down.device, base_down.dtype
        extra = sum(d.shape[0] for d, _ in pairs)
        pad = -(base_down.shape[1] + extra) % RANK_GRANULARITY
        new_down = torch.zeros(n_in, base_down.shape[1] + extra + pad, device=dev, dtype=dt)
        new_up = torch.zeros(n_out, base_up.shape[1] + extra + pad, device=dev, dtype=dt)
        new_down[:, : base_down.shape[1]] = base_down
        new_up[:, : base_up.shape[1]] = base_up
        at = base_down.shape[1]
        for down, up in pairs:
            r = down.shape[0]
            new_down[:, at : at + r] = down.t().to(dev, dt)
            new_up[:, at : at + r] = up.to(dev, dt)
            at += r
        module._lora_base = (base_down, base_up, module.rank)
        module.proj_down.data, module.proj_up.data = new_down, new_up
        module.rank = new_down.shape[1]
    else:
        ref = next((p for p in module.parameters() if p.is_floating_point()), None)
        if ref is None:
            raise ValueError(f"{type(module).__name__} has no floating-point parameter to take the LoRA dtype from")
        hook = _AddLowRank((d.to(ref.device, ref.dtype), u.to(ref.device, ref.dtype)) for d, u in pairs)
        module._lora_hook = (hook, module.register_forward_hook(hook))


def detach_lora(module: nn.Module) -> None:
    """Undo :func:`attach_lora`; a layer with nothing attached is left alone."""
    if hasattr(module, "_lora_base"):
        base_down, base_up, rank = module._lora_base
        dev = module.proj_down.device  # the layer may have moved since
        module.proj_down.data, module.proj_up.data = base_down.to(dev), base_up.to(dev)
        module.rank = rank
        del module._lora_base
    if hasattr(module, "_lora_hook"):
        module._lora_hook[1].remove()
        del module._lora_hook


def attached_rank(module: nn.Module) -> int:
    """Ranks added on top of the layer's own low-rank branch (padding included); 0 when nothing is attached."""
    if hasattr(module, "_lora_base"):
        return module.proj_down.shape[1] - module._lora_base[0].shape[1]
    if hasattr(module, "_lora_hook"):
        return sum(d.shape[0] for d, _ in module._lora_hook[0].pairs)
    return 0

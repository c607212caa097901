"""Runtime LoRA on the quantised layers (the per-layer half of the reference's ``nunchaku/lora/runtime.py``)."""

from .runtime import attach_lora, attached_rank, detach_lora

__all__ = ["attach_lora", "attached_rank", "detach_lora"]

"""
Backend selection, reduced to the one backend this package has.

The reference's model classes branch on the literal string ``get_backend() == "triton"`` to choose
natural layouts and the natural rotary table (nunchaku/models/transformers/transformer_flux_v2.py:427,531),
which are the layouts the kernels here read, so :func:`get_backend` returns that constant.
Signatures follow nunchaku/ops/backend.py:31-98.
"""

from __future__ import annotations

import os

__all__ = ["get_backend", "set_backend", "has_cuda_extension", "load_cuda_ops"]

_VALID = ("cuda", "triton")
_NAME = "triton"


def has_cuda_extension() -> bool:
    """The upstream ``nunchaku._C`` extension (mma-fragment layouts) is never part of this build."""
    return False


def load_cuda_ops():
    raise RuntimeError(
        "nunchaku._C is not part of this build; the sm_100a kernels are reached through nunchaku_rocm_b200.ops"
    )


def get_backend() -> str:
    """Always ``"triton"``: the natural-layout seam.  A ``NUNCHAKU_BACKEND`` value is validated, not obeyed."""
    env = os.environ.get("NUNCHAKU_BACKEND")
    if env is not None and env.strip().lower() not in _VALID:
        raise ValueError(f"NUNCHAKU_BACKEND must be one of {_VALID}, got {env.strip().lower()!r}")
    return _NAME


def set_backend(name: str | None) -> None:
    """Accepts the reference's names; ``"cuda"`` (the fragment-layout seam) cannot be selected."""
    if name is None:
        return
    name = name.strip().lower()
    if name not in _VALID:
        raise ValueError(f"backend must be one of {_VALID}, got {name!r}")
    if name != _NAME:
        raise RuntimeError("only the natural-layout backend exists in this build")

"""Operator API with the signatures of the reference's ``nunchaku/ops`` package."""

from . import backend, gemm, quantize  # noqa: F401

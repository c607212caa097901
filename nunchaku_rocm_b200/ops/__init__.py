"""Operator API with the signatures of the reference's ``nunchaku/ops`` package."""

from . import backend, dispatch, gemm, gemv, quantize  # noqa: F401

"""
B200-native (sm_100a) implementation of the SVDQuant hot path of nunchaku-rocm: W4A4 GEMM with its
low-rank branch and fused epilogues, the activation quantizer, AWQ W4A16 and attention, behind the
reference's ``nunchaku.ops`` operator signatures.  Python is plumbing only: every operator launches
a hand-written CUDA kernel from ``libnunchaku_b200.so`` through its C ABI, and raises if that
library is absent.
"""

__version__ = "0.1.0"

from . import ops  # noqa: F401

"""
Kernel-level entry points under the module names the reference's models and tests import
(``nunchaku.ops.triton.{gemm_w4a4, awq, attention, layout}``).  The package name is kept for
import compatibility only; every function launches a CUDA kernel of ``libnunchaku_b200.so``.
"""

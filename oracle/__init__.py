"""
CPU restatement of the reference's SVDQuant hot path.  Test infrastructure only: nothing under
the product package imports it, and the product raises when its CUDA library is missing instead
of falling back to this code.
"""

from . import awq_attn, w4a4  # noqa: F401

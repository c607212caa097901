"""Host helpers the reference exposes from ``nunchaku.ops.triton.native`` (row orders, reasons)."""

"""Host-side mirrors of the reference's layer containers that call the operators (callers, not kernels)."""

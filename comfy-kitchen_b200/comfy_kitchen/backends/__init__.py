"""Backends of the quantized-linear operators: one, the sm_100a C-ABI library (``cuda``)."""

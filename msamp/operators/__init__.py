"""Operators with the reference's calling conventions, backed by ``msamp.ops`` kernels."""

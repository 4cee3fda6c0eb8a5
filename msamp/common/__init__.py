"""Device-agnostic core: quantised dtypes, scaling tensors and utilities."""

"""Kernel layer.

Every operator has two implementations behind one Python function:

* tensors on a CUDA device run hand-written sm_100a kernels from ``libmsamp_b200.so``
  (sources in ``msamp/ops/csrc``), loaded with ctypes;
* tensors on the CPU run a bit-faithful emulation built from ``torch.float8_*`` conversions with
  explicit saturation, which is also the oracle the GPU tests compare against.

There is no silent fallback from the first to the second: a CUDA tensor with no native library
raises ``RuntimeError``.
"""

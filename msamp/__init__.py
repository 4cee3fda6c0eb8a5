"""msamp: FP8 mixed-precision training for NVIDIA B200."""
__version__ = '0.4.0'

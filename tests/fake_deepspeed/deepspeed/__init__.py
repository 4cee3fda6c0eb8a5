"""A minimal stand-in for the ``deepspeed`` package, used only by tests/test_deepspeed_adapter_cpu.py.

It reproduces the parts of DeepSpeed's engine and config that msamp's adapter hooks into - constructor flow,
``_configure_optimizer`` / ``_configure_basic_optimizer`` / ``_configure_lr_scheduler``, the config accessors and
the backward / step loop - so that the adapter can be exercised without the real library (which is not installed in
the test environment).  It is NOT DeepSpeed and implements nothing else.
"""
__version__ = '0.0.fake'

"""Deferred module import (reference: msamp/common/utils/lazy_import.py:9-65)."""
import importlib


class LazyImport:
    """Proxy that imports ``module`` (and optionally picks ``attr`` from it) on first use."""
    def __init__(self, module, attr=None):
        self.__dict__['_lazy_module'] = module
        self.__dict__['_lazy_attr'] = attr
        self.__dict__['_lazy_target'] = None

    def _resolve(self):
        target = self.__dict__['_lazy_target']
        if target is None:
            target = importlib.import_module(self.__dict__['_lazy_module'])
            if self.__dict__['_lazy_attr'] is not None:
                target = getattr(target, self.__dict__['_lazy_attr'])
            self.__dict__['_lazy_target'] = target
        return target

    def __getattr__(self, name):
        return getattr(self._resolve(), name)

    def __setattr__(self, name, value):
        setattr(self._resolve(), name, value)

    def __call__(self, *args, **kwargs):
        return self._resolve()(*args, **kwargs)

    def __dir__(self):
        return dir(self._resolve())

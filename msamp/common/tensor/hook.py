"""Ordered registry of callbacks.

Hooks are called as ``fn(manager, args, args[0])`` – the same three-argument shape the reference
gets from implementing its registry with module forward hooks
(msamp/common/tensor/hook.py:9-82) – so callbacks written as ``hook(module, input, output)`` work.
The attribute names ``hooks`` and ``history_counter`` are part of the pickled checkpoint layout.
"""


class HookManager:
    """Keeps callbacks in registration order and invokes them together."""
    class _RemoveHandle:
        """Returned by ``register_hook``; ``remove()`` unregisters that one callback."""
        def __init__(self, manager, hook_id):
            self.manager = manager
            self.hook_id = hook_id

        def remove(self):
            self.manager.hooks.pop(self.hook_id, None)

    def __init__(self):
        self.hooks = dict()
        self.history_counter = 0

    def __call__(self, *args, **kwargs):
        if not self.hooks:
            return
        first = args[0] if args else None
        for fn in list(self.hooks.values()):
            fn(self, args, first, **kwargs)

    def register_hook(self, fn):
        """Add ``fn`` and return a handle whose ``remove()`` deletes it."""
        hook_id = self.history_counter
        self.hooks[hook_id] = fn
        self.history_counter += 1
        return self._RemoveHandle(self, hook_id)

    def __len__(self):
        return len(self.hooks)

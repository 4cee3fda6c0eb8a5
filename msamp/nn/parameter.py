"""Parameter flavour of ScalingTensor (reference: msamp/nn/parameter.py:9-28)."""
from msamp.common.tensor import ScalingTensor


class ScalingParameter(ScalingTensor):
    """A ScalingTensor that a module registers as one of its parameters."""
    def __init__(self, tensor, requires_grad=True):
        super().__init__(tensor.value, tensor.meta)
        self._requires_grad = bool(requires_grad)
        self._is_param = True

    def __repr__(self):
        return f'ScalingParameter({super().__repr__()}, requires_grad={self._requires_grad})'

    def clone(self):
        return ScalingParameter(super().clone(), requires_grad=self._requires_grad)

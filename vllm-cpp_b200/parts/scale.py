"""Layer scale: a sublayer's result, after its norm, is multiplied coordinate by coordinate by a learned
vector before it joins the residual stream.  "vector": the learned factor (one tensor, the slot's prefix
itself); "none": no factor.  The arrangement folds the vector into the gain of the norm in front of it, so
no kernel of its own runs.  The reference has no such part.
"""
from __future__ import annotations

from typing import Dict

from .base import ParamSpec, Scale, register_scale


@register_scale("vector")
class VectorScale(Scale):
    def __init__(self, size: int, dtype, device):
        if size <= 0:
            raise ValueError("layer scale: size must be positive")
        self.size = size
        self.vector = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"": ParamSpec((self.size,), "gain")}

    def load_params(self, tensors):
        self.vector = tensors[""].contiguous()


@register_scale("none")
class NoScale(Scale):
    def __init__(self, dtype=None, device=None):
        pass

"""Gates on a sublayer's result, computed from the sublayer's input.

"sigmoid_linear": result * sigmoid(W x + b).  The part runs the product; bias and sigmoid are applied by
the kernel that consumes the gate together with the norm and the residual addition
(ops.gated_norm_residual).  "none": no gate.  The reference has no gated residual branches.
"""
from __future__ import annotations

from typing import Dict

from ..csrc import ops
from .base import Gate, ParamSpec, register_gate


@register_gate("sigmoid_linear")
class SigmoidLinearGate(Gate):
    def __init__(self, in_size: int, out_size: int, dtype, device):
        if in_size <= 0 or out_size <= 0:
            raise ValueError("gate: sizes must be positive")
        self.in_size, self.out_size = in_size, out_size
        self.weight = None
        self.bias = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"": ParamSpec((self.out_size, self.in_size)), ".b": ParamSpec((self.out_size,), "bias")}

    def load_params(self, tensors):
        self.weight = tensors[""].contiguous()
        self.bias = tensors[".b"].contiguous()

    def forward(self, x, pre):
        ops.linear(x, self.weight, pre)


@register_gate("none")
class NoGate(Gate):
    def __init__(self, dtype=None, device=None):
        pass

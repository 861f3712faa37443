"""Token shift: a sublayer reads, instead of row t of the residual stream, a mix of rows t and t - 1 of
the same request,  s[t] = x[t] + (x[t-1] - x[t]) * mu  with one learned mu per coordinate and x[-1] = 0.
Row t - 1 of a step's first row is what the request's previous step ended with: per-request state of
``size`` floats, kept in a slot of the cache manager and rewritten by every step.  The reference has no
such part.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import ParamSpec, StateSpec, TokenShift, register_token_shift


@register_token_shift("lerp_previous")
class LerpPrevious(TokenShift):
    def __init__(self, size: int, dtype, device):
        if size <= 0:
            raise ValueError("token shift: size must be positive")
        self.size = size
        self.mu: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"": ParamSpec((self.size,), "bias")}

    def load_params(self, tensors):
        self.mu = tensors[""].contiguous()

    def state_spec(self):
        return StateSpec((self.size,), torch.float32)

    def forward(self, x, shifted, plain, step, state):
        ops.token_shift(x, self.mu, state.slots, shifted, plain, step.q_start, step.req_of_token, step.positions,
                        step.state_slots)

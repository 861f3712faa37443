"""Two mixers side by side: both read the same input, and the layer's result is
``left_scale * left(x) + right_scale * right(x)``.  The members are any registered mixers (PartSpecs); their
tensors sit under ``left.`` and ``right.``, and each keeps the cache it would keep alone: the pair declares a
CompositeSpec and hands each member its own view.  The reference has no such part.
"""
from __future__ import annotations

from typing import Dict

from ..config.model_spec import PartSpec
from ..csrc import ops
from .base import MIXERS, CompositeSpec, Mixer, ParamSpec, build_part, register_mixer, workspace_piece


@register_mixer("parallel")
class ParallelMixers(Mixer):
    def __init__(self, hidden_size: int, left: PartSpec, right: PartSpec, left_scale: float, right_scale: float, dtype, device):
        self.hidden, self.dtype = hidden_size, dtype
        self.left = build_part(MIXERS, "mixer", left, dtype=dtype, device=device)
        self.right = build_part(MIXERS, "mixer", right, dtype=dtype, device=device)
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)

    def members(self):
        return (("left.", self.left), ("right.", self.right))

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {prefix + name: ps for prefix, m in self.members() for name, ps in m.param_specs().items()}

    def load_params(self, tensors):
        for prefix, m in self.members():
            m.load_params({name: tensors[prefix + name] for name in m.param_specs()})

    def product_weights(self):
        return [pw for _, m in self.members() for pw in m.product_weights()]

    def step_arrays(self):
        out = {}
        for _, m in self.members():
            out.update(m.step_arrays())
        return out

    def reserve(self, n_tokens, n_reqs, device):
        for _, m in self.members():
            m.reserve(n_tokens, n_reqs, device)

    def cache_spec(self):
        return CompositeSpec((self.left.cache_spec(), self.right.cache_spec()))

    def workspace_bytes(self, n_tokens, n_reqs):
        return 2 * workspace_piece((n_tokens, self.hidden), self.dtype) + max(m.workspace_bytes(n_tokens, n_reqs) for _, m in self.members())

    def forward(self, x, out, step, cache, writes_cache, ws):
        mark = ws.mark()
        n = x.shape[0]
        a = ws.take((n, self.hidden), self.dtype)
        b = ws.take((n, self.hidden), self.dtype)
        self.left.forward(x, a, step, cache.views[0], writes_cache, ws)
        self.right.forward(x, b, step, cache.views[1], writes_cache, ws)
        ops.scaled_sum(a, b, out, self.left_scale, self.right_scale)
        ws.release(mark)

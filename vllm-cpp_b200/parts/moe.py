"""A feed-forward of routed experts.

    s = softmax(W_r h)                      float32, over ``num_experts`` + ``num_identity`` router outputs
    chosen = the ``top`` outputs with the largest s + correction;  weights = s[chosen], as they are
    out = sum over chosen of weight * expert(h)

Outputs 0 .. num_experts - 1 are small gated feed-forwards with tensors ``e<i>.gate``, ``e<i>.up``, ``e<i>.down``:
g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), W_down (g * sigmoid(alpha * g) * (u + 1)).  The last
``num_identity`` outputs are identity experts, expert(h) = h, without tensors.

Everything runs on the device (csrc/moe.cu): the router (logits, then selection), a sort of the (token, choice) pairs by expert, one product
per tile of an expert's rows for gate-and-up (with the activation) and one for down, and the weighted sum.  The
grids are sized for the most tiles a step can have, so a step's launches do not depend on the routing and the host
never reads it.  The reference has no routed feed-forward (src/layers/mlp.cpp).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, ParamSpec, register_feed_forward, workspace_piece


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, expert_size: int, num_experts: int, num_identity: int, top: int, limit: float,
                 dtype, device, alpha: float = 1.702):
        if min(hidden_size, expert_size, num_experts, top) <= 0 or num_identity < 0:
            raise ValueError("routed_experts: sizes must be positive")
        if top > num_experts + num_identity:
            raise ValueError(f"routed_experts: {top} of {num_experts + num_identity} router outputs cannot be chosen")
        if not limit > 0:
            raise ValueError("routed_experts: limit must be positive")
        self.hidden, self.ff, self.E, self.I, self.top = hidden_size, expert_size, num_experts, num_identity, top
        self.limit, self.alpha = float(limit), float(alpha)
        self.dtype, self.device = dtype, device
        self.w_gate_up = self.w_down = self.w_router = self.correction = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {}
        for e in range(self.E):
            specs[f"e{e}.gate"] = ParamSpec((self.ff, self.hidden))
            specs[f"e{e}.up"] = ParamSpec((self.ff, self.hidden))
            specs[f"e{e}.down"] = ParamSpec((self.hidden, self.ff))
        specs["router"] = ParamSpec((self.E + self.I, self.hidden), "bias")       # held in float32: the router is
        specs["correction"] = ParamSpec((self.E + self.I,), "bias")
        return specs

    def load_params(self, tensors):
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0) for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(self.E)]).contiguous()
        self.w_router = tensors["router"].contiguous()
        self.correction = tensors["correction"].contiguous()

    def product_weights(self):
        return []                 # the experts' products are this part's own kernels; nothing to measure or tile

    def workspace_bytes(self, n_tokens, n_reqs):
        pairs = n_tokens * self.top
        tiles = max(ops.moe_max_tiles(n_tokens, self.top, self.E, tm) for tm in ops.MOE_TILE_ROWS)
        ints = 3 * workspace_piece((pairs,), torch.int32) + 3 * workspace_piece((tiles,), torch.int32) + workspace_piece((4,), torch.int32)
        return (ints + workspace_piece((pairs,), torch.float32) + workspace_piece((n_tokens, self.E + self.I), torch.float32)
                + workspace_piece((pairs, self.ff), self.dtype)
                + workspace_piece((pairs, self.hidden), torch.float32))

    def forward(self, x, out, step, ws):
        n = x.shape[0]
        mark = ws.mark()
        pairs = n * self.top
        tm = ops.moe_tile_rows(n, self.top, self.E)
        tiles = ops.moe_max_tiles(n, self.top, self.E, tm)
        ids = ws.take((n, self.top), torch.int32)
        weights = ws.take((n, self.top), torch.float32)
        sorted_token = ws.take((pairs,), torch.int32)
        pos = ws.take((pairs,), torch.int32)
        tile_expert, tile_row0, tile_rows = (ws.take((tiles,), torch.int32) for _ in range(3))
        meta = ws.take((4,), torch.int32)
        logits = ws.take((n, self.E + self.I), torch.float32)
        ops.moe_router(x, self.w_router, self.correction, ids, weights, logits)
        ops.moe_sort(ids, self.E, tm, sorted_token, pos, tile_expert, tile_row0, tile_rows, meta)
        act = ws.take((pairs, self.ff), self.dtype)
        lists = (sorted_token, tile_expert, tile_row0, tile_rows, meta, tiles, tm)
        ops.moe_expert_gemm(x, self.w_gate_up, act, *lists, gated=True, limit=self.limit, alpha=self.alpha)
        y = ws.take((pairs, self.hidden), torch.float32)
        ops.moe_expert_gemm(act, self.w_down, y, *lists, gated=False)
        ops.moe_combine(y, x, pos, weights, out)
        ws.release(mark)

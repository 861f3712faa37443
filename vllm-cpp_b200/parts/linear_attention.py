"""Mixers whose memory is a matrix per head instead of a cache of keys: every token decays the matrix and adds
the outer product of its key and value, and reads it with its query,

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,      S: [head_dim, v_head_dim] float32, zero at admission.

The state lives in a slot of the cache manager (StateSpec), is read at the start of a request's portion and left
there at its end, so a prompt may be cut anywhere and decoding continues from what the prompt left.  One kernel
runs the recurrence for portions and single tokens alike (csrc/recurrent.cu); a second norms the result and
applies the output gate.

"gated_linear_attention": a decay per key channel and token, a_t = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau); queries
scaled by head_dim^(-1/2); each head's result RMS-normed over its value channels with one gain vector shared by the
heads, times silu(W_g h), then W_o.

"lightning_attention": one constant decay per head (``decay``); q, k and v pass through silu; the heads' results
are RMS-normed together, times sigmoid(W_g h), then W_o.

The reference has no recurrent mixer (src/layers/attention.cpp is its only one).
"""
from __future__ import annotations

from typing import Dict, Sequence

import numpy as np
import torch

from ..csrc import ops
from .base import Mixer, ParamSpec, StateSpec, register_mixer, workspace_piece

DEFAULT_DECAY_RANK = 32      # inner width of the decay's two products where no checkpoint gives it (random weights)


class DecayedStateMixer(Mixer):
    """What the two mixers share: sizes, the state's spec, the input product, the recurrence, norm and gate,
    the output product.  A subclass lists the rows of its input product (``in_rows``) and says how the decay
    and the norm are made."""

    def _init_sizes(self, hidden_size, num_heads, head_dim, v_head_dim, eps, dtype, device):
        if min(hidden_size, num_heads, head_dim, v_head_dim) <= 0:
            raise ValueError(f"{type(self).__name__}: sizes must be positive")
        if head_dim > 512:
            raise ValueError(f"{type(self).__name__}: head_dim {head_dim} exceeds 512, the most the recurrence kernel keeps")
        if not eps > 0:
            raise ValueError(f"{type(self).__name__}: eps must be positive")
        self.hidden, self.heads, self.dk, self.dv, self.eps = hidden_size, num_heads, head_dim, v_head_dim, float(eps)
        self.dtype, self.device = dtype, device
        self.w_in = None
        self.w_o = None
        self.w_norm = None

    def cache_spec(self):
        return StateSpec((self.heads, self.dk, self.dv), torch.float32)

    def in_rows(self) -> Sequence[int]:
        """Row counts of the tensors concatenated into the input product, in order; q, k, v and g come first."""
        return (self.heads * self.dk, self.heads * self.dk, self.heads * self.dv, self.heads * self.dv)

    def workspace_bytes(self, n_tokens, n_reqs):
        c = self.heads * self.dv
        most_pieces = n_tokens // ops.SCAN_PIECE + n_reqs
        pieces = (workspace_piece((most_pieces, self.heads, self.dk, self.dv), torch.float32)
                  + workspace_piece((n_tokens, self.heads * self.dk), torch.float32) + workspace_piece((most_pieces, self.heads * self.dk), torch.float32))
        return (workspace_piece((n_tokens, sum(self.in_rows())), self.dtype) + workspace_piece((n_tokens, self.heads * self.dk), self.dtype)
                + workspace_piece((n_tokens, c), torch.float32) + workspace_piece((n_tokens, c), self.dtype)
                + (pieces if n_tokens > ops.SCAN_PIECE else 0))

    def step_arrays(self):
        """A step with a portion longer than ops.SCAN_PIECE tokens runs the recurrence in pieces side by side
        (ops.decayed_state_scan with ``pieces``): the pieces' first rows, the pieces of each request and the scratch
        slots they use, and their number as a launch shape.  Other steps get placeholders."""
        def cut(host):
            if max(host.q_lens) <= ops.SCAN_PIECE:
                return None
            starts, per_req = ops.scan_pieces(host.q_lens)
            host.shapes["scan_pieces"] = len(starts) - 1
            return starts, per_req
        none = np.zeros(1, dtype=np.int32)
        return {"scan_piece_start": lambda host: none if cut(host) is None else cut(host)[0],
                "scan_piece_req": lambda host: none if cut(host) is None else cut(host)[1],
                "scan_piece_slots": lambda host: none if cut(host) is None else np.arange(len(cut(host)[0]) - 1, dtype=np.int32)}

    def pieces(self, step, ws):
        """The ``pieces`` argument of ops.decayed_state_scan for this step (None: the step has no long portion)."""
        count = step.shapes.get("scan_pieces")
        if not count or step.max_q_len <= ops.SCAN_PIECE:
            return None
        return {"start": step.extras["scan_piece_start"], "req": step.extras["scan_piece_req"], "slots": step.extras["scan_piece_slots"],
                "count": count, "state": ws.take((count, self.heads, self.dk, self.dv), torch.float32),
                "qp": ws.take((step.n_tokens, self.heads * self.dk), torch.float32), "dtot": ws.take((count, self.heads * self.dk), torch.float32)}

    def product_weights(self):
        return [(self.w_in, 0), (self.w_o, 0)]

    def _split(self, proj):
        qk, vg = self.heads * self.dk, self.heads * self.dv
        return proj[:, :qk], proj[:, qk: 2 * qk], proj[:, 2 * qk: 2 * qk + vg], proj[:, 2 * qk + vg: 2 * qk + 2 * vg]


@register_mixer("gated_linear_attention")
class GatedLinearAttention(DecayedStateMixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, tau: float, eps: float, dtype, device):
        self._init_sizes(hidden_size, num_heads, head_dim, v_head_dim, eps, dtype, device)
        if not tau > 0:
            raise ValueError("gated_linear_attention: tau must be positive")
        self.tau = float(tau)
        self.rank = None          # inner width of the decay's products: the checkpoint's tensors give it
        self.w_a2 = None
        self.b_a = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        qk, vg, r = self.heads * self.dk, self.heads * self.dv, DEFAULT_DECAY_RANK
        return {"q": ParamSpec((qk, self.hidden)), "k": ParamSpec((qk, self.hidden)), "v": ParamSpec((vg, self.hidden)),
                "g": ParamSpec((vg, self.hidden)), "o": ParamSpec((self.hidden, vg)), "norm": ParamSpec((self.dv,), "gain"),
                "a1": ParamSpec((-1, self.hidden), default_shape=(r, self.hidden)),
                "a2": ParamSpec((qk, -1), default_shape=(qk, r)), "a2.b": ParamSpec((qk,), "bias")}

    def load_params(self, tensors):
        if tensors["a1"].shape[0] != tensors["a2"].shape[1]:
            raise ValueError(f"gated_linear_attention: the decay's products do not fit: a1 {tuple(tensors['a1'].shape)}, "
                             f"a2 {tuple(tensors['a2'].shape)}")
        self.rank = int(tensors["a1"].shape[0])
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "g", "a1")], dim=0).contiguous()
        self.w_a2 = tensors["a2"].contiguous()
        self.b_a = tensors["a2.b"].contiguous()
        self.w_norm = tensors["norm"].contiguous()
        self.w_o = tensors["o"].contiguous()

    def in_rows(self):
        return (*super().in_rows(), self.rank if self.rank is not None else DEFAULT_DECAY_RANK)

    def product_weights(self):
        return [(self.w_in, 0), (self.w_a2, 0), (self.w_o, 0)]

    def forward(self, x, out, step, cache, writes_cache, ws):
        n, H = x.shape[0], self.heads
        mark = ws.mark()
        proj = ws.take((n, sum(self.in_rows())), self.dtype)
        ops.linear(x, self.w_in, proj)
        q, k, v, g = self._split(proj)
        low = proj[:, 2 * H * (self.dk + self.dv):]
        pre = ws.take((n, H * self.dk), self.dtype)
        ops.linear(low, self.w_a2, pre)
        o = ws.take((n, H * self.dv), torch.float32)
        ops.decayed_state_scan(q, k, v, cache.slots, o, step.q_start, step.state_slots, step.n_reqs, num_heads=H,
                               decay_pre=pre, decay_bias=self.b_a, tau=self.tau, q_scale=float(self.dk) ** -0.5,
                               pieces=self.pieces(step, ws))
        act = ws.take((n, H * self.dv), self.dtype)
        ops.gated_group_norm(o, g, self.w_norm, act, group=self.dv, eps=self.eps, gate_act="silu")
        ops.linear(act, self.w_o, out)
        ws.release(mark)


@register_mixer("lightning_attention")
class LightningAttention(DecayedStateMixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, decay: Sequence[float], eps: float,
                 dtype, device):
        self._init_sizes(hidden_size, num_heads, head_dim, v_head_dim, eps, dtype, device)
        decay = [float(d) for d in decay]
        if len(decay) != num_heads or not all(0.0 <= d <= 1.0 for d in decay):
            raise ValueError(f"lightning_attention: one decay in [0, 1] per head, got {decay} for {num_heads} heads")
        self.decay_values = decay
        self.decay = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        qk, vg = self.heads * self.dk, self.heads * self.dv
        return {"q": ParamSpec((qk, self.hidden)), "k": ParamSpec((qk, self.hidden)), "v": ParamSpec((vg, self.hidden)),
                "g": ParamSpec((vg, self.hidden)), "o": ParamSpec((self.hidden, vg)), "norm": ParamSpec((vg,), "gain")}

    def load_params(self, tensors):
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_norm = tensors["norm"].contiguous()
        self.w_o = tensors["o"].contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)

    def forward(self, x, out, step, cache, writes_cache, ws):
        n, H = x.shape[0], self.heads
        mark = ws.mark()
        proj = ws.take((n, sum(self.in_rows())), self.dtype)
        ops.linear(x, self.w_in, proj)
        q, k, v, g = self._split(proj)
        o = ws.take((n, H * self.dv), torch.float32)
        ops.decayed_state_scan(q, k, v, cache.slots, o, step.q_start, step.state_slots, step.n_reqs, num_heads=H,
                               decay_const=self.decay, silu_inputs=True, pieces=self.pieces(step, ws))
        act = ws.take((n, H * self.dv), self.dtype)
        ops.gated_group_norm(o, g, self.w_norm, act, group=H * self.dv, eps=self.eps, gate_act="sigmoid")
        ops.linear(act, self.w_o, out)
        ws.release(mark)

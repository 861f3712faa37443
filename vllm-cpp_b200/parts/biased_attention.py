"""Grouped-query attention over the paged cache without rotation, whose positions enter through a learned bias
by distance:

    q = rms(W_q h) * w_q,  k = rms(W_k h) * w_k      RMS norm over the whole projection (all heads at once)
    v = W_v h                                        heads of ``v_head_dim``, which may differ from ``head_dim``
    score(i, j) = cap * tanh(scale * (q_i . k_j) / cap) + rel[bucket(i - j), head]        0 <= i - j < window
    out = W_o (concat_heads(softmax(score) v) * sigmoid(W_g h))

``rel`` has B rows (the checkpoint's tensor gives B).  Distances below B // 2 have a row each; from there the
rows are spread evenly over the logarithm of the distance up to ``bias_reach``, and every distance from
``bias_reach`` on uses the last row:  bucket(n) = n  for n < B // 2,  else
min(B - 1, B // 2 + floor(ln(n / (B // 2)) / ln(bias_reach / (B // 2)) * (B - B // 2))).  At load the table is
expanded to one row per distance (up to the window, or to ``bias_reach``, where it becomes constant), so the
kernel looks a distance up directly.  ``cap`` 0 switches the cap off, ``window`` 0 the window.

The cache holds the normed keys and the values in rows of max(head_dim, v_head_dim) elements
(PagedKVSpec.head_dim); with a window, pages behind it are given back.  q, k, v and the gate are one product.
In bfloat16 with key and value heads of one size, 64 or 128, attention runs on the engine's tensor-core kernels
(tcgen05 for portions, mma.sync split over the keys for single tokens), which cap and bias the scores inside their
softmax; other sizes and float32 run the plain kernel of csrc/attention_biased.cu.
The reference's attention (src/layers/attention.cpp) has rotation and none of the rest.
"""
from __future__ import annotations

import math
from typing import Dict

import numpy as np
import torch

from ..csrc import ops
from .attention import PagedAttentionKernels
from .base import PagedKVSpec, ParamSpec, register_mixer, workspace_piece

DEFAULT_BIAS_ROWS = 64       # rows of the bias table where no checkpoint gives them (random weights)


def distance_buckets(rows: int, reach: float, count: int) -> np.ndarray:
    """bucket(n) for n = 0 .. count - 1 (see the module's text), in double precision."""
    half = rows // 2
    out = np.empty(count, dtype=np.int64)
    for n in range(count):
        if n < half:
            out[n] = n
        else:
            out[n] = min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(reach / half) * (rows - half))))
    return out


@register_mixer("biased_window_attention")
class BiasedWindowAttention(PagedAttentionKernels):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, scale: float,
                 softcap: float, window: int, bias_reach: float, eps: float, dtype, device, qk_norm: bool = True,
                 output_gate: bool = True):
        if min(hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim) <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"biased_window_attention: {num_heads} heads cannot share {num_kv_heads} kv heads")
        if v_head_dim > 256 or head_dim > 1024:
            raise ValueError("biased_window_attention: head sizes up to 1024 (keys) and 256 (values)")
        if window < 0 or softcap < 0 or not eps > 0 or not bias_reach > 0:
            raise ValueError("biased_window_attention: window and softcap must not be negative, eps and bias_reach positive")
        self.hidden, self.nh, self.nkv, self.dk, self.dv = hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim
        self.row = max(head_dim, v_head_dim)
        self.d = self.row              # a cached row's width, as the paged attention kernels see it
        self.scale, self.cap, self.window, self.reach, self.eps = float(scale), float(softcap), int(window), float(bias_reach), float(eps)
        self.qk_norm, self.output_gate = bool(qk_norm), bool(output_gate)
        self.dtype, self.device = dtype, device
        self.w_in = self.w_o = self.w_qn = self.w_kn = self.bias = self.bias_t = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        q, kk, vv = self.nh * self.dk, self.nkv * self.dk, self.nkv * self.dv
        specs = {"q": ParamSpec((q, self.hidden)), "k": ParamSpec((kk, self.hidden)), "v": ParamSpec((vv, self.hidden))}
        if self.qk_norm:
            specs["q.norm"] = ParamSpec((q,), "gain")
            specs["k.norm"] = ParamSpec((kk,), "gain")
        specs["rel"] = ParamSpec((-1, self.nh), "bias", default_shape=(DEFAULT_BIAS_ROWS, self.nh))
        if self.output_gate:
            specs["g"] = ParamSpec((self.nh * self.dv, self.hidden))
        specs["o"] = ParamSpec((self.hidden, self.nh * self.dv))
        return specs

    def load_params(self, tensors):
        rows = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.output_gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        if self.qk_norm:
            self.w_qn, self.w_kn = tensors["q.norm"].contiguous(), tensors["k.norm"].contiguous()
        rel = tensors["rel"].to(torch.float32)
        B = int(rel.shape[0])
        if B < 2 or self.reach <= B // 2:
            raise ValueError(f"biased_window_attention: a bias table of {B} rows cannot reach distance {self.reach}")
        # one row per distance; from ceil(bias_reach) on every distance reads the last row of the table
        count = int(math.ceil(self.reach)) + 1
        if self.window > 0:
            count = min(count, self.window)
        idx = torch.from_numpy(distance_buckets(B, self.reach, count)).to(rel.device)
        self.bias = rel.index_select(0, idx).contiguous()           # [distances, heads]
        self.bias_t = self.bias.t().contiguous()                    # [heads, distances], for the tensor-core kernels
        if self.dk == self.dv:
            self.warn_if_plain()

    def _tensor_core_path(self) -> bool:
        return self.dk == self.dv and super()._tensor_core_path()

    def score_shaping(self):
        return {"cap": self.cap, "bias_t": self.bias_t}

    def product_weights(self):
        return [(self.w_in, 0), (self.w_o, 0)]

    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.row, self.window)

    def in_width(self) -> int:
        return self.nh * self.dk + self.nkv * (self.dk + self.dv) + (self.nh * self.dv if self.output_gate else 0)

    def workspace_bytes(self, n_tokens, n_reqs):
        return (workspace_piece((n_tokens, self.in_width()), self.dtype) + workspace_piece((n_tokens, self.nh * self.dk), self.dtype)
                + workspace_piece((n_tokens, self.nh * self.dv), self.dtype))

    def forward(self, x, out, step, cache, writes_cache, ws):
        n = x.shape[0]
        mark = ws.mark()
        proj = ws.take((n, self.in_width()), self.dtype)
        ops.linear(x, self.w_in, proj)
        q_off, k_off = 0, self.nh * self.dk
        v_off = k_off + self.nkv * self.dk
        g_off = v_off + self.nkv * self.dv
        block_table = step.block_tables[cache.group]
        pages = cache.pages.view(cache.pages.shape[0], -1)
        sizes = dict(num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.dk, v_head_dim=self.dv, row=self.row,
                     page_size=cache.page_size)
        q = ws.take((n, self.nh * self.dk), self.dtype)
        ops.qk_norm_cache_write(proj, q_off, k_off, v_off, self.w_qn, self.w_kn, q, pages, step.positions, step.req_of_token,
                                block_table, eps=self.eps, write_kv=writes_cache, **sizes)
        attn = ws.take((n, self.nh * self.dv), self.dtype)
        gate = proj[:, g_off:] if self.output_gate else None
        if self._tensor_core_path() and cache.page_size % 8 == 0:
            self.attend(q, attn, step, cache, block_table)
            if gate is not None:
                ops.sigmoid_gate(attn, gate)
        else:
            ops.attention_biased(q, pages, attn, gate, step.positions, step.req_of_token, block_table, self.bias,
                                 window=self.window, scale=self.scale, cap=self.cap, **sizes)
        ops.linear(attn, self.w_o, out)
        ws.release(mark)

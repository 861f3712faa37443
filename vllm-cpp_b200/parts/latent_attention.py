"""Latent attention: keys and values of every head are projections of one low-rank row per token, and
only that row (the latent) is cached.

    q_h = Wq_h s                                    per head, `head_dim` wide; no position enters
    c   = rms(Wdkv s) * w_c                         the latent, `kv_rank` wide, RMS-normed in float
    k_h = Wuk_h c,  v_h = Wuv_h c                   `head_dim` and `v_head_dim` wide
    p   = softmax_j((q_h . k_h[j]) * scale),  j in the window (the query's own position included)
    out = Wo (concat_h(sum_j p v_h[j]) * sigmoid(Wg s))

Since q_h . (Wuk_h c) = (Wuk_h^T q_h) . c and sum_j p (Wuv_h c_j) = Wuv_h (sum_j p c_j), the queries are
moved into the latent space, attention runs against the cached rows themselves (multi-query attention
with one row per token that is key and value at once, PagedKVSpec.planes = 1, on the engine's paged
attention kernels), and its result is moved out again; keys and values are never formed.

A layer may read another layer's cached latents (a run-order entry with ``writes_cache`` False): it then
has no down-projection of its own (``owns_latent`` False), but its own queries, window and up-projections.
``cache_window`` is the window the cache layer is kept for (the widest of its readers).  The reference
has no such mixer (its one mixer is src/layers/attention.cpp).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .attention import PagedAttentionKernels
from .base import PagedKVSpec, ParamSpec, register_mixer, workspace_piece


@register_mixer("latent_attention")
class LatentAttention(PagedAttentionKernels):
    planes = 1

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, kv_rank: int, scale: float,
                 window: int, cache_window: int, owns_latent: bool, eps: float, output_gate: bool, dtype, device):
        if min(hidden_size, num_heads, head_dim, v_head_dim, kv_rank) <= 0:
            raise ValueError("latent_attention: sizes must be positive")
        if kv_rank > ops.SIMT_MAX_HEAD_DIM:
            raise ValueError(f"latent_attention: kv_rank {kv_rank} exceeds {ops.SIMT_MAX_HEAD_DIM}, the widest row the attention kernels take")
        if window < 0 or cache_window < 0 or (cache_window and (window == 0 or window > cache_window)):
            raise ValueError("latent_attention: the cache must be kept for at least the mixer's window")
        if not eps > 0:
            raise ValueError("latent_attention: eps must be positive")
        self.hidden, self.heads, self.qk, self.vd, self.rank = hidden_size, num_heads, head_dim, v_head_dim, kv_rank
        # as the attention kernels see it: every head reads the one cached row of a token
        self.nh, self.nkv, self.d = num_heads, 1, kv_rank
        self.scale, self.window, self.cache_window = float(scale), int(window), int(cache_window)
        self.owns_latent, self.eps, self.output_gate = bool(owns_latent), float(eps), bool(output_gate)
        self.dtype, self.device = dtype, device
        self.w_in = None          # [q | dkv | g] rows: one product on the mixer's input
        self.w_c = None           # gain of the latent's norm
        self.w_uk_t = None        # [heads, kv_rank, head_dim]: Wuk_h^T
        self.w_uv = None          # [heads, v_head_dim, kv_rank]
        self.w_o = None

    # -- tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        h = self.heads
        specs = {"q": ParamSpec((h * self.qk, self.hidden))}
        if self.owns_latent:
            specs["dkv"] = ParamSpec((self.rank, self.hidden))
            specs["dkv.norm"] = ParamSpec((self.rank,), "gain")
        specs["uk"] = ParamSpec((h * self.qk, self.rank))
        specs["uv"] = ParamSpec((h * self.vd, self.rank))
        if self.output_gate:
            specs["g"] = ParamSpec((h * self.vd, self.hidden))
        specs["o"] = ParamSpec((self.hidden, h * self.vd))
        return specs

    def load_params(self, tensors):
        rows = [tensors["q"]] + ([tensors["dkv"]] if self.owns_latent else []) + ([tensors["g"]] if self.output_gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_c = tensors["dkv.norm"].contiguous() if self.owns_latent else None
        self.w_uk_t = tensors["uk"].unflatten(0, (self.heads, self.qk)).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"].unflatten(0, (self.heads, self.vd)).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.warn_if_plain()

    def product_weights(self):
        return [(self.w_in, 0), (self.w_o, 0)]

    # -- cache
    def cache_spec(self):
        return PagedKVSpec(1, self.rank, self.cache_window, planes=1)

    def workspace_bytes(self, n_tokens, n_reqs):
        h = self.heads
        return (workspace_piece((n_tokens, self.w_rows()), self.dtype) + 2 * workspace_piece((n_tokens, h * self.rank), self.dtype)
                + workspace_piece((n_tokens, h * self.vd), self.dtype))

    def w_rows(self) -> int:
        return self.heads * self.qk + (self.rank if self.owns_latent else 0) + (self.heads * self.vd if self.output_gate else 0)

    # -- run
    def forward(self, x, out, step, cache, writes_cache, ws):
        if writes_cache != self.owns_latent:
            raise ValueError("latent_attention: a layer writes the cache layer it reads exactly when it has a down-projection")
        n, h = x.shape[0], self.heads
        mark = ws.mark()
        proj = ws.take((n, self.w_rows()), self.dtype)
        ops.linear(x, self.w_in, proj)
        q0 = h * self.qk
        g0 = q0 + (self.rank if self.owns_latent else 0)
        block_table = step.block_tables[cache.group]
        pages = cache.pages.view(cache.pages.shape[0], -1)
        if self.owns_latent:
            ops.latent_cache_write(proj[:, q0:g0], self.w_c, step.positions, step.req_of_token, block_table, pages,
                                   page_size=cache.page_size, eps=self.eps)
        q_lat = ws.take((n, h * self.rank), self.dtype)
        ops.headwise_linear(proj[:, :q0], self.w_uk_t, q_lat)
        o_lat = ws.take((n, h * self.rank), self.dtype)
        self.attend(q_lat, o_lat, step, cache, block_table)
        o = ws.take((n, h * self.vd), self.dtype)
        ops.headwise_linear(o_lat, self.w_uv, o, gate=proj[:, g0:] if self.output_gate else None)
        ops.linear(o, self.w_o, out)
        ws.release(mark)

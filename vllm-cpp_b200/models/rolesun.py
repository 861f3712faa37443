"""Rolesun: a decoder of latent-attention layers with token shift, gated residual branches and norms on
the sublayers' results; typed configuration and its description as parts.

config.json names the design in ``architecture`` and gives every size and constant:

    vocab, width, residual_mult, logit_scale, embedding.scale, norm.eps,
    layers[i] = {type, mixer: {heads, dim, vdim, kv_rank, scale, mask: {size}, [kv_from]}, mlp: {kind, ff} | null}

Layer i's tensors are ``l<i>.*``: ``shift``, ``rg1`` / ``rg1.b`` / ``norm1`` around the mixer ``mix.*``,
``rg2`` / ``rg2.b`` / ``norm2`` around the feed-forward ``mlp.*``; outside the layers ``embed``,
``final.norm`` and ``head``.  A layer with ``kv_from: j`` reads the latents layer j caches and has no
down-projection.  What the design fixes (the base of the position vector, silu in the feed-forward, the
sigmoid of the gates) is in the parts' code.  The reference has no model of this kind (its registry
holds llama, qwen and gemma, src/core/engine.cpp:26-28).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from ..config.engine_config import ConfigError
from ..config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture

POSITION_BASE = 10000.0          # of the sinusoidal position vector
MAX_POSITIONS = 1 << 22          # positions are exact in float far beyond this; the cache bounds a request first


@dataclass
class RolesunMixer:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int                      # 0: all keys
    kv_from: Optional[int] = None


@dataclass
class RolesunLayer:
    mixer: RolesunMixer
    ff: Optional[int] = None         # width of the dense feed-forward; None: the layer has none


@dataclass
class RolesunConfig:
    vocab: int
    width: int
    residual_mult: float
    logit_scale: float
    embedding_scale: float
    eps: float
    layers: List[RolesunLayer] = field(default_factory=list)

    @classmethod
    def from_dict(cls, cfg: dict) -> "RolesunConfig":
        problems: List[str] = []

        def number(d, key, where, integer=False, positive=True, default=None):
            v = d.get(key, default) if isinstance(d, dict) else None
            if v is None:
                problems.append(f"missing {where}'{key}'")
                return 1
            ok = isinstance(v, int) if integer else isinstance(v, (int, float))
            if isinstance(v, bool) or not ok:
                problems.append(f"{where}'{key}' must be {'an integer' if integer else 'a number'}, got {v!r}")
                return 1
            if positive and not v > 0:
                problems.append(f"{where}'{key}' must be positive, got {v!r}")
                return 1
            return v

        vocab = number(cfg, "vocab", "", integer=True)
        width = number(cfg, "width", "", integer=True)
        mult = number(cfg, "residual_mult", "", positive=False)
        logit_scale = number(cfg, "logit_scale", "", positive=False, default=1.0)
        emb_scale = number(cfg.get("embedding"), "scale", "embedding.", positive=False)
        eps = number(cfg.get("norm"), "eps", "norm.")
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            problems.append("'layers' must be a non-empty list")
            raw_layers = []
        layers: List[RolesunLayer] = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                problems.append(f"layers[{i}] must be an object with a 'mixer'")
                continue
            if entry.get("type") != "latent_attention":
                problems.append(f"{where}type {entry.get('type')!r} is not a mixer of this design (known: 'latent_attention')")
                continue
            m = entry["mixer"]
            mw = where + "mixer."
            mask = m.get("mask")
            window = 0
            if mask is not None:
                window = number(mask, "size", mw + "mask.", integer=True)
            kv_from = m.get("kv_from")
            if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int)):
                problems.append(f"{mw}'kv_from' must be a layer index, got {kv_from!r}")
                kv_from = None
            mixer = RolesunMixer(heads=number(m, "heads", mw, integer=True), dim=number(m, "dim", mw, integer=True),
                                 vdim=number(m, "vdim", mw, integer=True), kv_rank=number(m, "kv_rank", mw, integer=True),
                                 scale=number(m, "scale", mw, positive=False), window=window, kv_from=kv_from)
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    problems.append(f"{where}mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not "
                                    "a feed-forward of this design (known: 'dense')")
                else:
                    ff = number(mlp, "ff", where + "mlp.", integer=True)
            layers.append(RolesunLayer(mixer, ff))
        if not problems:
            for i, layer in enumerate(layers):
                j = layer.mixer.kv_from
                if j is None:
                    continue
                if not 0 <= j < i:
                    problems.append(f"layers[{i}].mixer.kv_from = {j} must name an earlier layer")
                elif layers[j].mixer.kv_from is not None:
                    problems.append(f"layers[{i}].mixer.kv_from = {j}: that layer has no latents of its own")
                elif layers[j].mixer.kv_rank != layer.mixer.kv_rank:
                    problems.append(f"layers[{i}].mixer.kv_rank {layer.mixer.kv_rank} differs from layer {j}'s "
                                    f"{layers[j].mixer.kv_rank}, whose latents it reads")
        if problems:
            raise ConfigError("Rolesun config.json: " + "; ".join(problems))
        return cls(vocab=vocab, width=width, residual_mult=float(mult), logit_scale=float(logit_scale),
                   embedding_scale=float(emb_scale), eps=float(eps), layers=layers)

    def cache_window(self, layer: int) -> int:
        """The window for which the latents that layer ``layer`` caches are kept: the widest window of the
        layers that read them (0, all keys, if any of them sees all keys)."""
        windows = [l.mixer.window for i, l in enumerate(self.layers) if i == layer or l.mixer.kv_from == layer]
        return 0 if min(windows) == 0 else max(windows)


def rolesun_model_spec(c: RolesunConfig) -> ModelSpec:
    layers, order, absent = [], [], []
    # cache layers: first the latents of the layers that own some, in layer order, then every layer's token-shift row
    owners = [i for i, layer in enumerate(c.layers) if layer.mixer.kv_from is None]
    latent_layer = {i: k for k, i in enumerate(owners)}
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        source = i if m.kv_from is None else m.kv_from
        norm = PartSpec("rmsnorm_scalar", {"size": c.width, "eps": c.eps})
        has_ff = layer.ff is not None
        layers.append(LayerSpec(
            shift=PartSpec("lerp_previous", {"size": c.width}),
            mixer=PartSpec("latent_attention", {
                "hidden_size": c.width, "num_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "window": m.window, "cache_window": c.cache_window(source),
                "owns_latent": m.kv_from is None, "eps": c.eps, "output_gate": True}),
            mixer_gate=PartSpec("sigmoid_linear", {"in_size": c.width, "out_size": c.width}),
            mixer_norm=norm,
            feed_forward=PartSpec("gated_mlp", {"hidden_size": c.width, "intermediate_size": layer.ff, "activation": "silu",
                                                "tensor_names": ("gate", "up", "down")}) if has_ff else PartSpec("none"),
            feed_forward_gate=PartSpec("sigmoid_linear", {"in_size": c.width, "out_size": c.width}) if has_ff else PartSpec("none"),
            feed_forward_norm=PartSpec("rmsnorm_scalar", dict(norm.params)) if has_ff else PartSpec("none"),
            block="shift_gate_postnorm",
            block_params={"residual_mult": c.residual_mult},
            names={"shift": p + "shift", "mixer": p + "mix.", "mixer_gate": p + "rg1", "mixer_norm": p + "norm1",
                   "feed_forward": p + "mlp.", "feed_forward_gate": p + "rg2", "feed_forward_norm": p + "norm2"},
        ))
        if not has_ff:          # a file may still hold the tensors around a feed-forward that the layer does not have
            absent += [p + "norm2", p + "rg2", p + "rg2.b"]
        order.append(LayerCall(layer=i, cache=latent_layer[source], writes_cache=m.kv_from is None, state=len(owners) + i))
    return ModelSpec(
        architecture="Rolesun",
        hidden_size=c.width,
        vocab_size=c.vocab,
        layers=layers,
        run_order=order,
        final_norm=PartSpec("rmsnorm_scalar", {"size": c.width, "eps": c.eps, "out_scale": c.logit_scale}),
        tie_word_embeddings=False,
        max_position_embeddings=MAX_POSITIONS,
        embed_name="embed",
        final_norm_prefix="final.norm",
        lm_head_name="head",
        ignored_tensors=absent,
        init_std=0.05,
        init_gain_std=0.05,
        model_class="scaled_sinusoid_decoder",
        model_params={"embedding_scale": c.embedding_scale, "position_base": POSITION_BASE},
    )


@register_architecture("Rolesun", "rolesun")
def build_rolesun(config: dict):
    typed = RolesunConfig.from_dict(config)
    return typed, rolesun_model_spec(typed)

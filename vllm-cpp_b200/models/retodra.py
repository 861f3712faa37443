"""Retodra: a decoder whose layers mix tokens either by gated linear attention or by a windowed softmax attention
beside a lightning attention, with a norm before and after every sublayer, layer scale, and dense or routed
feed-forwards; typed configuration and its description as parts.

config.json names the design in ``architecture`` and gives every size and constant:

    vocab, width, embedding.scale, norm.eps,
    layers[i] = {type: "gla",      mixer: {heads, dim, vdim, tau},
                 type: "parallel", mixer: {left: {heads, kv_heads, dim, vdim, scale, softcap, bias_max, mask: {size}},
                                           right: {heads, dim, vdim, decay: [per head]}, left_scale, right_scale},
                 mlp: null | {kind: "dense", ff} | {kind: "moe", expert: {ff, limit}, router: {experts, identity, top}}}

Layer i's tensors are ``l<i>.*``: ``norm1`` / ``norm1b`` / ``ls1`` around the mixer ``mix.*`` (``mix.left.*`` and
``mix.right.*`` in a parallel layer), ``norm2`` / ``norm2b`` / ``ls2`` around the feed-forward ``mlp.*``; outside
the layers ``embed``, ``final.norm`` and ``head``.  The layers' norms store their gain around zero.  Two sizes come
from the tensors alone: the rows of the distance-bias table ``rel`` and the inner width of the decay's products
``a1`` / ``a2``.  What the design fixes (silu and sigmoid gates, the experts' activation constant, the bucket
rule of the bias) is in the parts.  The reference has no model of this kind (src/core/engine.cpp:26-28).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from ..config.engine_config import ConfigError
from ..config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture

MAX_POSITIONS = 1 << 22          # no position table bounds a request; the cache does first
EXPERT_ACTIVATION_ALPHA = 1.702  # y = g * sigmoid(alpha * g) * (u + 1) in the experts


@dataclass
class RetodraLayer:
    kind: str                        # "gla" or "parallel"
    mixer: dict                      # the layer's "mixer" object, checked
    mlp: Optional[dict] = None       # the layer's "mlp" object, checked; None: no feed-forward


@dataclass
class RetodraConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: List[RetodraLayer] = field(default_factory=list)

    @classmethod
    def from_dict(cls, cfg: dict) -> "RetodraConfig":
        problems: List[str] = []

        def number(d, key, where, integer=False, positive=True):
            v = d.get(key) if isinstance(d, dict) else None
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

        def numbers(d, where, integers=(), reals=(), any_sign=()):
            out = {k: number(d, k, where, integer=True) for k in integers}
            out.update({k: float(number(d, k, where)) for k in reals})
            out.update({k: float(number(d, k, where, positive=False)) for k in any_sign})
            return out

        vocab = number(cfg, "vocab", "", integer=True)
        width = number(cfg, "width", "", integer=True)
        emb_scale = number(cfg.get("embedding"), "scale", "embedding.", positive=False)
        eps = number(cfg.get("norm"), "eps", "norm.")
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            problems.append("'layers' must be a non-empty list")
            raw_layers = []
        layers: List[RetodraLayer] = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                problems.append(f"layers[{i}] must be an object with a 'mixer'")
                continue
            kind, m, mw = entry.get("type"), entry["mixer"], where + "mixer."
            if kind == "gla":
                mixer = numbers(m, mw, integers=("heads", "dim", "vdim"), reals=("tau",))
            elif kind == "parallel":
                left, right = m.get("left"), m.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    problems.append(f"{mw}'left' and {mw}'right' must be objects")
                    continue
                lw, rw = mw + "left.", mw + "right."
                lm = numbers(left, lw, integers=("heads", "dim", "vdim"), reals=("scale", "bias_max"))
                lm["kv_heads"] = lm["heads"] if left.get("kv_heads") is None else number(left, "kv_heads", lw, integer=True)
                cap = left.get("softcap")           # absent or 0: scores are not capped
                lm["softcap"] = 0.0 if not cap and not isinstance(cap, bool) else float(number(left, "softcap", lw))
                mask = left.get("mask")
                lm["window"] = 0 if mask is None else number(mask, "size", lw + "mask.", integer=True)
                if lm["heads"] % lm["kv_heads"]:
                    problems.append(f"{lw}heads {lm['heads']} is no multiple of kv_heads {lm['kv_heads']}")
                rm = numbers(right, rw, integers=("heads", "dim", "vdim"))
                decay = right.get("decay")
                if (not isinstance(decay, list) or len(decay) != rm["heads"]
                        or not all(isinstance(d, (int, float)) and not isinstance(d, bool) and 0 <= d <= 1 for d in decay)):
                    problems.append(f"{rw}'decay' must list one number in [0, 1] per head, got {decay!r}")
                    decay = [1.0] * rm["heads"]
                rm["decay"] = [float(d) for d in decay]
                mixer = {"left": lm, "right": rm, **numbers(m, mw, any_sign=("left_scale", "right_scale"))}
            else:
                problems.append(f"{where}type {kind!r} is not a mixer of this design (known: 'gla', 'parallel')")
                continue
            mlp, checked = entry.get("mlp"), None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    problems.append(f"{where}mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not a "
                                    "feed-forward of this design (known: 'dense', 'moe')")
                elif mlp["kind"] == "dense":
                    checked = {"kind": "dense", "ff": number(mlp, "ff", where + "mlp.", integer=True)}
                else:
                    ex, ro = mlp.get("expert"), mlp.get("router")
                    checked = {"kind": "moe", "ff": number(ex, "ff", where + "mlp.expert.", integer=True),
                               "limit": float(number(ex, "limit", where + "mlp.expert.")),
                               "experts": number(ro, "experts", where + "mlp.router.", integer=True),
                               "top": number(ro, "top", where + "mlp.router.", integer=True)}
                    identity = ro.get("identity", 0) if isinstance(ro, dict) else 0
                    if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
                        problems.append(f"{where}mlp.router.'identity' must be a count, got {identity!r}")
                        identity = 0
                    checked["identity"] = identity
                    if checked["top"] > checked["experts"] + identity:
                        problems.append(f"{where}mlp.router.top {checked['top']} exceeds the router's {checked['experts'] + identity} outputs")
            layers.append(RetodraLayer(kind, mixer, checked))
        if problems:
            raise ConfigError("Retodra config.json: " + "; ".join(problems))
        return cls(vocab=vocab, width=width, embedding_scale=float(emb_scale), eps=float(eps), layers=layers)


def retodra_model_spec(c: RetodraConfig) -> ModelSpec:
    layers, order, absent = [], [], []
    norm = lambda: PartSpec("rmsnorm", {"size": c.width, "eps": c.eps, "tensor_name": "", "unit_offset": True})
    scale = lambda: PartSpec("vector", {"size": c.width})
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.kind == "gla":
            mixer = PartSpec("gated_linear_attention", {"hidden_size": c.width, "num_heads": m["heads"], "head_dim": m["dim"],
                                                        "v_head_dim": m["vdim"], "tau": m["tau"], "eps": c.eps})
        else:
            l, r = m["left"], m["right"]
            mixer = PartSpec("parallel", {
                "hidden_size": c.width, "left_scale": m["left_scale"], "right_scale": m["right_scale"],
                "left": PartSpec("biased_window_attention", {
                    "hidden_size": c.width, "num_heads": l["heads"], "num_kv_heads": l["kv_heads"], "head_dim": l["dim"],
                    "v_head_dim": l["vdim"], "scale": l["scale"], "softcap": l["softcap"], "window": l["window"],
                    "bias_reach": l["bias_max"], "eps": c.eps, "qk_norm": True, "output_gate": True}),
                "right": PartSpec("lightning_attention", {
                    "hidden_size": c.width, "num_heads": r["heads"], "head_dim": r["dim"], "v_head_dim": r["vdim"],
                    "decay": r["decay"], "eps": c.eps})})
        mlp = layer.mlp
        if mlp is None:
            ff = PartSpec("none")
            absent += [p + "norm2", p + "norm2b", p + "ls2"]      # a file may still hold them
        elif mlp["kind"] == "dense":
            ff = PartSpec("gated_mlp", {"hidden_size": c.width, "intermediate_size": mlp["ff"], "activation": "silu",
                                        "tensor_names": ("gate", "up", "down")})
        else:
            ff = PartSpec("routed_experts", {"hidden_size": c.width, "expert_size": mlp["ff"], "num_experts": mlp["experts"],
                                             "num_identity": mlp["identity"], "top": mlp["top"], "limit": mlp["limit"],
                                             "alpha": EXPERT_ACTIVATION_ALPHA})
        has_ff = mlp is not None
        layers.append(LayerSpec(
            mixer=mixer, feed_forward=ff,
            mixer_norm=norm(), mixer_post_norm=norm(), mixer_scale=scale(),
            feed_forward_norm=norm() if has_ff else PartSpec("none"),
            feed_forward_post_norm=norm() if has_ff else PartSpec("none"),
            feed_forward_scale=scale() if has_ff else PartSpec("none"),
            block="sandwich_norm",
            names={"mixer": p + "mix.", "feed_forward": p + "mlp.", "mixer_norm": p + "norm1", "mixer_post_norm": p + "norm1b",
                   "mixer_scale": p + "ls1", "feed_forward_norm": p + "norm2", "feed_forward_post_norm": p + "norm2b",
                   "feed_forward_scale": p + "ls2"},
        ))
        order.append(LayerCall(layer=i, cache=i))
    return ModelSpec(
        architecture="Retodra",
        hidden_size=c.width,
        vocab_size=c.vocab,
        layers=layers,
        run_order=order,
        final_norm=PartSpec("rmsnorm", {"size": c.width, "eps": c.eps, "tensor_name": "", "unit_offset": True}),
        tie_word_embeddings=False,
        max_position_embeddings=MAX_POSITIONS,
        embed_name="embed",
        final_norm_prefix="final.norm",
        lm_head_name="head",
        ignored_tensors=absent,
        init_std=0.05,
        init_gain_std=0.05,
        model_class="scaled_embedding_decoder",
        model_params={"embedding_scale": c.embedding_scale},
    )


@register_architecture("Retodra", "retodra")
def build_retodra(config: dict):
    typed = RetodraConfig.from_dict(config)
    return typed, retodra_model_spec(typed)

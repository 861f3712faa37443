"""Plain, slow implementation of the Rolesun decoder in numpy float64: the oracle of the tests.

One function per mechanism, written from the design's equations and sharing no code with the engine.
A model is (config dict, {tensor name: float64 array}).  Everything is computed for one sequence at
a time, all positions at once, with explicit loops where the engine has kernels.

Notation.  x: residual stream [T, width].  For layer l with residual multiplier m:

    g1 = sigmoid(x R1^T + b1)                      gate of the mixer's result, from the unshifted x
    s  = x + (prev(x) - x) * shift                 token shift; prev(x)[t] = x[t-1], zeros at t = 0
    x  = x + m * snorm1(mixer(s) * g1)             snorm(z) = z / sqrt(mean(z^2) + eps) * one number
    g2 = sigmoid(x R2^T + b2)
    x  = x + m * snorm2(ff(x) * g2)

Mixer "latent_attention" on input s:  q = s Wq^T (heads of `dim`);  c = rms(s Wdkv^T) * w_c (the latent,
`kv_rank` wide; a layer with `kv_from` takes the c of that layer instead);  per head k = c Wuk_h^T,
v = c Wuv_h^T;  p = softmax over the keys j with 0 <= t - j < mask.size of (q_h . k_h) * scale;
o_h = sum p v;  result = (concat(o) * sigmoid(s Wg^T)) Wo^T.
"""
import json
import os
import struct

import numpy as np

SINUSOID_BASE = 10000.0


# ------------------------------------------------------------------ files
def read_safetensors(path):
    """{name: float64 (or int64) array}: 8-byte length, JSON header, data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        raw = data[lo:hi]
        if e["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif e["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: type {e['dtype']}")
        out[name] = a.reshape(e["shape"])
    return out


def read_model_folder(path):
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(path, "model.safetensors"))


def round_to_bf16(weights):
    """The values a bfloat16 checkpoint of these weights holds (round to nearest even)."""
    out = {}
    for k, v in weights.items():
        u = v.astype(np.float32).view(np.uint32).astype(np.uint64)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        out[k] = u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(v.shape)
    return out


# ------------------------------------------------------------- mechanisms
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms(z, eps):
    return z / np.sqrt(np.mean(z * z, axis=-1, keepdims=True) + eps)


def scalar_norm(z, gain, eps):
    """RMS norm whose gain is one number for all coordinates."""
    return rms(z, eps) * float(gain)


def embed(cfg, w, tokens, first_position=0):
    """Scaled embedding rows plus the sinusoidal position vector (sin at even, cos at odd entries)."""
    width = cfg["width"]
    x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    p = np.arange(first_position, first_position + len(tokens), dtype=np.float64)[:, None]
    i = np.arange(width // 2, dtype=np.float64)[None, :]
    angle = p * SINUSOID_BASE ** (-2.0 * i / width)
    pe = np.zeros((len(tokens), width))
    pe[:, 0::2] = np.sin(angle)
    pe[:, 1::2] = np.cos(angle)[:, : pe[:, 1::2].shape[1]]
    return x + pe


def token_shift(x, shift):
    """s[t] = x[t] + (x[t-1] - x[t]) * shift, x[-1] = 0."""
    prev = np.zeros_like(x)
    prev[1:] = x[:-1]
    return x + (prev - x) * shift


def latent(w, prefix, s, eps):
    """The latent rows of a layer that owns a down-projection."""
    return rms(s @ w[prefix + "mix.dkv"].T, eps) * w[prefix + "mix.dkv.norm"]


def windowed_softmax_attention(q, k, v, scale, window):
    """q [T, H, d], k [T, H, d], v [T, H, dv] -> [T, H, dv]; query t sees keys t - window < j <= t."""
    T, H, _ = q.shape
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        lo = max(0, t - window + 1) if window > 0 else 0
        for h in range(H):
            sc = (k[lo: t + 1, h] @ q[t, h]) * scale
            p = np.exp(sc - sc.max())
            p /= p.sum()
            out[t, h] = p @ v[lo: t + 1, h]
    return out


def latent_attention(w, prefix, mixer, s, c):
    """The mixer on shifted input s with latent rows c (its own or another layer's)."""
    H, d, dv = mixer["heads"], mixer["dim"], mixer["vdim"]
    T = s.shape[0]
    q = (s @ w[prefix + "mix.q"].T).reshape(T, H, d)
    k = (c @ w[prefix + "mix.uk"].T).reshape(T, H, d)
    v = (c @ w[prefix + "mix.uv"].T).reshape(T, H, dv)
    window = int(mixer["mask"]["size"]) if mixer.get("mask") else 0
    o = windowed_softmax_attention(q, k, v, mixer["scale"], window).reshape(T, H * dv)
    o = o * sigmoid(s @ w[prefix + "mix.g"].T)
    return o @ w[prefix + "mix.o"].T


def dense_ff(w, prefix, x):
    return (silu(x @ w[prefix + "mlp.gate"].T) * (x @ w[prefix + "mlp.up"].T)) @ w[prefix + "mlp.down"].T


def residual_gate(w, name, x):
    return sigmoid(x @ w[name].T + w[name + ".b"])


# ------------------------------------------------------------------ model
def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the residual stream after every layer)."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = embed(cfg, w, tokens)
    latents, after = {}, []
    for l, layer in enumerate(cfg["layers"]):
        if layer["type"] != "latent_attention":
            raise ValueError(f"layer {l}: mixer {layer['type']!r}")
        p, mixer = f"l{l}.", layer["mixer"]
        g1 = residual_gate(w, p + "rg1", x)
        s = token_shift(x, w[p + "shift"])
        if "kv_from" in mixer and mixer["kv_from"] is not None:
            c = latents[mixer["kv_from"]]
        else:
            c = latents[l] = latent(w, p, s, eps)
        y = latent_attention(w, p, mixer, s, c)
        x = x + m * scalar_norm(y * g1, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"layer {l}: feed-forward {layer['mlp']['kind']!r}")
            g2 = residual_gate(w, p + "rg2", x)
            x = x + m * scalar_norm(dense_ff(w, p, x) * g2, w[p + "norm2"], eps)
        after.append(x.copy())
    logits = (scalar_norm(x, w["final.norm"], eps) @ w["head"].T) * cfg["logit_scale"]
    return (logits, np.stack(after)) if return_layers else logits


def greedy(logits_row):
    return int(np.argmax(logits_row))


# ------------------------------------------------------- weights for tests
def tensor_shapes(cfg):
    """{name: shape} of every tensor a model of this configuration has."""
    width = cfg["width"]
    shapes = {"embed": (cfg["vocab"], width), "head": (cfg["vocab"], width), "final.norm": ()}
    for l, layer in enumerate(cfg["layers"]):
        p, m = f"l{l}.", layer["mixer"]
        H, d, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
        shapes.update({p + "shift": (width,), p + "rg1": (width, width), p + "rg1.b": (width,), p + "norm1": (),
                       p + "mix.q": (H * d, width), p + "mix.uk": (H * d, r), p + "mix.uv": (H * dv, r),
                       p + "mix.g": (H * dv, width), p + "mix.o": (width, H * dv)})
        if m.get("kv_from") is None:
            shapes.update({p + "mix.dkv": (r, width), p + "mix.dkv.norm": (r,)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            shapes.update({p + "rg2": (width, width), p + "rg2.b": (width,), p + "norm2": (),
                           p + "mlp.gate": (ff, width), p + "mlp.up": (ff, width), p + "mlp.down": (width, ff)})
    return shapes


def random_weights(cfg, seed, sharp=1.0):
    """Random weights with activations of order one everywhere; ``sharp`` multiplies the queries' matrices
    so that attention is peaked and a wrong or missing key shows in the logits."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[1] if name[0] == "l" and name[1].isdigit() else name
        if shape == ():
            w[name] = np.asarray(1.0 + 0.2 * rng.standard_normal())
        elif leaf == "shift":
            w[name] = rng.uniform(0.0, 1.0, shape)
        elif leaf == "mix.dkv.norm":
            w[name] = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf.endswith(".b"):
            w[name] = 0.5 * rng.standard_normal(shape)
        elif name == "embed":
            w[name] = rng.standard_normal(shape)
        else:
            w[name] = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if leaf == "mix.q":
                w[name] *= sharp
    return w


def to_bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def write_model_folder(path, cfg, weights, store="F32"):
    """config.json and model.safetensors with the tensors as float32 or bfloat16."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name in sorted(weights):
        a = np.asarray(weights[name], dtype=np.float32)          # a norm's single number keeps its empty shape
        raw = a.tobytes() if store == "F32" else to_bf16_bits(a).tobytes()
        header[name] = {"dtype": store, "shape": list(np.shape(weights[name])), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hb = json.dumps(header).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for raw in blobs:
            f.write(raw)

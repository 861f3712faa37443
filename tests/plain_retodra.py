"""Plain, slow implementation of the Retodra decoder in numpy float64: the oracle of the tests.

One function per mechanism, written from the design's equations and sharing no code with the engine.
A model is (config dict, {tensor name: float64 array}).  One sequence at a time, token by token where
the design has a recurrence.

Notation.  x: residual stream [T, width];  n(z, w) = z / sqrt(mean(z^2) + eps) * (1 + w) (the layers' norm,
gain stored around zero);  r(z, w) = z / sqrt(mean(z^2) + eps) * w (norms inside mixers, plain gain).

    x = embed[token] * embedding.scale
    layer:  x = x + ls1 * n(mixer(n(x, norm1)), norm1b);   x = x + ls2 * n(ff(n(x, norm2)), norm2b)
    logits = head n(x, final.norm)

Mixer "gla" (heads H, key size d, value size e, temperature tau) on input h:
    q = Wq h / sqrt(d), k = Wk h, v = Wv h;   a = sigmoid(Wa2 (Wa1 h) + b)^(1/tau)      one decay per key channel
    S_t = diag(a_t) S_(t-1) + k_t v_t^T   per head, S_(-1) = 0;   o_t = S_t^T q_t
    result = Wo (concat_heads r(o_head, norm) * silu(Wg h))                            norm over e, shared by heads

Mixer "parallel": left_scale * left(h) + right_scale * right(h).
  left (H query heads on G key/value heads, window W, cap c, scale s, bias table rel [B, H], reach D):
    q = r(Wq h, q.norm), k = r(Wk h, k.norm)  over the whole projection;  v = Wv h
    score(i, j) = c tanh(s (q_i . k_j) / c) + rel[bucket(i - j), head]      for 0 <= i - j < W
    bucket(n) = n if n < B/2 else min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(D / (B/2)) * (B - B/2)))
    result = Wo (concat_heads softmax(score) v * sigmoid(Wg h))
  right (H heads, constant decay lambda_head):
    q, k, v = silu(Wq h), silu(Wk h), silu(Wv h);   S_t = lambda S_(t-1) + k_t v_t^T;   o_t = S_t^T q_t
    result = Wo (r(concat_heads o, norm) * sigmoid(Wg h))

Feed-forward "dense": Wdown (silu(Wgate h) * (Wup h)).
Feed-forward "moe" (E experts with tensors, I identity experts after them, k chosen per token, clamp L):
    s = softmax(Wrouter h) over E + I;  chosen = the k largest of s + correction;  weights = s[chosen]
    expert(h) = Wdown (g sigmoid(1.702 g) (u + 1)),  g = min(Wgate h, L), u = clip(Wup h, -L, L);  identity(h) = h
"""
import json
import math
import os
import struct

import numpy as np


# ------------------------------------------------------------------ files
def read_safetensors(path):
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
    out = {}
    for k, v in weights.items():
        u = v.astype(np.float32).view(np.uint32).astype(np.uint64)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        out[k] = u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(v.shape)
    return out


def write_model_folder(path, cfg, weights, store="F32"):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name in sorted(weights):
        a = np.ascontiguousarray(weights[name], dtype=np.float32)
        if store == "BF16":
            raw = (a.view(np.uint32) >> 16).astype("<u2").tobytes()      # the values are bfloat16 already
        else:
            raw = a.astype("<f4").tobytes()
        header[name] = {"dtype": store, "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))


# ------------------------------------------------------------- mechanisms
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit(z, eps):
    return z / np.sqrt(np.mean(z * z, axis=-1, keepdims=True) + eps)


def layer_norm(z, w, eps):
    """The layers' norm: gain stored around zero."""
    return unit(z, eps) * (1.0 + w)


def plain_norm(z, w, eps):
    return unit(z, eps) * w


def decayed_outer_recurrence(q, k, v, decay, state=None):
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t.  q, k, decay: [T, d]; v: [T, e]."""
    T, d = q.shape
    S = np.zeros((d, v.shape[1])) if state is None else state.copy()
    o = np.zeros((T, v.shape[1]))
    for t in range(T):
        S = decay[t][:, None] * S + np.outer(k[t], v[t])
        o[t] = S.T @ q[t]
    return o, S


def gla_mixer(w, p, m, h, eps):
    H, d, e, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T) / math.sqrt(d)
    k = h @ w[p + "k"].T
    v = h @ w[p + "v"].T
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    a = sigmoid(z) ** (1.0 / tau)
    outs = []
    for i in range(H):
        o, _ = decayed_outer_recurrence(q[:, i * d:(i + 1) * d], k[:, i * d:(i + 1) * d], v[:, i * e:(i + 1) * e],
                                        a[:, i * d:(i + 1) * d])
        outs.append(plain_norm(o, w[p + "norm"], eps))
    o = np.concatenate(outs, axis=1) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def distance_bucket(n, rows, reach):
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(reach / half) * (rows - half))))


def capped_biased_attention(q, k, v, rel, H, G, W, cap, scale, reach):
    """q [T, H*d], k [T, G*d], v [T, G*e] of one sequence -> [T, H*e]: capped scores plus the bias of the distance,
    softmax over the keys j with 0 <= i - j < W (W 0: all j <= i)."""
    T = q.shape[0]
    d, e = q.shape[1] // H, v.shape[1] // G
    out = np.zeros((T, H * e))
    far = T if not W else min(T, W)
    buckets = np.array([distance_bucket(n, rel.shape[0], reach) for n in range(far)], dtype=np.int64)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            lo = max(0, i - W + 1) if W else 0
            s = scale * (k[lo:i + 1, g * d:(g + 1) * d] @ q[i, head * d:(head + 1) * d])
            if cap:
                s = cap * np.tanh(s / cap)
            s = s + rel[buckets[i - np.arange(lo, i + 1)], head]
            pr = np.exp(s - s.max())
            pr /= pr.sum()
            out[i, head * e:(head + 1) * e] = pr @ v[lo:i + 1, g * e:(g + 1) * e]
    return out


def biased_window_attention(w, p, m, h, eps):
    W = m["mask"]["size"] if m.get("mask") else 0            # 0: every earlier key is seen
    q = plain_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps)
    k = plain_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps)
    v = h @ w[p + "v"].T
    out = capped_biased_attention(q, k, v, w[p + "rel"], m["heads"], m["kv_heads"], W, m.get("softcap", 0.0), m["scale"],
                                  m["bias_max"])
    return (out * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def lightning_mixer(w, p, m, h, eps):
    H, d, e = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q, k, v = silu(h @ w[p + "q"].T), silu(h @ w[p + "k"].T), silu(h @ w[p + "v"].T)
    outs = []
    for i in range(H):
        o, _ = decayed_outer_recurrence(q[:, i * d:(i + 1) * d], k[:, i * d:(i + 1) * d], v[:, i * e:(i + 1) * e],
                                        np.full((T, d), float(m["decay"][i])))
        outs.append(o)
    o = plain_norm(np.concatenate(outs, axis=1), w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def parallel_mixer(w, p, m, h, eps):
    return (m["left_scale"] * biased_window_attention(w, p + "left.", m["left"], h, eps)
            + m["right_scale"] * lightning_mixer(w, p + "right.", m["right"], h, eps))


def dense_ff(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def clamped_expert(w, p, h, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(w, p, r, h, margins=None):
    """(chosen [T, top], weights [T, top]) over experts + identity outputs.  ``margins`` (a list) receives, per
    token, how far the last chosen output's choice score lies above the best one left out."""
    z = h @ w[p + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=-1, keepdims=True)
    choice = s + w[p + "correction"]
    order = np.argsort(-choice, axis=-1, kind="stable")
    chosen = order[:, : r["top"]]
    if margins is not None and order.shape[1] > r["top"]:
        ranked = np.take_along_axis(choice, order, axis=-1)
        margins.extend(ranked[:, r["top"] - 1] - ranked[:, r["top"]])
    return chosen, np.take_along_axis(s, chosen, axis=-1)


def moe_ff(w, p, mlp, h, margins=None):
    r = mlp["router"]
    chosen, weights = route(w, p, r, h, margins)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for c, wt in zip(chosen[t], weights[t]):
            if c >= r["experts"]:
                out[t] += wt * h[t]
            else:
                out[t] += wt * clamped_expert(w, f"{p}e{c}.", h[t:t + 1], mlp["expert"]["limit"])[0]
    return out


def forward(cfg, w, tokens, return_layers=False, margins=None):
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "gla":
            y = gla_mixer(w, p + "mix.", layer["mixer"], h, eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(w, p + "mix.", layer["mixer"], h, eps)
        else:
            raise ValueError(layer["type"])
        x = x + w[p + "ls1"] * layer_norm(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[p + "norm2"], eps)
            y = dense_ff(w, p + "mlp.", h) if mlp["kind"] == "dense" else moe_ff(w, p + "mlp.", mlp, h, margins)
            x = x + w[p + "ls2"] * layer_norm(y, w[p + "norm2b"], eps)
        layers.append(x.copy())
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(layers)) if return_layers else logits


def greedy(logits_row):
    return int(np.argmax(logits_row))


def routing_margin(cfg, w, tokens):
    """The smallest margin of any routing decision on these tokens (inf without routed layers): a test that
    compares logits asks for tokens whose decisions rounding cannot turn."""
    margins = []
    forward(cfg, w, tokens, margins=margins)
    return min(margins) if margins else math.inf


# ------------------------------------------------------------ random models
def tensor_shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b", "ls1"):
            s[p + n] = (W,)
        if layer["type"] == "gla":
            H, d, e = m["heads"], m["dim"], m["vdim"]
            rank = m.get("decay_rank", 8)
            s.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * e, W), p + "mix.g": (H * e, W),
                      p + "mix.o": (W, H * e), p + "mix.norm": (e,), p + "mix.a1": (rank, W), p + "mix.a2": (H * d, rank),
                      p + "mix.a2.b": (H * d,)})
        else:
            l, r = m["left"], m["right"]
            H, G, d, e = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            s.update({p + "mix.left.q": (H * d, W), p + "mix.left.k": (G * d, W), p + "mix.left.v": (G * e, W),
                      p + "mix.left.q.norm": (H * d,), p + "mix.left.k.norm": (G * d,), p + "mix.left.rel": (l["rel_rows"], H),
                      p + "mix.left.g": (H * e, W), p + "mix.left.o": (W, H * e)})
            H, d, e = r["heads"], r["dim"], r["vdim"]
            s.update({p + "mix.right.q": (H * d, W), p + "mix.right.k": (H * d, W), p + "mix.right.v": (H * e, W),
                      p + "mix.right.g": (H * e, W), p + "mix.right.o": (W, H * e), p + "mix.right.norm": (H * e,)})
        mlp = layer.get("mlp")
        if mlp is not None:
            for n in ("norm2", "norm2b", "ls2"):
                s[p + n] = (W,)
            if mlp["kind"] == "dense":
                s.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                r, ff = mlp["router"], mlp["expert"]["ff"]
                for e_ in range(r["experts"]):
                    s.update({f"{p}mlp.e{e_}.gate": (ff, W), f"{p}mlp.e{e_}.up": (ff, W), f"{p}mlp.e{e_}.down": (W, ff)})
                s[p + "mlp.router"] = (r["experts"] + r["identity"], W)
                s[p + "mlp.correction"] = (r["experts"] + r["identity"],)
    return s


def random_weights(cfg, seed, std=None, sharp=1.0, decisive_routing=False):
    """Random weights for a configuration made by the tests ('rel_rows' in a left mixer and 'decay_rank' in a gla
    mixer are the tests' own keys: the engine reads those sizes from the tensors).  ``sharp`` scales the
    left mixers' q and k gains, so that their softmax is peaked.  ``decisive_routing``: the routers' corrections lie
    1.5 apart in a random order (scores differ by less than 1), so that no rounding turns a choice (the weights still follow the scores).
    In a gla mixer the key matrix is the query matrix plus noise: a head's result is normed by itself, and at a
    sequence's first token it is v_0 (k_0 . q_0), whose sign would hang on the rounding of one dot product of
    unrelated vectors; with related ones the product is clearly positive and the comparison means something."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    std = std if std is not None else 1.0 / math.sqrt(W)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith(("left.q.norm", "left.k.norm")):
            w[name] = sharp * (1.0 + 0.1 * rng.standard_normal(shape))
        elif name.endswith(("mix.norm", "right.norm")):
            w[name] = 1.0 + 0.1 * rng.standard_normal(shape)
        elif leaf in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            w[name] = 0.1 * rng.standard_normal(shape)
        elif leaf in ("ls1", "ls2"):
            w[name] = 0.5 + 0.2 * rng.standard_normal(shape)
        elif leaf == "rel":
            w[name] = rng.standard_normal(shape)
        elif leaf == "correction":
            w[name] = 1.5 * rng.permutation(shape[0]) if decisive_routing else 0.05 * rng.standard_normal(shape)
        elif name.endswith("a2.b"):
            w[name] = 2.0 + rng.standard_normal(shape)
        elif name.endswith(".a2"):
            w[name] = rng.standard_normal(shape) / math.sqrt(shape[1])
        elif name.endswith(".o") or name.endswith(".down"):
            w[name] = rng.standard_normal(shape) / math.sqrt(shape[1])
        elif name == "embed":
            w[name] = rng.standard_normal(shape) * std
        else:
            w[name] = rng.standard_normal(shape) * std
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] == "gla":
            w[f"l{i}.mix.k"] = w[f"l{i}.mix.q"] + 0.5 * w[f"l{i}.mix.k"]
    return w

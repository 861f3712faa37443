"""The Retodra design on the GPU against the plain implementation of plain_retodra.py: each mechanism alone
(the recurrence with both kinds of decay under every cut, the group norm with its gates, the fused norms around the
residual stream, attention with planted keys at the window's edges and page borders, the router and the experts),
then whole models under every way of cutting the work (whole prompts, prefill against token-by-token decoding,
portions down to two tokens, unequal requests in one batch on few pages and slots that are used again, decoding far
past every window) and greedy generation through the engine's entry point, the replay program and the command line.
Configurations and weights are made here."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_retodra as plain
from helpers import MEAN_TOL, TOL, Replayer
from test_retodra_config import config, dense, gla, moe, par

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}

# key and value sizes that differ, three query heads per kv head, a window, a cap, identity experts, a constant decay of 1
CFG_A = config([gla(3, 16, 24, tau=4.0, rank=8, mlp=dense(96)),
                par(6, 2, 32, 16, 20, 2, 16, 32, (0.9, 1.0), scale=0.3, cap=12.0, reach=40, rows=12, mlp=moe(40, 5, 2, 3)),
                gla(2, 48, 8, tau=12.0, rank=4, mlp=moe(24, 3, 0, 1, limit=0.7)),
                par(2, 2, 64, 64, 33, 3, 40, 24, (0.5, 0.97, 0.999), scale=0.125, cap=30.0, reach=100, rows=32, ls=0.7, rs=1.1,
                    mlp=dense(72))])
# widths with odd factors, an odd vocabulary, no cap, one layer that sees every key and one that sees only itself, a layer
# without feed-forward, every router output chosen, one kv head, an odd number of bias rows, tau of 1, a decay of 0
CFG_B = config([par(4, 1, 24, 40, 0, 1, 8, 8, (0.0,), scale=0.4, cap=0.0, reach=9.5, rows=7, ls=1.0, rs=1.0, mlp=moe(16, 2, 1, 3)),
                gla(1, 8, 72, tau=1.0, rank=3, mlp=None),
                par(5, 5, 16, 16, 1, 2, 24, 8, (0.8, 0.6), scale=0.25, cap=5.0, reach=50, rows=16, mlp=dense(50)),
                gla(5, 20, 12, tau=9.0, rank=16, mlp=dense(56))], width=72, vocab=301, emb=1.0, eps=1e-6)
CONFIGS = {"A": (CFG_A, 16), "B": (CFG_B, 32)}
SHARP = {"float32": 3.0, "bfloat16": 1.0}
MARGIN = {"float32": 2e-5, "bfloat16": 6e-3}        # routing decisions closer than this are left to rounding


def compare(got, want, dtype, what=""):
    """Rows of logits against the plain implementation's.  float32: every row within TOL of the largest logit.
    bfloat16: the mean error within MEAN_TOL, and every row within TOL but for one row in fifty (at least one), which
    may reach twice that: a gated-linear-attention head's result is normed by itself, and where its terms nearly cancel
    the norm multiplies the rounding of the projections by the inverse of what is left."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    scale = np.abs(want).max()
    rows = np.abs(got - want).max(axis=1) / scale
    over = int((rows > TOL[dtype]).sum())
    allowed = 0 if dtype == "float32" else max(1, len(rows) // 50)
    assert over <= allowed and rows.max() <= 2 * TOL[dtype], (
        f"{what}: {over} of {len(rows)} rows over {TOL[dtype]:.0e} of the largest logit, worst {rows.max():.3e} at row {int(rows.argmax())}")
    assert np.abs(got - want).mean() <= MEAN_TOL[dtype] * scale, f"{what}: mean error {np.abs(got - want).mean() / scale:.3e}"


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def stored(a, dtype):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(DT[dtype]).float().numpy().astype(np.float64)


def make_weights(cfg, seed, dtype):
    # bfloat16 rounds the routers' inputs: there the corrections alone decide who is chosen (the mechanism's own test
    # and the float32 runs cover choices that follow the input)
    w = plain.random_weights(cfg, seed, sharp=SHARP[dtype], decisive_routing=dtype == "bfloat16")
    return plain.round_to_bf16(w) if dtype == "bfloat16" else w


def ids_of(cfg, w, n, seed, dtype):
    """Token ids whose routing decisions in the plain implementation all have a clear margin."""
    for k in range(40):
        ids = np.random.default_rng(seed * 1000 + k).integers(0, cfg["vocab"], size=n).tolist()
        if plain.routing_margin(cfg, w, ids) > MARGIN[dtype]:
            return ids
    raise AssertionError("no token sequence with clear routing found")


def build(tmp_path, name, dtype, num_pages, seed=1, max_seqs=4, graphs=False, cfg_page=None):
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.engine import factory
    cfg, page = cfg_page or CONFIGS[name]
    weights = make_weights(cfg, seed, dtype)
    folder = str(tmp_path / f"retodra_{name}_{dtype}")
    plain.write_model_folder(folder, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    ecfg = EngineConfig(model_path=folder, dtype=dtype, block_size=page, num_gpu_blocks=num_pages, max_num_seqs=max_seqs,
                        max_model_len=num_pages * page, max_num_batched_tokens=1024, use_cuda_graphs=graphs)
    model, cache, runner = factory.build(ecfg)
    return cfg, weights, folder, cache, runner


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dv,kind", [(3, 16, 24, "channel"), (2, 56, 64, "channel"), (1, 40, 8, "channel"), (2, 96, 80, "head"),
                                          (4, 64, 64, "head"), (1, 300, 33, "channel")])
def test_recurrence_under_every_cut_with_slots_used_again(dtype, H, dk, dv, kind):
    """Requests of unequal length fed in portions of changing size, several in one launch, slots given back and taken
    again (stale numbers in them zeroed by the test as the cache manager does at admission)."""
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(dk * dv)
    tau, scale = 3.0, 0.37
    lengths = {"a": 37, "b": 5, "c": 64, "d": 18}
    data, want = {}, {}
    bias = rng.standard_normal(H * dk).astype(np.float32) + 2
    lam = rng.uniform(0.5, 1.0, H).astype(np.float32)
    lam[0] = 1.0
    for r, n in lengths.items():
        q, k = stored(rng.standard_normal((n, H * dk)), dtype), stored(rng.standard_normal((n, H * dk)) / np.sqrt(dk), dtype)
        v, pre = stored(rng.standard_normal((n, H * dv)), dtype), stored(2 * rng.standard_normal((n, H * dk)), dtype)
        data[r] = (q, k, v, pre)
        outs = []
        for h in range(H):
            sl, vs = slice(h * dk, (h + 1) * dk), slice(h * dv, (h + 1) * dv)
            if kind == "channel":
                a = plain.sigmoid(pre[:, sl] + bias[sl]) ** (1 / tau)
                o, _ = plain.decayed_outer_recurrence(q[:, sl] * scale, k[:, sl], v[:, vs], a)
            else:
                o, _ = plain.decayed_outer_recurrence(plain.silu(q[:, sl]), plain.silu(k[:, sl]), plain.silu(v[:, vs]),
                                                      np.full((n, dk), float(lam[h])))
            outs.append(o)
        want[r] = np.concatenate(outs, axis=1)
    state = torch.full((2, H, dk, dv), 9.0, device="cuda")
    free, slot, at, got = [1, 0], {}, {}, {r: [] for r in lengths}
    schedule = [[("a", 1), ("b", 3)], [("b", 2), ("a", 2)], [("a", 17), ("c", 30)], [("c", 1), ("a", 16)], [("c", 33), ("a", 1)],
                [("d", 2)], [("d", 15)], [("d", 1)]]
    for step in schedule:
        for r, _ in step:
            if r not in slot:
                slot[r], at[r] = free.pop(), 0
                state[slot[r]].zero_()
        rows = [np.concatenate([data[r][i][at[r]: at[r] + n] for r, n in step]) for i in range(4)]
        # rows as column slices of one wide buffer, as a fused projection leaves them
        wide = np.concatenate([rows[0], rows[1], rows[2], np.zeros((len(rows[0]), 3))], axis=1)
        wd = dev(wide, DT[dtype])
        q, k, v = wd[:, : H * dk], wd[:, H * dk: 2 * H * dk], wd[:, 2 * H * dk: 2 * H * dk + H * dv]
        q_start = dev(np.cumsum([0] + [n for _, n in step]).astype(np.int32))
        slots = dev(np.array([slot[r] for r, _ in step], dtype=np.int32))
        out = torch.empty((len(rows[0]), H * dv), dtype=torch.float32, device="cuda")
        if kind == "channel":
            ops.decayed_state_scan(q, k, v, state, out, q_start, slots, len(step), num_heads=H, decay_pre=dev(rows[3], DT[dtype]),
                                   decay_bias=dev(bias), tau=tau, q_scale=scale)
        else:
            ops.decayed_state_scan(q, k, v, state, out, q_start, slots, len(step), num_heads=H, decay_const=dev(lam), silu_inputs=True)
        o, t0 = out.cpu().numpy(), 0
        for r, n in step:
            got[r].append(o[t0: t0 + n])
            t0 += n
            at[r] += n
            if at[r] == lengths[r]:
                free.append(slot.pop(r))
    for r in lengths:
        g = np.concatenate(got[r])
        assert np.abs(g - want[r]).max() <= 2e-5 * np.abs(want[r]).max(), (r, np.abs(g - want[r]).max(), np.abs(want[r]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dv,kind", [(2, 56, 64, "channel"), (3, 16, 24, "head"), (1, 72, 130, "channel")])
def test_recurrence_in_pieces_side_by_side(dtype, H, dk, dv, kind):
    """Long portions cut into pieces that run side by side and are joined: the same outputs and the same final state
    as token by token, for a long request beside a short one, over two steps."""
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(dk + dv)
    tau, scale = 2.0, 0.5
    lengths = {"a": 415, "b": 131}
    bias = rng.standard_normal(H * dk).astype(np.float32) + 3
    lam = rng.uniform(0.9, 1.0, H).astype(np.float32)
    data, want, final = {}, {}, {}
    for r, n in lengths.items():
        q, k = stored(rng.standard_normal((n, H * dk)), dtype), stored(rng.standard_normal((n, H * dk)) / np.sqrt(dk), dtype)
        v, pre = stored(rng.standard_normal((n, H * dv)), dtype), stored(2 * rng.standard_normal((n, H * dk)), dtype)
        data[r] = (q, k, v, pre)
        outs, ends = [], []
        for h in range(H):
            sl, vs = slice(h * dk, (h + 1) * dk), slice(h * dv, (h + 1) * dv)
            if kind == "channel":
                o, S = plain.decayed_outer_recurrence(q[:, sl] * scale, k[:, sl], v[:, vs], plain.sigmoid(pre[:, sl] + bias[sl]) ** (1 / tau))
            else:
                o, S = plain.decayed_outer_recurrence(plain.silu(q[:, sl]), plain.silu(k[:, sl]), plain.silu(v[:, vs]), np.full((n, dk), float(lam[h])))
            outs.append(o)
            ends.append(S)
        want[r], final[r] = np.concatenate(outs, axis=1), np.stack(ends)
    state = torch.zeros((2, H, dk, dv), device="cuda")
    slot, at, got = {"a": 1, "b": 0}, {"a": 0, "b": 0}, {"a": [], "b": []}
    for step in ([("a", 300), ("b", 1)], [("b", 130), ("a", 115)]):
        rows = [dev(np.concatenate([data[r][i][at[r]: at[r] + n] for r, n in step]), DT[dtype]) for i in range(4)]
        n_rows = rows[0].shape[0]
        starts, per_req = ops.scan_pieces([n for _, n in step])
        count = len(starts) - 1
        pieces = {"start": dev(starts), "req": dev(per_req), "slots": dev(np.arange(count, dtype=np.int32)), "count": count,
                  "state": torch.full((count, H, dk, dv), 7.0, device="cuda"), "qp": torch.empty((n_rows, H * dk), device="cuda"),
                  "dtot": torch.empty((count, H * dk), device="cuda")}
        q_start = dev(np.cumsum([0] + [n for _, n in step]).astype(np.int32))
        slots = dev(np.array([slot[r] for r, _ in step], dtype=np.int32))
        out = torch.empty((n_rows, H * dv), dtype=torch.float32, device="cuda")
        kw = dict(decay_pre=rows[3], decay_bias=dev(bias), tau=tau, q_scale=scale) if kind == "channel" else dict(decay_const=dev(lam), silu_inputs=True)
        ops.decayed_state_scan(rows[0], rows[1], rows[2], state, out, q_start, slots, len(step), num_heads=H, pieces=pieces, **kw)
        o, t0 = out.cpu().numpy(), 0
        for r, n in step:
            got[r].append(o[t0: t0 + n])
            t0 += n
            at[r] += n
    for r in lengths:
        g = np.concatenate(got[r])
        assert np.abs(g - want[r]).max() <= 3e-5 * np.abs(want[r]).max(), (r, np.abs(g - want[r]).max(), np.abs(want[r]).max())
        assert np.abs(state[slot[r]].cpu().numpy() - final[r]).max() <= 3e-5 * np.abs(final[r]).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dv,whole,act", [(3, 24, False, "silu"), (5, 40, True, "sigmoid"), (1, 72, False, "sigmoid"), (2, 320, True, "silu")])
def test_group_norm_with_gate(dtype, heads, dv, whole, act):
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(heads)
    n, C, eps = 7, heads * dv, 2e-5
    o = (3 * rng.standard_normal((n, C))).astype(np.float32)
    gate = stored(rng.standard_normal((n, C + 5)), dtype)
    w = (1 + 0.3 * rng.standard_normal(C if whole else dv)).astype(np.float32)
    out = torch.empty((n, C), dtype=DT[dtype], device="cuda")
    ops.gated_group_norm(dev(o), dev(gate, DT[dtype])[:, 2: 2 + C], dev(w), out, group=C if whole else dv, eps=eps, gate_act=act)
    g = gate[:, 2: 2 + C]
    f = plain.silu(g) if act == "silu" else plain.sigmoid(g)
    if whole:
        want = plain.plain_norm(o.astype(np.float64), w, eps) * f
    else:
        want = np.concatenate([plain.plain_norm(o[:, h * dv:(h + 1) * dv].astype(np.float64), w, eps) for h in range(heads)], axis=1) * f
    assert np.abs(out.float().cpu().numpy() - want).max() <= (3e-6 if dtype == "float32" else 1e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,with_next", [(72, True), (72, False), (2500, True), (320, True)])
def test_post_norm_addition_and_next_norm(dtype, width, with_next):
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(width)
    n, eps, eps2 = 5, 1e-5, 3e-6
    y = stored(4 * rng.standard_normal((n, width)), dtype)
    x = rng.standard_normal((n, width)).astype(np.float32)
    w1, ls, w2 = (0.2 * rng.standard_normal(width) for _ in range(3))
    gain = ((1 + w1) * (0.5 + ls)).astype(np.float32)
    xd = dev(x)
    nxt = torch.empty((n, width), dtype=DT[dtype], device="cuda") if with_next else None
    ops.norm_residual_norm(dev(y, DT[dtype]), dev(gain), xd, eps, next_gain=dev((1 + w2).astype(np.float32)) if with_next else None,
                           next_out=nxt, next_eps=eps2)
    want = x + (0.5 + ls).astype(np.float32) * plain.layer_norm(y, w1.astype(np.float32), eps)
    assert np.abs(xd.cpu().numpy() - want).max() <= 3e-6 * np.abs(want).max()
    if with_next:
        want2 = plain.layer_norm(want, w2.astype(np.float32), eps2)
        assert np.abs(nxt.float().cpu().numpy() - want2).max() <= (3e-6 if dtype == "float32" else 1e-2) * np.abs(want2).max()


def attention_harness(att, page, pages, max_len, max_seqs=3):
    """The engine's cache manager and step packing around one mixer: steps come out of ModelRunner._prepare with the
    work lists the mixer asked for."""
    import types
    from vllm_cpp_b200.cache.manager import CacheManager
    from vllm_cpp_b200.engine.runner import ModelRunner
    cache = CacheManager([att.cache_spec()], page, pages, max_seqs, att.dtype, "cuda")
    fake = types.SimpleNamespace(vocab=100, blocks=[types.SimpleNamespace(parts={"mixer": att})], final_norm=None,
                                 spec=types.SimpleNamespace(max_position_embeddings=max_len))
    return cache, ModelRunner(fake, cache, 1024, max_seqs, max_len, torch.device("cuda", 0))


@pytest.mark.parametrize("dtype,H,G,dk,dv,window,page,cap,plain_kernel", [
    ("float32", 4, 2, 32, 16, 20, 16, 12.0, True), ("float32", 3, 3, 24, 40, 37, 16, 0.0, True), ("float32", 2, 1, 8, 8, 0, 16, 3.0, True),
    ("bfloat16", 6, 2, 64, 64, 70, 16, 18.0, False), ("bfloat16", 6, 2, 64, 64, 70, 16, 18.0, True), ("bfloat16", 2, 1, 128, 128, 33, 32, 8.0, False),
    ("bfloat16", 4, 4, 64, 64, 1, 16, 5.0, False), ("bfloat16", 20, 1, 64, 64, 0, 16, 0.0, False), ("bfloat16", 6, 2, 128, 128, 130, 16, 30.0, False),
    ("bfloat16", 3, 1, 48, 80, 50, 16, 10.0, True)])
def test_attention_with_planted_keys(dtype, H, G, dk, dv, window, page, cap, plain_kernel):
    """The mixer itself (its products are identities, so its input rows are q, k, v and the gate) through the cache
    manager's pages.  The bias table is made so that the keys at the window's far edge outweigh all others: the row of
    the last distance inside the window gets a large bonus and the row of the first distance outside a larger one
    (without a window, the last row, which every distance from the reach on reads: keys far away).  A window that is
    one token off, a page border that is misread, a page that the window gave back or a bias row taken one distance
    off then changes the result beyond any rounding.  Two requests, prompt portions beside single tokens; bfloat16
    heads of 64 and 128 run the tensor-core kernels unless the case asks for the plain one."""
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.runner import StepEntry
    from vllm_cpp_b200.parts.base import Workspace
    from vllm_cpp_b200.parts.biased_attention import BiasedWindowAttention
    rng = np.random.default_rng(window + dk)
    T, rows_rel, scale, eps = 150, 32, 0.5, 1e-5
    reach = float(window + 5) if window > 20 else 40.0
    rel = rng.standard_normal((rows_rel, H))
    if window > 1:
        rel[plain.distance_bucket(window - 1, rows_rel, reach)] += 6.0
        if plain.distance_bucket(window, rows_rel, reach) != plain.distance_bucket(window - 1, rows_rel, reach):
            rel[plain.distance_bucket(window, rows_rel, reach)] += 9.0
    elif window == 0:
        rel[rows_rel - 1] += 6.0
    rel = stored(rel, "bfloat16")
    width = H * dk + G * dk + G * dv + H * dv
    att = BiasedWindowAttention(width, H, G, dk, dv, scale, cap, window, reach, eps, DT[dtype], "cuda")
    sharp = 2.0 / np.sqrt(scale * np.sqrt(dk))        # normed rows have unit mean square: scores of standard deviation 4
    wq = ((1 + 0.1 * rng.standard_normal(H * dk)) * sharp).astype(np.float32)
    wk = ((1 + 0.1 * rng.standard_normal(G * dk)) * sharp).astype(np.float32)
    eye = np.eye(width, dtype=np.float32)
    o0, o1, o2, o3 = H * dk, H * dk + G * dk, H * dk + G * dk + G * dv, width
    att.load_params({"q": dev(eye[:o0], DT[dtype]), "k": dev(eye[o0:o1], DT[dtype]), "v": dev(eye[o1:o2], DT[dtype]),
                     "g": dev(eye[o2:o3], DT[dtype]), "o": dev(eye[:, : H * dv], DT[dtype]), "q.norm": dev(wq), "k.norm": dev(wk),
                     "rel": dev(rel.astype(np.float32))})
    if plain_kernel:
        att._tensor_core_path = lambda: False
    else:
        assert att._tensor_core_path()
    cache, runner = attention_harness(att, page, pages=2 * (-(-T // page)) + 2, max_len=T + page)
    ws = Workspace("cuda")
    x = {r: stored(rng.standard_normal((T, width)), dtype) for r in ("a", "b")}
    want = {}
    for r in x:
        q, k, v, gate = x[r][:, :o0], x[r][:, o0:o1], x[r][:, o1:o2], x[r][:, o2:]
        qn, kn = stored(plain.plain_norm(q, wq, eps), dtype), stored(plain.plain_norm(k, wk, eps), dtype)
        want[r] = plain.capped_biased_attention(qn, kn, v, rel, H, G, window, cap, scale, reach) * plain.sigmoid(gate)
        if r == "a" and window > 1:
            # the planted rows matter: one key more or fewer at the window's far edge moves the result far beyond rounding
            for other_window in (window + 1, window - 1):
                other = plain.capped_biased_attention(qn, kn, v, rel, H, G, other_window, cap, scale, reach) * plain.sigmoid(gate)
                assert np.abs(other - want[r]).max() > 0.1 * np.abs(want[r]).max()
    got = {r: np.zeros((T, H * dv)) for r in x}
    at = {"a": 0, "b": 0}
    steps = [[("a", 70), ("b", 3)], [("b", 90), ("a", 1)]] + [[("a", 1), ("b", 1)]] * 57 + [[("a", 22)]]
    for entries in steps:
        for r, _ in entries:
            if r not in cache.requests:
                cache.add_request(r)
        step = runner._prepare([StepEntry(r, [0] * n, []) for r, n in entries])
        rows = dev(np.concatenate([x[r][at[r]: at[r] + n] for r, n in entries]), DT[dtype])
        out = torch.empty_like(rows)
        ws.reset()
        att.forward(rows, out, step, runner.views[0], True, ws)
        o, t0 = out.float().cpu().numpy(), 0
        for r, n in entries:
            got[r][at[r]: at[r] + n] = o[t0: t0 + n, : H * dv]
            t0 += n
            at[r] += n
            cache.commit(r, n)
    ops.check_status()
    for r in x:
        n = at[r]
        err = np.abs(got[r][:n] - want[r][:n]).max(axis=1)
        tol = (2e-5 if dtype == "float32" else 2.5e-2) * np.abs(want[r]).max()
        assert err.max() <= tol, f"{r}: first wrong token {int(np.argmax(err > tol))}, error {err.max():.3e} of {np.abs(want[r]).max():.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,width,ff,experts,identity,top", [(9, 72, 40, 5, 2, 3), (150, 64, 24, 3, 0, 1), (33, 80, 16, 2, 1, 3), (700, 48, 20, 4, 1, 2)])
def test_routed_experts(dtype, n, width, ff, experts, identity, top):
    """Router (scores over all outputs, choice by score + correction, plain scores as weights), identity experts, the
    clamped activation, tiles of 16 and of 64 rows, experts that get no token."""
    from vllm_cpp_b200.parts.base import Workspace
    from vllm_cpp_b200.parts.moe import RoutedExperts
    rng = np.random.default_rng(n)
    p, limit = "x.", 0.8
    mlp = {"expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}
    w = {p + "router": 3 * rng.standard_normal((experts + identity, width)) / np.sqrt(width),
         p + "correction": 0.2 * rng.standard_normal(experts + identity)}
    if experts > 3:
        w[p + "router"][1] -= 50.0 / np.sqrt(width)              # an expert that no token reaches
    for e in range(experts):
        w[f"{p}e{e}.gate"] = stored(2 * rng.standard_normal((ff, width)) / np.sqrt(width), dtype)
        w[f"{p}e{e}.up"] = stored(2 * rng.standard_normal((ff, width)) / np.sqrt(width), dtype)
        w[f"{p}e{e}.down"] = stored(rng.standard_normal((width, ff)) / np.sqrt(ff), dtype)
    w[p + "router"] = stored(w[p + "router"], "bfloat16")
    w[p + "correction"] = stored(w[p + "correction"], "bfloat16")
    h = stored(rng.standard_normal((n, width)) + 1.0, dtype)
    margins = []
    want = plain.moe_ff(w, p, mlp, h, margins)
    clear = np.asarray(margins) > 1e-4 if margins else np.ones(n, dtype=bool)
    part = RoutedExperts(width, ff, experts, identity, top, limit, DT[dtype], "cuda")
    part.load_params({k[len(p):]: dev(v.astype(np.float32), DT[dtype] if k[len(p)] == "e" else torch.float32) for k, v in w.items()})
    out = torch.empty((n, width), dtype=DT[dtype], device="cuda")
    ws = Workspace("cuda")
    part.forward(dev(h, DT[dtype]), out, None, ws)
    got = out.float().cpu().numpy()
    assert clear.sum() > 0.9 * n
    err = np.abs(got - want)[clear].max()
    assert err <= (1e-5 if dtype == "float32" else 2e-2) * np.abs(want).max(), err


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompts_and_the_first_tokens(tmp_path, name, dtype):
    cfg, w, _, cache, runner = build(tmp_path, name, dtype, 16)
    rp = Replayer(runner, cache)
    for n in (1, 2, 3, 47, 130):
        ids = ids_of(cfg, w, n, n, dtype)
        rp.step([(f"r{n}", ids, range(n))], end=[f"r{n}"])
        compare(rp.logits_of(f"r{n}", range(n)), plain.forward(cfg, w, ids), dtype, f"{name} whole {n}")
    assert cache.num_free_pages() == 16


# models of one kind of layer: no pages at all (state slots only), and pages in every layer
CFG_ONLY_GLA = config([gla(2, 16, 32, tau=8.0, rank=5, mlp=dense(40)), gla(4, 8, 16, tau=2.0, rank=2, mlp=None)], width=48, vocab=97)
CFG_ONLY_PARALLEL = config([par(2, 1, 16, 16, 9, 2, 8, 16, (0.7, 0.95), mlp=moe(24, 2, 1, 2)),
                            par(4, 2, 8, 24, 40, 1, 16, 8, (0.99,), cap=0.0, mlp=dense(64))], width=40, vocab=120, emb=6.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["gla", "parallel"])
def test_models_of_one_kind_of_layer(tmp_path, which, dtype):
    cfg = CFG_ONLY_GLA if which == "gla" else CFG_ONLY_PARALLEL
    cfg, w, _, cache, runner = build(tmp_path, which, dtype, 12, cfg_page=(cfg, 16))
    assert bool(cache.paged) == (which == "parallel")
    rp = Replayer(runner, cache)
    n = 140
    ids = ids_of(cfg, w, n, 3, dtype)
    want = plain.forward(cfg, w, ids)
    t = 0
    for s in (50, 1, 1, 80, 2, 1, 1, 1, 1, 1, 1):
        rp.step([("r", ids[t: t + s], range(s))])
        t += s
    assert t == n
    cache.free_request("r")
    compare(rp.logits_of("r", range(n)), want, dtype, f"only {which}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_prefill_against_token_by_token_and_long_decoding(tmp_path, name, dtype):
    """The same tokens as one portion and one by one (far past every window and many pages) give the same logits."""
    cfg, w, _, cache, runner = build(tmp_path, name, dtype, 24)
    n = 170
    ids = ids_of(cfg, w, n, 7, dtype)
    want = plain.forward(cfg, w, ids)
    rp = Replayer(runner, cache)
    rp.step([("p", ids, range(n))], end=["p"])
    compare(rp.logits_of("p", range(n)), want, dtype, f"{name} prefill")
    rp.step([("d", ids[:9], range(9))])
    for t in range(9, n):
        rp.step([("d", ids[t: t + 1], [0])])
    compare(rp.logits_of("d", range(n)), want, dtype, f"{name} decode")
    a, b = rp.logits_of("p", range(n)), rp.logits_of("d", range(n))
    assert np.abs(a - b).max() <= (2e-5 if dtype == "float32" else 3e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_down_to_two_tokens(tmp_path, name, dtype):
    cfg, w, _, cache, runner = build(tmp_path, name, dtype, 24)
    n = 150
    ids = ids_of(cfg, w, n, 9, dtype)
    want = plain.forward(cfg, w, ids)
    for k, sizes in enumerate(([2] * 75, [5, 2, 31, 2, 17, 64, 3, 26], [16, 16, 1, 15, 33, 2, 67], [149, 1])):
        assert sum(sizes) == n
        rp, t = Replayer(runner, cache), 0
        for s in sizes:
            rp.step([(f"c{k}", ids[t: t + s], range(s))])
            t += s
        cache.free_request(f"c{k}")
        compare(rp.logits_of(f"c{k}", range(n)), want, dtype, f"{name} portions {sizes[:4]}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_requests_together_on_few_pages(tmp_path, name, dtype):
    """Up to three live requests of unequal length, portions beside single tokens, on so few pages and slots that
    both are used again by later requests; every request's logits are those it has alone."""
    cfg, w, _, cache, runner = build(tmp_path, name, dtype, 28, max_seqs=3)
    rng = np.random.default_rng(3)
    lengths = {"a": 90, "b": 3, "c": 140, "d": 33, "e": 64, "f": 1, "g": 120}
    ids = {r: ids_of(cfg, w, n, 40 + i, dtype) for i, (r, n) in enumerate(lengths.items())}
    want = {r: plain.forward(cfg, w, ids[r]) for r in ids}
    rp = Replayer(runner, cache)
    waiting, live, at = list(lengths), [], {}
    slots_seen = []
    while waiting or live:
        while waiting and len(live) < 3:
            r = waiting.pop(0)
            live.append(r)
            at[r] = 0
        entries, end = [], []
        for r in live:
            s = int(min(lengths[r] - at[r], 1 if at[r] > 40 else rng.choice([1, 2, 7, 16, 29])))
            entries.append((r, ids[r][at[r]: at[r] + s], range(s)))
            at[r] += s
            if at[r] == lengths[r]:
                end.append(r)
        rp.step(entries, end=[])
        slots_seen += [cache.slot(r) for r, _, _ in entries]
        for r in end:
            cache.free_request(r)
            compare(rp.logits_of(r, range(lengths[r])), want[r], dtype, f"{name} mixed {r}")
            live.remove(r)
    assert cache.num_free_pages() == 28 and len(set(slots_seen)) == 3


# larger layers: heads of 128 and 64 on the tensor-core attention kernels, recurrences with 128 and 80 key channels,
# experts whose tiles are 64 and 16 rows high, portions that run in pieces
CFG_WIDE = config([gla(4, 128, 64, tau=8.0, rank=24, mlp=dense(640)),
                   par(8, 2, 128, 128, 200, 4, 64, 96, (0.9, 0.97, 0.99, 1.0), scale=0.09, cap=25.0, reach=300, rows=40, mlp=moe(192, 6, 1, 2)),
                   gla(2, 80, 128, tau=3.0, rank=7, mlp=moe(128, 3, 0, 1)),
                   par(4, 4, 64, 64, 50, 2, 32, 64, (0.95, 0.8), scale=0.125, cap=0.0, reach=64, rows=20, mlp=dense(512))],
                  width=384, vocab=700, emb=4.0)


def test_bfloat16_beside_float32_at_larger_sizes(tmp_path):
    """The same (bfloat16-valued) weights through the float32 engine, which the small configurations anchor to the plain
    implementation, and through the bfloat16 engine with its tensor-core kernels: a prompt of 450 tokens in two portions,
    then single tokens, beside a second request."""
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.engine import factory
    w = plain.round_to_bf16(plain.random_weights(CFG_WIDE, 3, sharp=1.0, decisive_routing=True))
    rng = np.random.default_rng(5)
    ids = {"a": rng.integers(0, 700, size=480).tolist(), "b": rng.integers(0, 700, size=70).tolist()}
    steps = [[("a", 300)], [("a", 150), ("b", 40)]] + [[("a", 1), ("b", 1)]] * 30
    got = {}
    for dtype in ("float32", "bfloat16"):
        folder = str(tmp_path / dtype)
        plain.write_model_folder(folder, CFG_WIDE, w, store="BF16" if dtype == "bfloat16" else "F32")
        ecfg = EngineConfig(model_path=folder, dtype=dtype, block_size=16, num_gpu_blocks=48, max_num_seqs=2, max_model_len=768,
                            max_num_batched_tokens=512, use_cuda_graphs=False)
        _, cache, runner = factory.build(ecfg)
        rp, at = Replayer(runner, cache), {"a": 0, "b": 0}
        for step in steps:
            rp.step([(r, ids[r][at[r]: at[r] + n], range(n)) for r, n in step])
            for r, n in step:
                at[r] += n
        got[dtype] = {r: rp.logits_of(r, range(at[r])) for r in ids}
        del runner, cache
    for r in ids:
        compare(got["bfloat16"][r], got["float32"][r], "bfloat16", f"larger sizes {r}")


@pytest.mark.parametrize("dtype,name,pages", [("float32", "A", 24), ("bfloat16", "A", 24), ("float32", "B", 7)])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype, name, pages):
    """LLM.generate: the scheduler cuts the prompts under a small token budget, decode steps are captured and
    replayed; every generated token is the plain implementation's best, or within rounding of it.  On 7 pages (of
    a model whose first layer keeps every key) requests are preempted and fed again from their first token: their
    state slots start from zero again."""
    from vllm_cpp_b200 import LLM, SamplingParams
    cfg, page = CONFIGS[name]
    weights = make_weights(cfg, 5, dtype)
    folder = str(tmp_path / f"gen_{dtype}")
    plain.write_model_folder(folder, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    llm = LLM(folder, dtype=dtype, block_size=page, num_gpu_blocks=pages, max_num_seqs=3, max_model_len=pages * page,
              max_num_batched_tokens=48)
    prompts = [np.random.default_rng(500 + n).integers(0, cfg["vocab"], size=n).tolist() for n in (3, 41, 100, 17)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=30, temperature=0.0, ignore_eos=True))
    if pages < 24:
        assert llm.engine.scheduler.num_preemptions > 0
    for p, o in zip(prompts, outs):
        assert len(o) == 30
        seq = list(p)
        for tok in o:
            if plain.routing_margin(cfg, weights, seq) < MARGIN[dtype]:
                break                                  # from a routing decision that rounding can turn on, nothing is compared
            logits = plain.forward(cfg, weights, seq)[-1]
            best = plain.greedy(logits)
            gap = (logits[best] - logits[tok]) / np.abs(logits).max()
            assert tok == best or gap < (1e-3 if dtype == "float32" else 5e-2), (dtype, len(p), tok, best, gap)
            seq.append(tok)


def random_retodra_config(rng):
    """Sizes with odd factors everywhere, both kinds of layer in any order, every kind of feed-forward or none, windows
    from one token to longer than any prompt, with and without cap.  (Value heads of a gla mixer have eight channels
    and more: a head's result is normed by itself, and the norm of three or four channels is too often nearly zero.)"""
    width = int(rng.choice([36, 50, 64, 90, 104, 136]))
    layers = []
    for _ in range(int(rng.integers(1, 5))):
        pick = rng.random()
        mlp = None if pick < 0.2 else dense(int(rng.integers(20, 160))) if pick < 0.6 else None
        if pick >= 0.6:
            experts, identity = int(rng.integers(1, 7)), int(rng.integers(0, 3))
            mlp = moe(int(rng.integers(8, 60)), experts, identity, int(rng.integers(1, experts + identity + 1)), limit=float(rng.uniform(0.5, 3)))
        if rng.random() < 0.5:
            layers.append(gla(int(rng.integers(1, 7)), int(rng.choice([4, 8, 12, 16, 40, 72])), int(rng.choice([8, 16, 33, 64])),
                              tau=float(rng.choice([1.0, 4.0, 12.0])), rank=int(rng.integers(1, 20)), mlp=mlp))
        else:
            g = int(rng.integers(1, 4))
            rh = int(rng.integers(1, 5))
            rows = int(rng.choice([4, 7, 12, 32]))
            layers.append(par(g * int(rng.integers(1, 4)), g, int(rng.choice([8, 16, 24, 64])), int(rng.choice([8, 12, 64])),
                              int(rng.choice([0, 1, 2, 17, 64, 300])), rh, int(rng.choice([8, 16, 20])), int(rng.choice([4, 16, 24])),
                              [float(x) for x in rng.uniform(0.3, 1.0, rh)], scale=float(rng.uniform(0.1, 0.4)),
                              cap=float(rng.choice([0.0, 6.0, 25.0])), reach=float(rng.uniform(rows // 2 + 1, 200)), rows=rows,
                              ls=float(rng.uniform(0.5, 1.5)), rs=float(rng.uniform(0.5, 1.5)), mlp=mlp))
    return config(layers, width=width, vocab=int(rng.integers(40, 500)), emb=float(rng.uniform(0.5, 8.0)),
                  eps=float(rng.choice([1e-5, 1e-6, 1e-4])))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [21, 22, 23, 24])
def test_the_replay_program_on_configurations_drawn_at_random(tmp_path, seed, dtype):
    """bin/trace_run as a user calls it, on a configuration drawn at random, under a schedule drawn at random: JSON
    lines in, <step>.f32 files and 'done' lines out; a pool of as many tokens as live requests hold, four slots."""
    rng = np.random.default_rng(seed)
    cfg = random_retodra_config(rng)
    weights = make_weights(cfg, seed, dtype)
    folder = str(tmp_path / "model")
    plain.write_model_folder(folder, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    lengths = {f"q{i}": int(n) for i, n in enumerate(rng.choice([1, 2, 30, 77, 150, 64], size=6))}
    ids = {r: ids_of(cfg, weights, n, seed * 100 + i, dtype) for i, (r, n) in enumerate(lengths.items())}
    waiting, live, at, lines, asked = list(lengths), [], {}, [], []
    most = 0
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
            at[live[-1]] = 0
        most = max(most, sum(-(-lengths[r] // 64) * 64 for r in live))
        entries, end, rows = [], [], []
        for r in live:
            s = int(min(lengths[r] - at[r], 1 if at[r] > 50 else rng.choice([1, 2, 3, 16, 37, 64])))
            want = sorted(set(int(x) for x in rng.integers(0, s, size=min(s, 3))))
            entries.append({"id": r, "tokens": ids[r][at[r]: at[r] + s], "want": want})
            rows += [(r, at[r] + x) for x in want]
            at[r] += s
            if at[r] == lengths[r]:
                end.append(r)
        lines.append({"step": len(lines), "entries": entries, "end": end})
        asked.append(rows)
        live = [r for r in live if r not in end]
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(most)],
                       input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(lines))]
    want = {r: plain.forward(cfg, weights, ids[r]) for r in ids}
    got_rows, want_rows = [], []
    for i, rows in enumerate(asked):
        if rows:
            got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
            assert got.shape[0] == len(rows), f"step {i}: {got.shape[0]} rows written, {len(rows)} asked for"
            got_rows.append(got)
            want_rows.append(np.stack([want[r][t] for r, t in rows]))
    # all steps' rows together: a step has one to three rows a request, too few for a mean to mean anything
    compare(np.concatenate(got_rows), np.concatenate(want_rows), dtype, f"seed {seed}: {cfg['layers']}")


def test_command_line_and_sampling_options(tmp_path):
    """python -m vllm_cpp_b200.engine.cli on a Retodra folder, the architecture taken from config.json or named by
    --arch: greedy ids are the plain implementation's; seeded sampling gives ids of the vocabulary, the same when asked again."""
    cfg, page = CONFIGS["B"]
    weights = make_weights(cfg, 8, "float32")
    folder = str(tmp_path / "cli_model")
    plain.write_model_folder(folder, cfg, weights, store="F32")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = ids_of(cfg, weights, 21, 3, "float32")
    base = [sys.executable, "-m", "vllm_cpp_b200.engine.cli", "--model", folder, "--dtype", "float32", "--num-gpu-blocks", "24",
            "--max-num-seqs", "2", "--max-model-len", "128", "--max-num-batched-tokens", "64", "--ignore-eos",
            "--prompt-ids", ",".join(map(str, prompt))]
    env = dict(os.environ, PYTHONPATH=root)

    def run(extra):
        p = subprocess.run(base + extra, capture_output=True, text=True, timeout=600, env=env, cwd=root)
        assert p.returncode == 0, p.stderr[-3000:]
        return [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")]

    greedy = run(["--max-tokens", "6", "--temperature", "0"])
    seq = list(prompt)
    for tok in greedy:
        logits = plain.forward(cfg, weights, seq)[-1]
        assert tok == plain.greedy(logits) or (logits.max() - logits[tok]) / np.abs(logits).max() < 1e-3
        seq.append(tok)
    options = ["--arch", "retodra", "--max-tokens", "12", "--temperature", "0.9", "--top-k", "20", "--top-p", "0.9",
               "--repetition-penalty", "1.2", "--sample-seed", "5"]
    drawn = run(options)
    assert len(drawn) == 12 and all(0 <= t < cfg["vocab"] for t in drawn)
    assert run(options) == drawn

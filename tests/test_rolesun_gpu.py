"""The Rolesun design on the GPU against the plain implementation of plain_rolesun.py: each mechanism
alone, then whole models under every way of cutting the work (whole prompts, prefill against token-by-token
decoding, portions down to two tokens, unequal requests mixed in one batch on few pages and slots that are
used again, decoding far past every window) and greedy generation through the engine's entry point.
Configurations and weights are made here; queries are scaled up so that a wrong or missing key shows."""
import types

import numpy as np
import pytest
import torch

import plain_rolesun as plain
from helpers import Replayer, compare, kv_pos
from test_rolesun_config import config, mixer

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}

# ranks 64 and 128 (tensor-core attention in bfloat16), a layer without feed-forward, layers that read layer 0's
# latents through narrower and wider windows than its own, one head, value size unlike the key size
CFG_A = config([(mixer(3, 16, 24, 64, 20), 96), (mixer(2, 8, 8, 64, 33, kv_from=0), None), (mixer(4, 16, 16, 128, 70), 80),
                (mixer(1, 8, 12, 64, 12, kv_from=0), 48)])
# widths with odd factors, an odd vocabulary, ranks without a tensor-core kernel (40) and beyond 256, a window of one
# token, a layer that sees all keys, multiplier and scales of 1
CFG_B = config([(mixer(5, 12, 20, 40, 1), 56), (mixer(2, 24, 8, 320, 45), 100), (dict(mixer(3, 8, 8, 40, 9, kv_from=0), mask=None), 64)],
               width=72, vocab=301, mult=1.0, logit_scale=1.0, emb=1.0, eps=1e-6)
CONFIGS = {"A": (CFG_A, 16), "B": (CFG_B, 32)}
SHARP = {"float32": 1.5, "bfloat16": 0.5}


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def stored(a, dtype):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(DT[dtype]).float().numpy().astype(np.float64)


def build(tmp_path, name, dtype, num_pages, seed=1, max_seqs=4, graphs=False):
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.engine import factory
    cfg, page = CONFIGS[name]
    weights = plain.random_weights(cfg, seed, sharp=SHARP[dtype])
    if dtype == "bfloat16":
        weights = plain.round_to_bf16(weights)
    folder = str(tmp_path / f"rolesun_{name}_{dtype}")
    plain.write_model_folder(folder, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    ecfg = EngineConfig(model_path=folder, dtype=dtype, block_size=page, num_gpu_blocks=num_pages, max_num_seqs=max_seqs,
                        max_model_len=num_pages * page, max_num_batched_tokens=1024, use_cuda_graphs=graphs)
    model, cache, runner = factory.build(ecfg)
    return cfg, weights, folder, cache, runner


def ids_of(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_with_scale_and_sinusoid(dtype):
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(0)
    width, vocab = 50, 31
    cfg = {"width": width, "embedding": {"scale": 2.5}}
    table = stored(rng.standard_normal((vocab, width)), dtype)
    ids = rng.integers(0, vocab, size=9)
    pos = np.array([0, 1, 2, 3, 500, 501, 4095, 7, 8])
    inv = np.power(10000.0, -2.0 * np.arange(width // 2) / width).astype(np.float32)
    out = torch.empty((9, width), dtype=torch.float32, device="cuda")
    ops.embedding_sinusoid(dev(table, DT[dtype]), dev(ids.astype(np.int32)), dev(pos.astype(np.int32)), dev(inv), out, 2.5)
    want = np.stack([plain.embed(cfg, {"embed": table}, [i], first_position=p)[0] for i, p in zip(ids, pos)])
    # the angle is a float product: at position 4095 its rounding alone moves a sine by 2e-4
    assert np.abs(out.cpu().numpy() - want).max() <= 5e-4
    assert np.abs(out.cpu().numpy()[:4] - want[:4]).max() <= 2e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_shift_keeps_the_last_row_between_steps(dtype):
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(1)
    width = 40
    mu = rng.uniform(0, 1, width).astype(np.float32)
    seqs = {"a": rng.standard_normal((11, width)).astype(np.float32), "b": rng.standard_normal((7, width)).astype(np.float32)}
    want = {k: plain.token_shift(v.astype(np.float64), mu.astype(np.float64)) for k, v in seqs.items()}
    state = torch.full((3, width), 77.0, device="cuda")            # stale rows: position 0 must not read them
    slots = {"a": 2, "b": 0}
    at = {"a": 0, "b": 0}
    got = {"a": [], "b": []}
    for step in ([("a", 3), ("b", 1)], [("b", 2), ("a", 1)], [("a", 5)], [("a", 2), ("b", 4)]):
        rows = np.concatenate([seqs[r][at[r]: at[r] + n] for r, n in step])
        q_start = np.cumsum([0] + [n for _, n in step]).astype(np.int32)
        req_of = np.concatenate([[i] * n for i, (_, n) in enumerate(step)]).astype(np.int32)
        pos = np.concatenate([np.arange(at[r], at[r] + n) for r, n in step]).astype(np.int32)
        sl = np.array([slots[r] for r, _ in step], dtype=np.int32)
        shifted = torch.empty(rows.shape, dtype=DT[dtype], device="cuda")
        plain_out = torch.empty(rows.shape, dtype=DT[dtype], device="cuda")
        ops.token_shift(dev(rows), dev(mu), state, shifted, plain_out, dev(q_start), dev(req_of), dev(pos), dev(sl))
        s = shifted.float().cpu().numpy()
        assert np.abs(plain_out.float().cpu().numpy() - rows).max() <= (0 if dtype == "float32" else 2e-2)
        for i, (r, n) in enumerate(step):
            got[r].append(s[q_start[i]: q_start[i + 1]])
            at[r] += n
    for r in seqs:
        assert np.abs(np.concatenate(got[r]) - want[r]).max() <= (1e-6 if dtype == "float32" else 3e-2), r
    assert np.array_equal(state.cpu().numpy()[2], seqs["a"][-1]) and np.array_equal(state.cpu().numpy()[0], seqs["b"][-1])
    assert (state.cpu().numpy()[1] == 77.0).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("vector_gain", [False, True])
@pytest.mark.parametrize("gated", [False, True])
def test_gate_norm_and_residual_addition(dtype, vector_gain, gated):
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(2)
    n, width, mult, eps = 6, 104, 0.6, 3e-5
    y = stored(2 * rng.standard_normal((n, width)), dtype)
    a = stored(rng.standard_normal((n, width)), dtype)
    b = rng.standard_normal(width).astype(np.float32)
    gain = (1 + 0.3 * rng.standard_normal(width if vector_gain else 1)).astype(np.float32)
    x = rng.standard_normal((n, width)).astype(np.float32)
    xd = dev(x)
    out = torch.empty((n, width), dtype=DT[dtype], device="cuda")
    ops.gated_norm_residual(dev(y, DT[dtype]), dev(a, DT[dtype]) if gated else None, dev(b) if gated else None, dev(gain), xd, out, mult, eps)
    z = y * plain.sigmoid(a + b) if gated else y
    want = x + mult * plain.rms(z, eps) * gain.astype(np.float64)
    assert np.abs(xd.cpu().numpy() - want).max() <= 3e-6 * np.abs(want).max()          # float32 in both precisions
    assert np.abs(out.float().cpu().numpy() - want).max() <= (3e-6 if dtype == "float32" else 1e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n", [5, 70, 200])
@pytest.mark.parametrize("N,K", [(40, 24), (40, 32), (136, 80)])
def test_headwise_products(dtype, n, N, K):
    """Both kernels (the plain one; tensor cores for short bfloat16 steps when K is a multiple of 16) and the
    library's batched product for long bfloat16 portions."""
    from vllm_cpp_b200.csrc import ops
    rng = np.random.default_rng(3)
    heads = 3
    x = stored(rng.standard_normal((n, heads * K + 8)), dtype)                         # a column slice of wider rows
    w = stored(rng.standard_normal((heads, N, K)) / 5, dtype)
    g = stored(rng.standard_normal((n, heads * N)), dtype)
    want = np.einsum("thk,hnk->thn", x[:, 8:].reshape(n, heads, K), w).reshape(n, heads * N)
    xd = dev(x, DT[dtype])
    for gate in (None, g):
        out = torch.empty((n, heads * N), dtype=DT[dtype], device="cuda")
        ops.headwise_linear(xd[:, 8:], dev(w, DT[dtype]), out, None if gate is None else dev(gate, DT[dtype]))
        ref = want if gate is None else want * plain.sigmoid(gate)
        assert np.abs(out.float().cpu().numpy() - ref).max() <= (1e-5 if dtype == "float32" else 2e-2) * np.abs(ref).max()


def attention_harness(att, page, pages, max_len, max_seqs=3):
    from vllm_cpp_b200.cache.manager import CacheManager
    from vllm_cpp_b200.engine.runner import ModelRunner
    cache = CacheManager([att.cache_spec()], page, pages, max_seqs, att.dtype, "cuda")
    fake = types.SimpleNamespace(vocab=100, blocks=[types.SimpleNamespace(parts={"mixer": att})], final_norm=None,
                                 spec=types.SimpleNamespace(max_position_embeddings=max_len))
    return cache, ModelRunner(fake, cache, 1024, max_seqs, max_len, torch.device("cuda", 0))


@pytest.mark.parametrize("dtype,rank,heads,window,page", [("float32", 48, 3, 37, 16), ("float32", 320, 2, 100, 16),
                                                          ("bfloat16", 64, 6, 37, 16), ("bfloat16", 128, 5, 130, 32),
                                                          ("bfloat16", 128, 20, 0, 16), ("bfloat16", 40, 2, 37, 16)])
def test_latent_rows_cached_and_attended_at_every_edge(dtype, rank, heads, window, page):
    """The latent's norm and cache write, then attention over the cached rows with queries already in the latent
    space: every query is a multiple of one cached row, so nearly all its weight lies on one key, and the keys are
    chosen far back, at page borders, and just inside and just outside the window; prompt portions and single
    tokens, cut at awkward places, with a page pool that makes the second request reuse the first one's pages."""
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.runner import StepEntry
    from vllm_cpp_b200.parts.latent_attention import LatentAttention
    rng = np.random.default_rng(4)
    eps = 1e-5
    att = LatentAttention(hidden_size=32, num_heads=heads, head_dim=8, v_head_dim=8, kv_rank=rank, scale=1.0, window=window,
                          cache_window=window, owns_latent=True, eps=eps, output_gate=True, dtype=DT[dtype], device="cuda")
    n = 300
    cache, runner = attention_harness(att, page, pages=-(-n // page) + 1, max_len=n + page)
    gain = (1 + 0.2 * rng.standard_normal(rank)).astype(np.float32)
    for rid in ("first", "second"):
        raw = stored(rng.standard_normal((n, rank + 4)), dtype)
        c = stored(plain.rms(raw[:, 4:], eps) * gain, dtype)                       # what the cache holds
        # query t of head h aims at key t - back: far back, the window's two sides, page borders, itself
        backs = np.array([0, 1, window - 1, window, window + 1, page, page - 1, 250, 3, window - 2])
        q = np.zeros((n, heads, rank))
        for t in range(n):
            for h in range(heads):
                j = max(0, t - max(0, int(backs[(t + h) % len(backs)])))
                q[t, h] = c[j] * (12.0 / rank)
        q = stored(q, dtype)
        kv = np.repeat(c[:, None, :], heads, axis=1)
        want = plain.windowed_softmax_attention(q, kv, kv, 1.0, window).reshape(n, heads * rank)
        cache.add_request(rid)
        got, at = [], 0
        cuts = [129, 2, 3, 1, 1, 60, 1, 1, 1, 37, 1, 2, 1] + [1] * 60
        for size in cuts:
            size = min(size, n - at)
            if size == 0:
                break
            step = runner._prepare([StepEntry(rid, [0] * size, [])])
            view = runner.views[0]
            bt = step.block_tables[view.group]
            ops.latent_cache_write(dev(raw[at: at + size], DT[dtype])[:, 4:], dev(gain), step.positions, step.req_of_token, bt,
                                   view.pages.view(view.pages.shape[0], -1), page_size=page, eps=eps)
            out = torch.empty((size, heads * rank), dtype=DT[dtype], device="cuda")
            att.attend(dev(q[at: at + size].reshape(size, -1), DT[dtype]), out, step, view, bt)
            got.append(out.float().cpu().numpy())
            cache.commit(rid, size)
            at += size
        got = np.concatenate(got)
        err = np.abs(got - want[:at]).max(axis=1)
        tol = (2e-5 if dtype == "float32" else 3e-2) * np.abs(want).max()
        assert err.max() <= tol, f"{rid}: first wrong token {int(np.argmax(err > tol))}, error {err.max():.3e}"
        if rid == "first":
            # the rows of one slot lie where the layout says
            blk = view.pages[cache.table(rid, 0)[-1]].float().cpu().numpy().ravel()
            slot = (at - 1) % page
            held = blk[kv_pos(rank, 4 if dtype == "float32" else 2, slot, page)]
            assert np.abs(held - c[at - 1]).max() <= (1e-6 if dtype == "float32" else 2e-2) * np.abs(c[at - 1]).max()
        cache.free_request(rid)
    ops.check_status()


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompts_and_every_layer(tmp_path, name, dtype):
    cfg, weights, _, cache, runner = build(tmp_path, name, dtype, num_pages=24)
    rp = Replayer(runner, cache)
    for i, n in enumerate([1, 2, 19, 64, 150]):
        ids = ids_of(cfg, n, 100 + i)
        rp.step([(f"r{i}", ids, range(n))], end=[f"r{i}"])
        compare(rp.logits_of(f"r{i}", range(n)), plain.forward(cfg, weights, ids), dtype, f"{name} whole n={n}")
    assert cache.num_free_pages() == 24


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_prefill_against_token_by_token(tmp_path, name, dtype):
    """The same prompt at once, one token a step from the start, and most of it at once with a long tail of
    single tokens that passes every window."""
    cfg, weights, _, cache, runner = build(tmp_path, name, dtype, num_pages=24)
    rp = Replayer(runner, cache)
    ids = ids_of(cfg, 180, 7)
    want = plain.forward(cfg, weights, ids)
    for t in range(60):
        rp.step([("one", ids[t: t + 1], [0])])
    compare(rp.logits_of("one", range(60)), want[:60], dtype, f"{name} token by token")
    rp.step([("tail", ids[:75], [74])])
    for t in range(75, 180):
        rp.step([("tail", ids[t: t + 1], [0])])
    compare(rp.logits_of("tail", range(74, 180)), want[74:], dtype, f"{name} long decoding")
    rp.step([("x", [1, 2], [])], end=["one", "tail", "x"])
    assert cache.num_free_pages() == 24


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_down_to_two_tokens(tmp_path, name, dtype):
    cfg, weights, _, cache, runner = build(tmp_path, name, dtype, num_pages=24)
    rp = Replayer(runner, cache)
    sizes = [7, 2, 13, 3, 2, 31, 16, 2, 5, 33, 2, 64, 17, 1, 1, 2]
    for i, n in enumerate([70, 201]):
        ids = ids_of(cfg, n, 300 + i)
        at, k = 0, i
        while at < n:
            s = min(sizes[k % len(sizes)], n - at)
            rp.step([("p", ids[at: at + s], range(s))])
            at, k = at + s, k + 1
        compare(rp.logits_of("p", range(n)), plain.forward(cfg, weights, ids), dtype, f"{name} portions n={n}")
        rp.step([("x", [3], [])], end=["p", "x"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_requests_together_on_few_pages(tmp_path, name, dtype):
    """Up to four live requests, portions of some beside single tokens of others; requests end and new ones take
    their pages and state slots, so a slot's stale row and a page's stale latents would show."""
    cfg, weights, _, cache, runner = build(tmp_path, name, dtype, num_pages=28, max_seqs=4)
    page = CONFIGS[name][1]
    rp = Replayer(runner, cache)
    lengths = {"a": 90, "b": 33, "c": 140, "d": 2, "e": 75, "f": 51, "g": 120}
    ids = {r: ids_of(cfg, n, 400 + i) for i, (r, n) in enumerate(lengths.items())}
    want = {r: plain.forward(cfg, weights, ids[r]) for r in ids}
    rng = np.random.default_rng(9)
    waiting, live, at = list(lengths), [], {}
    while waiting or live:
        while waiting and len(live) < 4:
            r = waiting.pop(0)
            live.append(r)
            at[r] = 0
        entries, end = [], []
        for r in live:
            left = lengths[r] - at[r]
            s = 1 if (at[r] > 40 or rng.random() < 0.2) else int(min(left, rng.choice([2, 3, 17, page, 29, 64])))
            if rng.random() < 0.15 and len(live) > 1 and entries:
                continue                              # a request may sit a step out
            entries.append((r, ids[r][at[r]: at[r] + s], range(s)))
            at[r] += s
            if at[r] == lengths[r]:
                end.append(r)
        if entries:
            rp.step(entries, end=end)
        for r in end:
            compare(rp.logits_of(r, range(lengths[r])), want[r], dtype, f"{name} mixed {r}")
            live.remove(r)
    assert cache.num_free_pages() == 28


@pytest.mark.parametrize("dtype,pages", [("float32", 24), ("bfloat16", 24), ("float32", 10)])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype, pages):
    """LLM.generate: the scheduler cuts the prompts under a small token budget, decode steps are captured and
    replayed; every generated token is the plain implementation's best, or within rounding of it.  With 10 pages
    requests are preempted and fed again from their first token (their state slot starts from zero again)."""
    from vllm_cpp_b200 import LLM, SamplingParams
    cfg, page = CONFIGS["A"]
    weights = plain.random_weights(cfg, 5, sharp=SHARP[dtype])
    if dtype == "bfloat16":
        weights = plain.round_to_bf16(weights)
    folder = str(tmp_path / f"gen_{dtype}")
    plain.write_model_folder(folder, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    llm = LLM(folder, dtype=dtype, block_size=page, num_gpu_blocks=pages, max_num_seqs=3, max_model_len=pages * page,
              max_num_batched_tokens=48)
    prompts = [ids_of(cfg, n, 500 + n) for n in (3, 41, 100, 17)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True))
    if pages < 24:
        assert llm.engine.scheduler.num_preemptions > 0
    for p, o in zip(prompts, outs):
        assert len(o) == 40
        seq = list(p)
        for tok in o:
            logits = plain.forward(cfg, weights, seq)[-1]
            best = plain.greedy(logits)
            gap = (logits[best] - logits[tok]) / np.abs(logits).max()
            assert tok == best or gap < (1e-3 if dtype == "float32" else 5e-2), (dtype, len(p), tok, best, gap)
            seq.append(tok)


def random_rolesun_config(rng):
    """Sizes with odd factors everywhere: widths that are no multiple of 8 or 4, ranks of any width, up to 9 heads,
    value sizes unlike the key sizes, layers with and without feed-forward, layers that read earlier layers' latents
    through windows of their own."""
    width = int(rng.choice([36, 50, 64, 90, 104, 136]))
    layers, owners = [], []
    for i in range(int(rng.integers(1, 6))):
        share = owners and rng.random() < 0.4
        src = int(rng.choice(owners)) if share else None
        rank = layers[src][0]["kv_rank"] if share else int(rng.choice([18, 36, 64, 96, 128, 200]))
        m = mixer(int(rng.integers(1, 10)), int(rng.choice([4, 6, 8, 16, 20])), int(rng.choice([3, 8, 12, 16])), rank,
                  int(rng.integers(1, 90)), scale=float(rng.uniform(0.1, 0.4)), kv_from=src)
        if rng.random() < 0.15:
            m["mask"] = None
        if not share:
            owners.append(i)
        layers.append((m, None if rng.random() < 0.25 else int(rng.integers(20, 160))))
    return config(layers, width=width, vocab=int(rng.integers(40, 500)), mult=float(rng.uniform(0.3, 1.2)),
                  logit_scale=float(rng.uniform(0.1, 2.0)), emb=float(rng.uniform(0.5, 8.0)), eps=float(rng.choice([1e-5, 1e-6, 1e-4])))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [11, 12, 13, 14])
def test_the_replay_program_on_configurations_drawn_at_random(tmp_path, seed, dtype):
    """bin/trace_run as a user calls it, on a configuration drawn at random, under a schedule drawn at random: JSON
    lines in, <step>.f32 files and 'done' lines out; a pool of as many tokens as live requests hold, four slots."""
    import json
    import os
    import subprocess
    import sys
    rng = np.random.default_rng(seed)
    cfg = random_rolesun_config(rng)
    weights = plain.random_weights(cfg, seed, sharp=SHARP[dtype])
    if dtype == "bfloat16":
        weights = plain.round_to_bf16(weights)
    folder = str(tmp_path / "model")
    plain.write_model_folder(folder, cfg, weights, store="BF16" if dtype == "bfloat16" else "F32")
    lengths = {f"q{i}": int(n) for i, n in enumerate(rng.choice([1, 2, 30, 77, 150, 64], size=6))}
    ids = {r: ids_of(cfg, n, seed * 100 + i) for i, (r, n) in enumerate(lengths.items())}
    waiting, live, at, lines, asked = list(lengths), [], {}, [], []
    most = 0
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
            at[live[-1]] = 0
        most = max(most, sum(-(-lengths[r] // 64) * 64 for r in live))
        entries, end = [], []
        for r in live:
            s = int(min(lengths[r] - at[r], 1 if at[r] > 50 else rng.choice([1, 2, 3, 16, 37, 64])))
            want = sorted(set(int(w) for w in rng.integers(0, s, size=min(s, 3))))
            entries.append({"id": r, "tokens": ids[r][at[r]: at[r] + s], "want": want})
            asked.append([(r, at[r] + w) for w in want])
            at[r] += s
            if at[r] == lengths[r]:
                end.append(r)
        lines.append({"step": len(lines), "entries": entries, "end": end})
        asked[-len(entries):] = [sum(asked[-len(entries):], [])]
        live = [r for r in live if r not in end]
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(most)],
                       input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(lines))]
    want = {r: plain.forward(cfg, weights, ids[r]) for r in ids}
    for i, rows in enumerate(asked):
        if rows:
            got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
            compare(got, np.stack([want[r][t] for r, t in rows]), dtype, f"seed {seed} step {i}: {cfg['layers']}")


def test_command_line_and_sampling_options(tmp_path):
    """python -m vllm_cpp_b200.engine.cli on a Rolesun folder, the architecture taken from config.json or named by
    --arch: greedy ids are the plain implementation's; seeded sampling with temperature, top-k, top-p and a repetition
    penalty gives ids of the vocabulary and the same ids when asked again."""
    import os
    import subprocess
    import sys
    cfg, page = CONFIGS["A"]
    weights = plain.random_weights(cfg, 8, sharp=SHARP["float32"])
    folder = str(tmp_path / "cli_model")
    plain.write_model_folder(folder, cfg, weights, store="F32")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = ids_of(cfg, 21, 3)
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
    options = ["--arch", "rolesun", "--max-tokens", "12", "--temperature", "0.9", "--top-k", "20", "--top-p", "0.9",
               "--repetition-penalty", "1.2", "--sample-seed", "5"]
    drawn = run(options)
    assert len(drawn) == 12 and all(0 <= t < cfg["vocab"] for t in drawn)
    assert run(options) == drawn

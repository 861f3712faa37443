"""The Rolesun architecture without a GPU: configuration, description as parts, tensor names, cache layers
and the cache manager's bookkeeping for latents and token-shift rows."""
import numpy as np
import pytest
import torch

import plain_rolesun as plain
from vllm_cpp_b200 import ConfigError, resolve_architecture
from vllm_cpp_b200.cache.manager import CacheManager
from vllm_cpp_b200.parts.base import PagedKVSpec, StateSpec
from vllm_cpp_b200.parts.model import build_model


def mixer(heads, dim, vdim, rank, window, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale or dim ** -0.5, "mask": {"size": window}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def config(layers, width=64, vocab=200, mult=0.6, logit_scale=0.5, emb=3.0, eps=1e-5):
    return {"architecture": "Rolesun", "vocab": vocab, "width": width, "residual_mult": mult, "logit_scale": logit_scale,
            "embedding": {"scale": emb}, "norm": {"eps": eps},
            "layers": [{"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
                       for m, ff in layers]}


CFG = config([(mixer(3, 16, 24, 64, 20), 96), (mixer(2, 8, 8, 64, 33, kv_from=0), None), (mixer(4, 16, 16, 128, 70), 80),
              (mixer(1, 8, 12, 64, 12, kv_from=0), 48)])


def test_registry_takes_the_name_from_architecture():
    typed, spec = resolve_architecture(CFG)
    assert spec.architecture == "Rolesun" and spec.model_class == "scaled_sinusoid_decoder"
    assert typed.layers[1].mixer.kv_from == 0 and typed.layers[1].ff is None
    _, again = resolve_architecture(dict(CFG, architecture="other"), "rolesun")
    assert len(again.layers) == 4


def test_tensor_names_and_shapes_are_the_checkpoints():
    _, spec = resolve_architecture(CFG)
    model = build_model(spec, torch.bfloat16, "meta")
    got = {k: tuple(v.shape) for k, v in model.param_specs().items()}
    assert got == {k: tuple(v) for k, v in plain.tensor_shapes(CFG).items()}
    assert "l1.mix.dkv" not in got and "l1.norm2" not in got and "l1.mlp.gate" not in got
    assert "l1.rg2" in spec.ignored_tensors


def test_cache_layers_windows_and_states():
    _, spec = resolve_architecture(CFG)
    model = build_model(spec, torch.float32, "meta")
    specs = model.cache_specs()
    # layer 0's latents are read by layers 1 and 3 too: kept for the widest of the three windows
    assert specs[0] == PagedKVSpec(1, 64, 33, planes=1) and specs[1] == PagedKVSpec(1, 128, 70, planes=1)
    assert specs[2:] == [StateSpec((64,), torch.float32)] * 4
    order = spec.run_order
    assert [(c.cache, c.writes_cache, c.state) for c in order] == [(0, True, 2), (0, False, 3), (1, True, 4), (0, False, 5)]
    assert model.blocks[1].mixer.window == 33 and model.blocks[3].mixer.window == 12 and model.blocks[3].mixer.cache_window == 33


def test_a_layer_that_sees_all_keys_keeps_all_latents():
    cfg = config([(mixer(2, 8, 8, 32, 16), 40), (dict(mixer(2, 8, 8, 32, 16, kv_from=0), mask=None), 40)])
    _, spec = resolve_architecture(cfg)
    model = build_model(spec, torch.float32, "meta")
    assert model.cache_specs()[0].window == 0 and model.blocks[0].mixer.window == 16 and model.blocks[1].mixer.window == 0


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "no latents of its own"),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=32), "differs from layer 0"),
    (lambda c: c["layers"][0].update(type="recurrent"), "not a mixer of this design"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "not a feed-forward"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["norm"].update(eps=0), "norm.'eps' must be positive"),
    (lambda c: c["layers"][2]["mixer"].pop("vdim"), "vdim"),
])
def test_bad_configurations_are_refused(change, message):
    import copy
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        resolve_architecture(cfg)


def test_pages_of_one_plane_and_state_slots_that_are_used_again():
    _, spec = resolve_architecture(CFG)
    model = build_model(spec, torch.float32, "meta")
    specs = model.cache_specs()
    assert CacheManager.bytes_per_page(specs, 16, torch.bfloat16) == (64 + 128) * 16 * 2
    cm = CacheManager(specs, page_size=16, num_pages=6, max_num_seqs=2)
    assert len(cm.paged) == 2 and len(cm.state) == 1 and cm.state[0].layers == [2, 3, 4, 5]
    cm.add_request("a")
    cm.reserve("a", 70)
    cm.commit("a", 70)
    # the window of 33 has passed positions 0..37: two pages of group 0 are back; group 1 (window 70) keeps all five
    assert cm.paged[0].pool.num_free == 3 and cm.paged[1].pool.num_free == 1
    slot = cm.slot("a")
    cm.add_request("b")
    with pytest.raises(Exception):
        cm.add_request("c")
    cm.free_request("a")
    cm.add_request("c")
    assert cm.slot("c") == slot and cm.paged[0].pool.num_free == 6


def test_oracle_shift_and_window():
    x = np.arange(12, dtype=np.float64).reshape(4, 3)
    s = plain.token_shift(x, np.array([0.0, 1.0, 0.5]))
    assert np.allclose(s[0], [0, 0, 1]) and np.allclose(s[2], [6, 4, 6.5])
    q = np.zeros((5, 1, 2)); q[:, 0, 0] = 50.0
    k = np.zeros((5, 1, 2)); k[1, 0, 0] = 1.0
    v = np.arange(5, dtype=np.float64).reshape(5, 1, 1)
    out = plain.windowed_softmax_attention(q, k, v, 1.0, window=3)[:, 0, 0]
    assert abs(out[3] - 1.0) < 1e-9 and abs(out[4] - 3.0) < 1e-9        # key 1 is inside the window of 3, outside that of 4

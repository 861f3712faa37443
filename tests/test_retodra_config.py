"""The Retodra design without a GPU: its configuration reader, its description as parts, the tensors it declares,
the cache manager's handling of a mixer with two caches, sizes that only the checkpoint gives, and the expanded
bias table against the plain implementation's bucket rule."""
import numpy as np
import pytest
import torch

import plain_retodra as plain


def gla(heads, dim, vdim, tau=8.0, rank=8, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}, "mlp": mlp}


def par(lh, lg, ld, lv, window, rh, rd, rv, decay, scale=0.2, cap=12.0, reach=40, rows=12, ls=1.3, rs=0.8, mlp=None):
    left = {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": lv, "scale": scale, "bias_max": reach, "rel_rows": rows}
    if cap:
        left["softcap"] = cap
    if window:
        left["mask"] = {"size": window}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": rh, "dim": rd, "vdim": rv, "decay": list(decay)},
                                          "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, identity, top, limit=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}


def config(layers, width=64, vocab=200, emb=3.0, eps=1e-5):
    return {"architecture": "Retodra", "vocab": vocab, "width": width, "embedding": {"scale": emb}, "norm": {"eps": eps}, "layers": layers}


SAMPLE = config([gla(3, 16, 24, mlp=dense(96)),
                 par(4, 2, 32, 16, 20, 2, 16, 32, (0.9, 0.99), mlp=moe(40, 5, 2, 3)),
                 par(2, 2, 8, 8, 0, 1, 8, 8, (1.0,), cap=0.0, mlp=None)])


def test_config_is_read_and_described_as_parts():
    from vllm_cpp_b200.config.registry import resolve_architecture
    typed, spec = resolve_architecture(SAMPLE)
    assert typed.width == 64 and typed.eps == 1e-5 and typed.embedding_scale == 3.0
    assert [l.kind for l in typed.layers] == ["gla", "parallel", "parallel"]
    assert typed.layers[2].mixer["left"]["window"] == 0 and typed.layers[2].mixer["left"]["softcap"] == 0.0
    assert typed.layers[1].mlp == {"kind": "moe", "ff": 40, "limit": 1.5, "experts": 5, "top": 3, "identity": 2}
    assert spec.model_class == "scaled_embedding_decoder" and spec.model_params == {"embedding_scale": 3.0}
    assert [l.block for l in spec.layers] == ["sandwich_norm"] * 3
    assert spec.layers[0].mixer.kind == "gated_linear_attention" and spec.layers[1].mixer.kind == "parallel"
    assert spec.layers[1].mixer.params["left"].kind == "biased_window_attention"
    assert spec.layers[1].mixer.params["right"].params["decay"] == [0.9, 0.99]
    assert spec.layers[2].feed_forward.kind == "none" and spec.layers[1].feed_forward.kind == "routed_experts"
    assert resolve_architecture(SAMPLE, "retodra")[1].architecture == "Retodra"


def test_every_fault_of_a_config_is_named():
    from vllm_cpp_b200.config.engine_config import ConfigError
    from vllm_cpp_b200.config.registry import resolve_architecture
    bad = config([{"type": "conv", "mixer": {}}, gla(3, 16, 0), par(3, 2, 8, 8, 5, 2, 8, 8, (0.5,)),
                  dict(gla(1, 8, 8), mlp={"kind": "sparse"}), dict(gla(1, 8, 8), mlp=moe(8, 2, 0, 3))])
    del bad["width"]
    with pytest.raises(ConfigError) as e:
        resolve_architecture(bad)
    msg = str(e.value)
    for piece in ("missing 'width'", "'conv' is not a mixer", "'vdim' must be positive", "no multiple of kv_heads",
                  "'decay' must list one number", "'sparse' is not a feed-forward", "top 3 exceeds"):
        assert piece in msg, (piece, msg)


def test_declared_tensors_are_the_design_s():
    from vllm_cpp_b200.config.registry import resolve_architecture
    from vllm_cpp_b200.parts.model import build_model
    _, spec = resolve_architecture(SAMPLE)
    model = build_model(spec, torch.bfloat16, "meta")
    declared = model.param_specs()
    want = plain.tensor_shapes(SAMPLE)
    assert set(declared) == set(want)
    for name, shape in want.items():
        assert declared[name].fits(shape), (name, declared[name].shape, shape)
    # the two sizes no key gives are free, and any size of them fits
    assert declared["l1.mix.left.rel"].shape == (-1, 4) and declared["l1.mix.left.rel"].fits((77, 4))
    assert declared["l0.mix.a1"].shape == (-1, 64) and not declared["l0.mix.a1"].fits((5, 63))
    assert declared["l0.norm1"].role == "offset_gain" and declared["l0.mlp.gate"].role == "matrix"
    assert declared["l1.mlp.router"].role == "bias"            # held in float32


def test_a_mixer_with_two_caches_gets_both():
    from vllm_cpp_b200.cache.manager import CacheManager
    from vllm_cpp_b200.config.registry import resolve_architecture
    from vllm_cpp_b200.parts.base import CompositeSpec, CompositeView, PagedKVSpec, PagedKVView, StateSpec, StateView
    from vllm_cpp_b200.parts.model import build_model
    _, spec = resolve_architecture(SAMPLE)
    specs = build_model(spec, torch.float32, "meta").cache_specs()
    assert specs[0] == StateSpec((3, 16, 24), torch.float32)
    assert specs[1] == CompositeSpec((PagedKVSpec(2, 32, 20), StateSpec((2, 16, 32), torch.float32)))
    assert specs[2] == CompositeSpec((PagedKVSpec(2, 8, 0), StateSpec((1, 8, 8), torch.float32)))
    cm = CacheManager(specs, 16, 12, 3, torch.float32, None)
    assert len(cm.paged) == 2 and len(cm.state) == 3
    views = cm.views()
    assert isinstance(views[0], StateView) and isinstance(views[1], CompositeView)
    assert isinstance(views[1].views[0], PagedKVView) and isinstance(views[1].views[1], StateView)
    assert views[1].views[0].group != views[2].views[0].group
    assert CacheManager.bytes_per_page(specs, 16, torch.float32) == 2 * 2 * 16 * 32 * 4 + 2 * 2 * 16 * 8 * 4
    # the windowed group gives pages back, the other keeps them
    cm.add_request("a")
    cm.reserve("a", 70)
    cm.commit("a", 70)
    assert cm.table("a", views[1].views[0].group)[:3] == [-1, -1, -1] and -1 not in cm.table("a", views[2].views[0].group)
    cm.free_request("a")
    assert cm.num_free_pages() == 12


@pytest.mark.parametrize("rows,reach,window", [(12, 40, 20), (32, 200, 90), (7, 9.5, 0), (16, 64, 200), (2, 3, 5)])
def test_bias_rows_by_distance(rows, reach, window):
    from vllm_cpp_b200.parts.biased_attention import distance_buckets
    count = 300
    got = distance_buckets(rows, reach, count)
    want = [plain.distance_bucket(n, rows, reach) for n in range(count)]
    assert got.tolist() == want
    assert all(b == rows - 1 for b in got[int(np.ceil(reach)):])      # constant from the reach on: the table ends there
    assert list(got[: rows // 2]) == list(range(rows // 2))


def test_random_weights_mode_fills_free_sizes(tmp_path):
    from vllm_cpp_b200.weights.random_init import write_random_model
    from vllm_cpp_b200.weights.safetensors_io import SafetensorsFile
    write_random_model(str(tmp_path), SAMPLE, seed=3, dtype="bfloat16")
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    assert tuple(f.shape("l1.mix.left.rel")) == (64, 4) and tuple(f.shape("l0.mix.a1")) == (32, 64)
    assert tuple(f.shape("l0.mix.a2")) == (48, 32)
    w = f.tensor("l0.norm1").float()
    assert abs(float(w.mean())) < 0.05                          # stored around zero

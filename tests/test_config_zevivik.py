"""Zevivik's configuration on the CPU: the keys of its ``config.json``, the registry's choice by the
``architecture`` key, the schedule of a looped range of layers, the tensors its parts ask for, and what the cache
keeps for blocks of positions and for latent layers."""
import json

import pytest
import torch

from nncpu_b200.cache import Cache, KVRequest
from nncpu_b200.config import ZevivikConfig, config_from_dict
from nncpu_b200.engine.model import parameter_list
from nncpu_b200.errors import BadFormat, InvalidArgument, UnsupportedModel
from nncpu_b200.kernels.ops import key_span
from nncpu_b200.weights import check_tensors, write_model_folder

CFG = {"architecture": "Zevivik", "vocab": 97, "width": 40, "norm": {"eps": 2e-6}, "embedding": {"scale": 5.0},
       "loop": {"start": 1, "stop": 3, "times": 3},
       "layers": [{"type": "attention", "mlp": {"kind": "dense", "ff": 72},
                   "mixer": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 12, "scale": 0.25, "mask": {"size": 33},
                             "rot": {"base": 1234.0, "dims": 6}}},
                  {"type": "latent_attention", "mixer": {"heads": 2, "dim": 12, "vdim": 20, "kv_rank": 28, "scale": 0.3},
                   "mlp": {"kind": "moe", "expert": {"ff": 16, "limit": 1.5}, "router": {"experts": 5, "top": 2},
                           "shared": {"ff": 24, "limit": 0.5}}},
                  {"type": "attention", "mlp": {"kind": "moe", "expert": {"ff": 8, "limit": 3.0}, "router": {"experts": 3, "top": 3}},
                   "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "scale": 0.5}},
                  {"type": "latent_attention", "mlp": None,
                   "mixer": {"heads": 1, "dim": 6, "vdim": 10, "kv_rank": 9, "scale": 0.4}}]}


def test_keys_round_trip_and_specs():
    cfg = config_from_dict(CFG)
    assert isinstance(cfg, ZevivikConfig)
    assert config_from_dict(cfg.to_dict()) == cfg and cfg.to_dict() == CFG
    spec = cfg.model_spec()
    a, l, b, z = spec.layers
    assert {x.kind for x in spec.layers} == {"parallel"} and z.feed_forward is None
    assert (a.mixer.n_heads, a.mixer.n_kv_heads, a.mixer.head_dim, a.mixer.v_head_dim) == (6, 3, 8, 12)
    assert (a.mixer.chunk, a.mixer.window, a.mixer.scale) == (33, 0, 0.25)
    assert (a.mixer.position.theta, a.mixer.position.rotary_dim) == (1234.0, 6)
    assert b.mixer.position is None and b.mixer.chunk == 0
    assert a.feed_forward.activation == "gelu_tanh" and a.feed_forward.intermediate_size == 72
    assert (l.mixer.n_heads, l.mixer.head_dim, l.mixer.v_head_dim, l.mixer.latent_dim, l.mixer.head_gate) == (2, 12, 20, 28, True)
    f = l.feed_forward
    assert (f.n_experts, f.top, f.intermediate_size, f.limit, f.activation) == (5, 2, 16, 1.5, "swish_clamp")
    assert (f.shared.intermediate_size, f.shared.limit, f.shared.name) == (24, 0.5, "l1.mlp.shared")
    assert b.feed_forward.shared is None and spec.embedding.scale == 5.0


def test_the_looped_layers_run_in_order_with_what_each_pass_receives():
    spec = config_from_dict(CFG).model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    marks = [(i, e.inject.embedding, e.inject.table, e.inject.row) for i, e in enumerate(spec.schedule) if e.inject]
    assert marks == [(1, False, "loop.step", 0), (3, True, "loop.step", 1), (5, True, "loop.step", 2)]
    d = json.loads(json.dumps(CFG))
    del d["loop"]
    spec = config_from_dict(d).model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3] and all(e.inject is None for e in spec.schedule)
    assert "loop.step" not in {p.name for p in parameter_list(spec)}


def test_tensor_names_and_shapes():
    params = parameter_list(config_from_dict(CFG).model_spec())
    names = {p.name: p.shape for p in params}
    for n in ("embed", "head", "final.norm", "loop.step", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.o",
              "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down", "l1.mix.q", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv",
              "l1.mix.g", "l1.mix.o", "l1.mlp.router", "l1.mlp.router.b", "l1.mlp.e0.gate", "l1.mlp.e4.down",
              "l1.mlp.shared.gate", "l1.mlp.shared.down", "l2.mlp.e2.up", "l3.norm1"):
        assert n in names, n
    assert "l2.mlp.shared.up" not in names and "l1.mlp.e5.gate" not in names and "l0.mix.q.b" not in names
    assert names["loop.step"] == (3, 40) and names["l1.mix.uk"] == (24, 28) and names["l1.mix.uv"] == (40, 28)
    assert names["l1.mix.g"] == (2, 40) and names["l0.mix.o"] == (40, 72) and names["l1.mlp.e0.down"] == (40, 16)
    # a layer without a feed-forward: a second norm that its file may still hold is taken, and not needed
    spare = [p for p in params if p.name == "l3.norm2"]
    assert len(spare) == 1 and not spare[0].required
    shapes = {n: s for n, s in names.items() if n != "l3.norm2"}
    check_tensors(shapes, params, "file")
    shapes["l1.mix.dkv.norm"] = (29,)
    with pytest.raises(BadFormat, match="l1.mix.dkv.norm"):
        check_tensors(shapes, params, "file")


def test_random_weights_folder(tmp_path):
    folder = write_model_folder(tmp_path / "m", config_from_dict(CFG), 1, torch.float32)
    d = json.loads((folder / "config.json").read_text())
    assert d["layers"][1]["mlp"]["shared"] == {"ff": 24, "limit": 0.5} and d["loop"]["times"] == 3


@pytest.mark.parametrize("change,error", [
    (lambda d: d["layers"][0].update(type="conv"), UnsupportedModel),
    (lambda d: d["layers"][0]["mlp"].update(kind="sparse"), UnsupportedModel),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=4), BadFormat),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=5), BadFormat),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=10), BadFormat),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=6), BadFormat),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), BadFormat),
    (lambda d: d["loop"].update(stop=5), BadFormat),
    (lambda d: d["loop"].update(start=3), BadFormat),
    (lambda d: d.pop("norm"), BadFormat),
])
def test_refusals(change, error):
    d = json.loads(json.dumps(CFG))
    change(d)
    with pytest.raises(error):
        config_from_dict(d).model_spec()


def test_the_one_number_for_what_a_query_sees():
    assert key_span() == 0 and key_span(window=40) == 40 and key_span(chunk=40) == -40
    with pytest.raises(InvalidArgument):
        key_span(window=3, chunk=4)


def test_cache_gives_back_the_blocks_that_are_over_and_keeps_one_vector_for_latent_layers():
    """A group whose queries see their own block only frees the pages of earlier blocks; a keys-only group has no
    value pages of its own."""
    reqs = [(KVRequest(2, 16, chunk=100), None), (KVRequest(1, 40, keys_only=True), None)]
    cache = Cache(reqs, [None, None], 64 * 12, torch.float32, "cpu")
    blocky, latent = cache.groups[0], cache.groups[1]
    assert latent.v is latent.k and latent.bytes() == latent.k.numel() * 4
    s = cache.alloc_slot()
    cache.prepare([s], [250])
    cache.commit([s], [250])          # position 250 is in block 200..299, which starts in page 3
    assert [p >= 0 for p in blocky.tables[s]] == [False, False, False, True]
    assert all(p >= 0 for p in latent.tables[s])
    assert blocky.pool.n_held == 1 and latent.pool.n_held == 4
    cache.prepare([s], [60])
    cache.commit([s], [60])           # position 310: block 300..399 starts in page 4
    assert [p >= 0 for p in blocky.tables[s]] == [False, False, False, False, True]
    with pytest.raises(InvalidArgument):
        cache.truncate(s, 280)        # the block that position 280 is in has been given back
    cache.check()
    cache.free_slot(s)
    assert blocky.pool.n_held == 0 and latent.pool.n_held == 0

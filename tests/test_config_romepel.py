"""Romepel's configuration on the CPU: the keys of its ``config.json``, the registry's choice by the
``architecture`` key, the tensors its parts ask for, and a size that only the file's tensors give."""
import json

import pytest
import torch

from nncpu_b200.config import RomepelConfig, config_from_dict
from nncpu_b200.engine.model import parameter_list
from nncpu_b200.errors import BadFormat, UnsupportedModel
from nncpu_b200.weights import check_tensors, write_model_folder

CFG = {"architecture": "Romepel", "vocab": 97, "width": 48, "max_positions": 300, "norm": {"eps": 2e-6},
       "logit_softcap": 20.0,
       "layers": [{"type": "attention", "mlp": {"kind": "dense", "ff": 80},
                   "mixer": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 12, "scale": 0.25, "mask": {"size": 33},
                             "q_temp": {"coef": 0.5, "every": 16}}},
                  {"type": "gla", "mlp": None, "mixer": {"heads": 2, "dim": 12, "vdim": 20, "tau": 4.0}}]}


def test_keys_round_trip_and_specs():
    cfg = config_from_dict(CFG)
    assert isinstance(cfg, RomepelConfig)
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    a, g = spec.layers[0], spec.layers[1]
    assert a.kind == g.kind == "sandwich" and g.feed_forward is None and g.norm2 is None
    assert (a.mixer.n_heads, a.mixer.n_kv_heads, a.mixer.head_dim, a.mixer.v_head_dim) == (6, 3, 8, 12)
    assert (a.mixer.window, a.mixer.scale, a.mixer.q_temp_coef, a.mixer.q_temp_every) == (33, 0.25, 0.5, 16)
    assert a.mixer.slope_base == 8.0 and a.norm1.offset == 1.0 and a.norm1_post.name == "l0.norm1b"
    assert (g.mixer.n_heads, g.mixer.key_dim, g.mixer.value_dim, g.mixer.tau, g.mixer.gate_rank) == (2, 12, 20, 4.0, 0)
    assert spec.output.softcap == 20.0 and spec.embedding.positions == "pos" and spec.embedding.n_positions == 300


def test_tensor_names_and_the_rank_the_file_decides():
    names = {p.name: p.shape for p in parameter_list(config_from_dict(CFG).model_spec())}
    for n in ("embed", "pos", "head", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.q",
              "l0.mix.q.b", "l0.mix.k.b", "l0.mix.v", "l0.mix.o", "l0.mlp.up", "l0.mlp.up.b", "l0.mlp.down.b",
              "l0.mlp.act", "l1.norm1", "l1.norm1b", "l1.mix.g", "l1.mix.norm", "l1.mix.a1", "l1.mix.a2", "l1.mix.a2.b"):
        assert n in names, n
    assert "l1.norm2" not in names and "l1.mlp.up" not in names
    assert names["l0.mix.v"] == (3 * 12, 48) and names["l0.mix.o"] == (48, 6 * 12) and names["l1.mix.a1"] == (-1, 48)
    params = parameter_list(config_from_dict(CFG).model_spec())
    shapes = {n: tuple(5 if d == -1 else d for d in s) for n, s in names.items()}
    check_tensors(shapes, params, "file")                      # any rank fits
    shapes["l1.mix.a2.b"] = (7,)
    with pytest.raises(BadFormat, match="l1.mix.a2.b"):
        check_tensors(shapes, params, "file")


def test_random_weights_need_a_rank(tmp_path):
    with pytest.raises(Exception):
        write_model_folder(tmp_path / "a", config_from_dict(CFG), 1, torch.float32)
    d = json.loads(json.dumps(CFG))
    d["layers"][1]["mixer"]["rank"] = 4
    folder = write_model_folder(tmp_path / "b", config_from_dict(d), 1, torch.float32)
    assert json.loads((folder / "config.json").read_text())["layers"][1]["mixer"]["rank"] == 4


@pytest.mark.parametrize("change,error", [
    (lambda d: d["layers"][0].update(type="conv"), UnsupportedModel),
    (lambda d: d["layers"][0]["mlp"].update(kind="experts"), UnsupportedModel),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=4), BadFormat),
    (lambda d: d["layers"][1]["mixer"].pop("tau"), BadFormat),
    (lambda d: d.pop("width"), BadFormat),
    (lambda d: d.update(layers=[]), BadFormat),
    (lambda d: d.update(architecture="Nobody"), UnsupportedModel),
])
def test_refusals(change, error):
    d = json.loads(json.dumps(CFG))
    change(d)
    with pytest.raises(error):
        config_from_dict(d)


def test_options_a_file_may_leave_out():
    d = json.loads(json.dumps(CFG))
    d.pop("logit_softcap")
    d["layers"][0]["mixer"].pop("mask")
    d["layers"][0]["mixer"].pop("q_temp")
    spec = config_from_dict(d).model_spec()
    assert spec.output.softcap == 0.0 and spec.layers[0].mixer.window == 0 and spec.layers[0].mixer.q_temp_coef == 0.0

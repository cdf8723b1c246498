"""Romepel: a decoder whose ``config.json`` lists its layers one by one.

Every layer is a "sandwich" block (a norm before and after each sublayer, all with weights stored around
zero) around one of two mixers, gated linear attention (a recurrent state per head, no keys kept) or
windowed softmax attention with a distance bias per head and a query temperature that grows with the
position, and an optional dense feed-forward with the xIELU activation.  Positions enter through a learned
table added to the embedding rows; the logits are soft-capped.

``config.json``::

    {"architecture": "Romepel", "vocab": V, "width": W, "max_positions": P, "norm": {"eps": e},
     "logit_softcap": c,
     "layers": [{"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"}, "mlp": null},
                {"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "q_temp": {"coef", "every"}},
                 "mlp": {"kind": "dense", "ff": F}}, ...]}

Tensor names: ``embed``, ``pos``, ``final.norm``, ``head`` and per layer i ``l<i>.norm1`` / ``norm1b`` /
``norm2`` / ``norm2b``, ``l<i>.mix.*`` and ``l<i>.mlp.*``; biases end in ``.b``.  The rank of a gla layer's decay
projection is the one size the file's tensors give (``mix.a1`` is [rank, width]); a configuration that is to be
filled with random weights names it as ``mixer.rank``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from ..errors import BadFormat, UnsupportedModel
from .registry import register_architecture
from .specs import (AttentionSpec, BlockSpec, DenseMlpSpec, EmbeddingSpec, GatedLinearAttentionSpec, ModelSpec, NormSpec,
                    OutputSpec, ScheduleEntry)

SLOPE_BASE = 8.0     # the design's distance bias: head h of H has slope 2^(-8 (h + 1) / H)


def _int(d: dict, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int):
        raise BadFormat(f'config.json: {where} needs an integer "{key}", not {v!r}')
    if v < minimum:
        raise BadFormat(f'config.json: {where}: "{key}" is {v}, expected at least {minimum}')
    return v


def _num(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise BadFormat(f'config.json: {where} needs a positive number "{key}", not {v!r}')
    return float(v)


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise BadFormat(f'config.json: {where} needs an object "{key}", not {v!r}')
    return v


@dataclass(frozen=True)
class RomepelLayer:
    """One entry of ``layers``, checked.  ``window`` 0: every earlier key; ``q_temp_coef`` 0: no temperature;
    ``ff`` 0: no feed-forward; ``rank`` 0: taken from the file's tensors."""
    type: str
    heads: int
    dim: int
    vdim: int
    tau: float = 0.0
    rank: int = 0
    kv_heads: int = 0
    scale: float = 0.0
    window: int = 0
    q_temp_coef: float = 0.0
    q_temp_every: int = 1
    ff: int = 0

    @classmethod
    def from_dict(cls, i: int, d: dict) -> "RomepelLayer":
        where = f"layers[{i}]"
        if not isinstance(d, dict):
            raise BadFormat(f"config.json: {where} is not an object")
        kind = d.get("type")
        m = _obj(d, "mixer", where)
        mw = f"{where}.mixer"
        heads, dim, vdim = _int(m, "heads", mw), _int(m, "dim", mw), _int(m, "vdim", mw)
        ff = 0
        mlp = d.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise UnsupportedModel(f'config.json: {where}.mlp must be null or of "kind": "dense", not {mlp!r}')
            ff = _int(mlp, "ff", f"{where}.mlp")
        if kind == "gla":
            rank = 0 if m.get("rank") is None else _int(m, "rank", mw)
            return cls("gla", heads, dim, vdim, tau=_num(m, "tau", mw), rank=rank, ff=ff)
        if kind == "attention":
            kv = _int(m, "kv_heads", mw)
            if heads % kv:
                raise BadFormat(f"config.json: {mw}: {heads} heads are no multiple of {kv} key/value heads")
            window = 0 if m.get("mask") is None else _int(_obj(m, "mask", mw), "size", f"{mw}.mask")
            coef, every = 0.0, 1
            if m.get("q_temp") is not None:
                qt = _obj(m, "q_temp", mw)
                coef = qt.get("coef")
                if isinstance(coef, bool) or not isinstance(coef, (int, float)) or not math.isfinite(coef):
                    raise BadFormat(f'config.json: {mw}.q_temp needs a number "coef", not {coef!r}')
                every = _int(qt, "every", f"{mw}.q_temp")
            return cls("attention", heads, dim, vdim, kv_heads=kv, scale=_num(m, "scale", mw), window=window,
                       q_temp_coef=float(coef), q_temp_every=every, ff=ff)
        raise UnsupportedModel(f'config.json: {where} has "type": {kind!r} (supported: "gla", "attention")')

    def to_dict(self) -> dict:
        if self.type == "gla":
            m = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
            if self.rank:
                m["rank"] = self.rank
        else:
            m = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
            if self.window:
                m["mask"] = {"size": self.window}
            if self.q_temp_coef:
                m["q_temp"] = {"coef": self.q_temp_coef, "every": self.q_temp_every}
        return {"type": self.type, "mixer": m, "mlp": {"kind": "dense", "ff": self.ff} if self.ff else None}


@register_architecture("Romepel")
@dataclass
class RomepelConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: Tuple[RomepelLayer, ...]
    logit_softcap: float = 0.0
    eos_token_id: Tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: dict) -> "RomepelConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise BadFormat('config.json needs a non-empty list "layers"')
        cap = d.get("logit_softcap")
        eos = d.get("eos_token_id")
        eos = tuple(eos) if isinstance(eos, list) else (() if eos is None else (eos,))
        cfg = cls(vocab=_int(d, "vocab", "the model"), width=_int(d, "width", "the model"),
                  max_positions=_int(d, "max_positions", "the model"),
                  norm_eps=_num(_obj(d, "norm", "the model"), "eps", "norm"),
                  layers=tuple(RomepelLayer.from_dict(i, l) for i, l in enumerate(layers)),
                  logit_softcap=0.0 if cap is None else _num(d, "logit_softcap", "the model"), eos_token_id=eos)
        for e in cfg.eos_token_id:
            if isinstance(e, bool) or not isinstance(e, int) or not 0 <= e < cfg.vocab:
                raise BadFormat(f'config.json: "eos_token_id" holds {e!r}')
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
             "layers": [l.to_dict() for l in self.layers]}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    def model_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps

        def norm(name: str) -> NormSpec:
            return NormSpec("rmsnorm", w, eps, name, suffix="", offset=1.0)

        blocks: List[BlockSpec] = []
        for i, l in enumerate(self.layers):
            p = f"l{i}"
            if l.type == "gla":
                mixer = GatedLinearAttentionSpec(kind="gla", name=f"{p}.mix", hidden_size=w, n_heads=l.heads,
                                                 key_dim=l.dim, value_dim=l.vdim, gate_rank=l.rank, tau=l.tau, eps=eps)
            else:
                mixer = AttentionSpec(kind="attention", name=f"{p}.mix", hidden_size=w, n_heads=l.heads,
                                      n_kv_heads=l.kv_heads, head_dim=l.dim, v_head_dim=l.vdim, qkv_bias=True,
                                      scale=l.scale, window=l.window, slope_base=SLOPE_BASE,
                                      q_temp_coef=l.q_temp_coef, q_temp_every=l.q_temp_every, tensor_names="short")
            ff: Optional[DenseMlpSpec] = None
            if l.ff:
                ff = DenseMlpSpec(kind="dense_mlp", name=f"{p}.mlp", hidden_size=w, intermediate_size=l.ff,
                                  activation="xielu")
            blocks.append(BlockSpec(kind="sandwich", norm1=norm(f"{p}.norm1"), mixer=mixer,
                                    norm1_post=norm(f"{p}.norm1b"), norm2=norm(f"{p}.norm2") if ff else None,
                                    feed_forward=ff, norm2_post=norm(f"{p}.norm2b") if ff else None))
        return ModelSpec(
            architecture=self.architecture, hidden_size=w, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=EmbeddingSpec("embed", self.vocab, w, suffix="", positions="pos", n_positions=self.max_positions),
            layers=tuple(blocks), schedule=tuple(ScheduleEntry(i) for i in range(len(blocks))),
            output=OutputSpec(norm=norm("final.norm"), name="head", tied=False, vocab_size=self.vocab, hidden_size=w,
                              suffix="", softcap=self.logit_softcap),
            stop_token_ids=tuple(self.eos_token_id))

"""Zevivik: a decoder whose ``config.json`` lists its layers one by one and may run a range of them several times.

Every layer is a "parallel" block: both sublayers read the stream as it enters the layer,
x += mixer(norm1(x)) + feed_forward(norm2(x)).  The mixer is grouped-query softmax attention with a (possibly
partial) half-split rotation whose queries see the keys of their own block of positions, or latent attention (keys
and values of all heads are products of one normed vector per position, the only thing kept; causal; a sigmoid gate
per head).  The feed-forward is gated with the tanh form of GELU, or routed experts with a clamped gate and an
optional shared expert, or absent.  The embedding rows are scaled.  ``loop`` names a range of layers that runs
``times`` times in a row with the same weights and a cache per pass: before every pass but the first the embedding
output is added to the stream, then (before every pass) row t of the tensor ``loop.step``.

``config.json``::

    {"architecture": "Zevivik", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"base", "dims"}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "latent_attention", "mixer": {"heads", "dim", "vdim", "kv_rank", "scale"},
                 "mlp": {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"},
                         "shared": {"ff", "limit"}}}, ...]}

Tensor names: ``embed``, ``loop.step``, ``final.norm``, ``head`` and per layer i ``l<i>.norm1`` / ``norm2``,
``l<i>.mix.*`` and ``l<i>.mlp.*`` (experts ``.e<j>.gate / .up / .down``, ``.router``, ``.router.b``, ``.shared.*``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from ..errors import BadFormat, UnsupportedModel
from .registry import register_architecture
from .specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMlpSpec, LatentAttentionSpec, ModelSpec, NormSpec,
                    OutputSpec, PositionSpec, RoutedExpertsSpec, ScheduleEntry, StreamInjection)

LOOP_TABLE = "loop.step"


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
class ZevivikMlp:
    """A layer's feed-forward, checked.  ``kind`` "dense": ``ff``.  ``kind`` "moe": ``ff`` and ``limit`` of an expert,
    ``experts`` and ``top`` of the router, and the shared expert's ``shared_ff`` / ``shared_limit`` (0: none)."""
    kind: str
    ff: int
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    shared_ff: int = 0
    shared_limit: float = 0.0

    @classmethod
    def from_dict(cls, d, where: str) -> Optional["ZevivikMlp"]:
        if d is None:
            return None
        if not isinstance(d, dict):
            raise BadFormat(f"config.json: {where} is neither null nor an object")
        kind = d.get("kind")
        if kind == "dense":
            return cls("dense", _int(d, "ff", where))
        if kind == "moe":
            ex, ro = _obj(d, "expert", where), _obj(d, "router", where)
            experts, top = _int(ro, "experts", f"{where}.router"), _int(ro, "top", f"{where}.router")
            if top > experts:
                raise BadFormat(f"config.json: {where}.router takes the top {top} of {experts} experts")
            sh_ff, sh_limit = 0, 0.0
            if d.get("shared") is not None:
                sh = _obj(d, "shared", where)
                sh_ff, sh_limit = _int(sh, "ff", f"{where}.shared"), _num(sh, "limit", f"{where}.shared")
            return cls("moe", _int(ex, "ff", f"{where}.expert"), _num(ex, "limit", f"{where}.expert"), experts, top,
                       sh_ff, sh_limit)
        raise UnsupportedModel(f'config.json: {where} has "kind": {kind!r} (supported: "dense", "moe")')

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
             "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return d


@dataclass(frozen=True)
class ZevivikLayer:
    """One entry of ``layers``, checked.  ``chunk`` 0: every earlier key; ``rot_dims`` 0: no rotation."""
    type: str
    heads: int
    dim: int
    vdim: int
    scale: float
    kv_heads: int = 0
    chunk: int = 0
    rot_base: float = 0.0
    rot_dims: int = 0
    kv_rank: int = 0
    mlp: Optional[ZevivikMlp] = None

    @classmethod
    def from_dict(cls, i: int, d: dict) -> "ZevivikLayer":
        where = f"layers[{i}]"
        if not isinstance(d, dict):
            raise BadFormat(f"config.json: {where} is not an object")
        kind = d.get("type")
        m = _obj(d, "mixer", where)
        mw = f"{where}.mixer"
        heads, dim, vdim = _int(m, "heads", mw), _int(m, "dim", mw), _int(m, "vdim", mw)
        scale = _num(m, "scale", mw)
        mlp = ZevivikMlp.from_dict(d.get("mlp"), f"{where}.mlp")
        if kind == "attention":
            kv = _int(m, "kv_heads", mw)
            if heads % kv:
                raise BadFormat(f"config.json: {mw}: {heads} heads are no multiple of {kv} key/value heads")
            chunk = 0 if m.get("mask") is None else _int(_obj(m, "mask", mw), "size", f"{mw}.mask")
            base, dims = 0.0, 0
            if m.get("rot") is not None:
                rot = _obj(m, "rot", mw)
                base, dims = _num(rot, "base", f"{mw}.rot"), _int(rot, "dims", f"{mw}.rot", minimum=2)
                if dims % 2 or dims > dim:
                    raise BadFormat(f"config.json: {mw}.rot turns {dims} of a head's {dim} lanes: an even number of "
                                    "at most all of them is needed")
            return cls("attention", heads, dim, vdim, scale, kv_heads=kv, chunk=chunk, rot_base=base, rot_dims=dims,
                       mlp=mlp)
        if kind == "latent_attention":
            return cls("latent_attention", heads, dim, vdim, scale, kv_rank=_int(m, "kv_rank", mw), mlp=mlp)
        raise UnsupportedModel(f'config.json: {where} has "type": {kind!r} (supported: "attention", "latent_attention")')

    def to_dict(self) -> dict:
        if self.type == "attention":
            m = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
            if self.chunk:
                m["mask"] = {"size": self.chunk}
            if self.rot_dims:
                m["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        else:
            m = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "scale": self.scale}
        return {"type": self.type, "mixer": m, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@register_architecture("Zevivik")
@dataclass
class ZevivikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[ZevivikLayer, ...]
    embedding_scale: float = 1.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1          # 1 with start == stop == 0: no loop (and no ``loop.step`` tensor)
    has_loop: bool = False
    max_positions: int = 1 << 20  # the design has no table of positions: rotary angles are computed, nothing runs out
    eos_token_id: Tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: dict) -> "ZevivikConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise BadFormat('config.json needs a non-empty list "layers"')
        scale = 1.0
        if d.get("embedding") is not None:
            scale = _num(_obj(d, "embedding", "the model"), "scale", "embedding")
        start = stop = 0
        times, has_loop = 1, False
        if d.get("loop") is not None:
            lp = _obj(d, "loop", "the model")
            start, stop = _int(lp, "start", "loop", minimum=0), _int(lp, "stop", "loop", minimum=0)
            times, has_loop = _int(lp, "times", "loop"), True
            if not start < stop <= len(layers):
                raise BadFormat(f"config.json: loop runs layers {start} to {stop - 1} of {len(layers)}")
        eos = d.get("eos_token_id")
        eos = tuple(eos) if isinstance(eos, list) else (() if eos is None else (eos,))
        cfg = cls(vocab=_int(d, "vocab", "the model"), width=_int(d, "width", "the model"),
                  norm_eps=_num(_obj(d, "norm", "the model"), "eps", "norm"),
                  layers=tuple(ZevivikLayer.from_dict(i, l) for i, l in enumerate(layers)), embedding_scale=scale,
                  loop_start=start, loop_stop=stop, loop_times=times, has_loop=has_loop,
                  max_positions=_int(d, "max_positions", "the model") if d.get("max_positions") is not None else 1 << 20,
                  eos_token_id=eos)
        for e in cfg.eos_token_id:
            if isinstance(e, bool) or not isinstance(e, int) or not 0 <= e < cfg.vocab:
                raise BadFormat(f'config.json: "eos_token_id" holds {e!r}')
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
             "layers": [l.to_dict() for l in self.layers]}
        if self.has_loop:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    def schedule(self) -> Tuple[ScheduleEntry, ...]:
        """The layers in running order.  The first layer of pass t of the loop carries what the stream receives
        before that pass: the embedding output (t > 0) and row t of ``loop.step``."""
        n = len(self.layers)
        if not self.has_loop:
            return tuple(ScheduleEntry(i) for i in range(n))
        a, b, times = self.loop_start, self.loop_stop, self.loop_times
        runs: List[ScheduleEntry] = [ScheduleEntry(i) for i in range(a)]
        for t in range(times):
            for i in range(a, b):
                inject = StreamInjection(embedding=t > 0, table=LOOP_TABLE, n_rows=times, row=t) if i == a else None
                runs.append(ScheduleEntry(i, inject=inject))
        return tuple(runs + [ScheduleEntry(i) for i in range(b, n)])

    def model_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps

        def norm(name: str) -> NormSpec:
            return NormSpec("rmsnorm", w, eps, name, suffix="")

        def gated(name: str, ff: int, activation: str, limit: float = 0.0) -> GatedMlpSpec:
            return GatedMlpSpec(kind="gated_mlp", name=name, hidden_size=w, intermediate_size=ff, activation=activation,
                                limit=limit, tensor_names="short")

        blocks: List[BlockSpec] = []
        for i, l in enumerate(self.layers):
            p = f"l{i}"
            if l.type == "attention":
                position = PositionSpec("rope_neox", l.rot_base, l.rot_dims) if l.rot_dims else None
                mixer = AttentionSpec(kind="attention", name=f"{p}.mix", hidden_size=w, n_heads=l.heads,
                                      n_kv_heads=l.kv_heads, head_dim=l.dim, v_head_dim=l.vdim, scale=l.scale,
                                      chunk=l.chunk, position=position, tensor_names="short")
            else:
                mixer = LatentAttentionSpec(kind="latent_attention", name=f"{p}.mix", hidden_size=w, n_heads=l.heads,
                                            head_dim=l.dim, v_head_dim=l.vdim, latent_dim=l.kv_rank, scale=l.scale,
                                            eps=eps, head_gate=True)
            ff = None
            if l.mlp is not None and l.mlp.kind == "dense":
                ff = gated(f"{p}.mlp", l.mlp.ff, "gelu_tanh")
            elif l.mlp is not None:
                m = l.mlp
                shared = gated(f"{p}.mlp.shared", m.shared_ff, "swish_clamp", m.shared_limit) if m.shared_ff else None
                ff = RoutedExpertsSpec(kind="routed_experts", name=f"{p}.mlp", hidden_size=w, intermediate_size=m.ff,
                                       n_experts=m.experts, top=m.top, activation="swish_clamp", limit=m.limit,
                                       shared=shared)
            # a layer without a feed-forward has no use for its second norm; a file that holds one all the same is taken
            blocks.append(BlockSpec(kind="parallel", norm1=norm(f"{p}.norm1"), mixer=mixer, norm2=norm(f"{p}.norm2"),
                                    feed_forward=ff))
        return ModelSpec(
            architecture=self.architecture, hidden_size=w, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=EmbeddingSpec("embed", self.vocab, w, scale=self.embedding_scale, suffix=""),
            layers=tuple(blocks), schedule=self.schedule(),
            output=OutputSpec(norm=norm("final.norm"), name="head", tied=False, vocab_size=self.vocab, hidden_size=w,
                              suffix=""),
            stop_token_ids=tuple(self.eos_token_id))

"""A plain, slow statement of the Zevivik decoder: one function per mechanism, float64 NumPy on the CPU, one
masked matrix per head.  It shares no code with the library: it has its own file reader, reads ``config.json``
itself and knows nothing of pages, slots or steps.  The tests hold the library to it.

Notation: x is the residual stream [T, W], h a sublayer's input, p a position (from 0), H heads, G key/value
heads, d the query/key size of a head, e its value size, r the size of the latent.

The design in short.  x0 = embed[token] * s.  The layers are listed one by one; a range [a, b) of them may run n
times in a row with the same weights (every pass with keys of its own): before pass t the vector step[t] is added
to x, and before every pass but the first x0 is added first.  A layer is parallel: x <- x + mixer(n1(x)) + ff(n2(x)).
Mixers: grouped-query softmax attention with a partial half-split rotation, where position i sees the keys
j <= i of its own block of ``size`` positions; or latent attention, where keys and values of all heads are
products of one normed latent vector per position, the mask is causal and every head's output is scaled by a
sigmoid gate.  Feed-forwards: a gated one with the tanh form of GELU, or routed experts (the ``top`` largest router
logits, softmax over those) with a clamped gate g * sigmoid(1.702 g) * (u + 1), plus an optional shared expert.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np

GATE_SLOPE = 1.702      # the experts' gate: g * sigmoid(1.702 g)


# -- files ----------------------------------------------------------------------------

def read_safetensors(path) -> dict:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf, dt = data[lo:hi], info["dtype"]
        if dt == "BF16":
            a = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif dt == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif dt == "I32":
            a = np.frombuffer(buf, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: element type {dt}")
        out[name] = a.reshape(info["shape"])
    return out


def load(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# -- small functions --------------------------------------------------------------------

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def softmax_rows(s, visible):
    s = np.where(visible, s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    w = np.exp(s)
    return w / w.sum(axis=-1, keepdims=True)


# -- positions ----------------------------------------------------------------------------

def rotate(u, positions, base, dims):
    """u [T, heads, d]: the first ``dims`` lanes of every head turn, lane i with lane i + dims/2 by the angle
    p * base^(-2i/dims); the other lanes stay."""
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    a = np.asarray(positions, dtype=np.float64)[:, None, None] * f[None, None, :]
    c, s = np.cos(a), np.sin(a)
    out = u.copy()
    lo, hi = u[..., :half], u[..., half:dims]
    out[..., :half] = lo * c - hi * s
    out[..., half:dims] = hi * c + lo * s
    return out


def masked_attention(q, k, v, q_pos, scale, size=0):
    """q [n, H, d] at positions q_pos; k [L, G, d] and v [L, G, e] hold the keys and values of positions 0 .. L-1.
    Head a reads key/value head a // (H / G).  Position i sees j <= i of its own block (size 0: every j <= i)."""
    n, H, _ = q.shape
    L, G, e = v.shape
    i, j = np.asarray(list(q_pos))[:, None], np.arange(L)[None, :]
    vis = j <= i
    if size:
        vis &= (i // size) == (j // size)
    out = np.zeros((n, H, e))
    for a in range(H):
        g = a // (H // G)
        out[:, a] = softmax_rows((q[:, a] @ k[:, g].T) * scale, vis) @ v[:, g]
    return out


# -- mixers ---------------------------------------------------------------------------------

def attention(h, w, m, name):
    """Grouped-query attention inside blocks of positions.  h [T, W]; w the tensors; m the layer's ``mixer``."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[f"{name}.q"].T).reshape(T, H, d)
    k = (h @ w[f"{name}.k"].T).reshape(T, G, d)
    v = (h @ w[f"{name}.v"].T).reshape(T, G, e)
    rot = m.get("rot")
    if rot:
        pos = np.arange(T)
        q, k = rotate(q, pos, rot["base"], rot["dims"]), rotate(k, pos, rot["base"], rot["dims"])
    out = masked_attention(q, k, v, range(T), m["scale"], (m.get("mask") or {}).get("size", 0))
    return out.reshape(T, H * e) @ w[f"{name}.o"].T


def latent_attention(h, w, m, name, eps):
    """Keys and values of all heads from one normed latent per position; causal; gated heads."""
    T = h.shape[0]
    H, d, e, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[f"{name}.q"].T).reshape(T, H, d)
    c = rms_norm(h @ w[f"{name}.dkv"].T, w[f"{name}.dkv.norm"], eps)
    assert c.shape == (T, r)
    k = (c @ w[f"{name}.uk"].T).reshape(T, H, d)
    v = (c @ w[f"{name}.uv"].T).reshape(T, H, e)
    gate = sigmoid(h @ w[f"{name}.g"].T)            # [T, H]
    out = masked_attention(q, k, v, range(T), m["scale"]) * gate[:, :, None]
    return out.reshape(T, H * e) @ w[f"{name}.o"].T


# -- feed-forwards ------------------------------------------------------------------------------

def dense_ff(h, w, name):
    return (gelu_tanh(h @ w[f"{name}.gate"].T) * (h @ w[f"{name}.up"].T)) @ w[f"{name}.down"].T


def expert(h, w, name, limit):
    g = np.minimum(h @ w[f"{name}.gate"].T, limit)
    u = np.clip(h @ w[f"{name}.up"].T, -limit, limit)
    return (g * sigmoid(GATE_SLOPE * g) * (u + 1.0)) @ w[f"{name}.down"].T


def route(h, w, name, top):
    """Per token: the ``top`` experts with the largest logits and the softmax over those logits."""
    z = h @ w[f"{name}.router"].T + w[f"{name}.router.b"]
    order = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zs = np.take_along_axis(z, order, axis=-1)
    ws = np.exp(zs - zs.max(axis=-1, keepdims=True))
    return order, ws / ws.sum(axis=-1, keepdims=True)


def moe_ff(h, w, mlp, name):
    ids, ws = route(h, w, name, mlp["router"]["top"])
    out = np.zeros((h.shape[0], w[f"{name}.e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], ws[t]):
            out[t] += a * expert(h[t:t + 1], w, f"{name}.e{e}", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out += expert(h, w, f"{name}.shared", mlp["shared"]["limit"])
    return out


# -- the model -------------------------------------------------------------------------------------

def layer(x, w, cfg, i):
    L, eps = cfg["layers"][i], cfg["norm"]["eps"]
    h1 = rms_norm(x, w[f"l{i}.norm1"], eps)
    if L["type"] == "attention":
        y = attention(h1, w, L["mixer"], f"l{i}.mix")
    elif L["type"] == "latent_attention":
        y = latent_attention(h1, w, L["mixer"], f"l{i}.mix", eps)
    else:
        raise ValueError(L["type"])
    mlp = L.get("mlp")
    if mlp:
        h2 = rms_norm(x, w[f"l{i}.norm2"], eps)
        y = y + (dense_ff(h2, w, f"l{i}.mlp") if mlp["kind"] == "dense" else moe_ff(h2, w, mlp, f"l{i}.mlp"))
    return x + y


def layer_runs(cfg):
    """(layer, pass number or None) in running order; the pass number is set on the first layer of a pass."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def greedy(cfg, w, prompt, n):
    """n tokens chosen greedily (the first largest logit), the whole sequence recomputed for every token."""
    seq, out = list(prompt), []
    for _ in range(n):
        out.append(int(np.argmax(forward(cfg, w, seq)[-1])))
        seq.append(out[-1])
    return out


def forward(cfg, w, tokens, trace=None):
    """Logits [T, vocab] of one sequence.  ``trace``: a list that receives x after every layer run."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    x = x0.copy()
    for i, t in layer_runs(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        x = layer(x, w, cfg, i)
        if trace is not None:
            trace.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T

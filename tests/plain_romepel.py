"""A plain, slow statement of the Romepel decoder: one function per mechanism,
float64 NumPy on the CPU, token by token where the design has a recurrence and
one masked matrix per head where it has attention.  It shares no code with the
library: it has its own file reader, reads ``config.json`` itself and knows
nothing of pages, slots or steps.  The tests hold the library to it.

Notation: x is the residual stream, h a sublayer's input, p a position (from 0),
H heads, G key/value heads, d the query/key size of a head, e its value size.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# -- files ----------------------------------------------------------------------------

def read_safetensors(path) -> dict:
    """name -> float64 array (integer tables stay integers).  The file is an 8-byte
    little-endian header length, a JSON header, then raw data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = data[lo:hi]
        dt = info["dtype"]
        if dt == "BF16":
            a = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif dt == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif dt == "F16":
            a = np.frombuffer(buf, dtype="<f2").astype(np.float64)
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


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def silu(z):
    return z * sigmoid(z)


def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """The layers' norm: the weight is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (np.expm1(np.minimum(z, 0.0)) - z) + 0.5 * z
    return np.where(z > 0, pos, neg)


def head_slopes(H):
    """Distance-bias slope of head h: 2^(-8 (h + 1) / H)."""
    return np.array([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])


def query_temperature(p, coef, every):
    """1 + coef ln(floor((p + 1) / every) + 1) at position p."""
    return 1.0 + coef * np.log(np.floor((np.asarray(p) + 1) / every) + 1.0)


# -- mixers -------------------------------------------------------------------------------

def gla_recurrence(q, k, v, alpha, S):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, head by head and token by token.
    q, k, alpha [T, H, d]; v [T, H, e]; S [H, d, e] is updated in place.  Returns o [T, H, e]."""
    T, H = q.shape[:2]
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        for hd in range(H):
            S[hd] = alpha[t, hd][:, None] * S[hd] + np.outer(k[t, hd], v[t, hd])
            out[t, hd] = S[hd].T @ q[t, hd]
    return out


def gla_mixer(h, w, name, m, state=None):
    """Gated linear attention over the rows of h (one sequence, in order).  ``state`` [H, d, e] is what earlier
    rows left (None: zeros); returns (output rows, state after the last row)."""
    H, d, e, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    T = h.shape[0]
    q = (h @ w[f"{name}.q"].T) * d ** -0.5
    k = h @ w[f"{name}.k"].T
    v = h @ w[f"{name}.v"].T
    g = h @ w[f"{name}.g"].T
    z = (h @ w[f"{name}.a1"].T) @ w[f"{name}.a2"].T + w[f"{name}.a2.b"]
    alpha = sigmoid(z) ** (1.0 / tau)
    q, k, alpha = (a.reshape(T, H, d) for a in (q, k, alpha))
    v = v.reshape(T, H, e)
    S = np.zeros((H, d, e)) if state is None else np.array(state, dtype=np.float64)
    out = gla_recurrence(q, k, v, alpha, S)
    out = rms(out, m["_eps"]) * w[f"{name}.norm"]          # per head over e, one weight shared by the heads
    out = out.reshape(T, H * e) * silu(g)
    return out @ w[f"{name}.o"].T, S


def biased_attention(q, k, v, pos, scale, window, slopes):
    """Softmax attention of queries at positions ``pos`` over keys 0 .. N-1: query i sees key j when
    0 <= i - j (< window, if there is one); head h takes slopes[h] * (i - j) off the scaled score.
    q [T, H, d]; k [N, G, d]; v [N, G, e].  Returns [T, H, e]."""
    T, H = q.shape[:2]
    G = k.shape[1]
    dist = np.asarray(pos)[:, None] - np.arange(k.shape[0])[None, :]      # i - j
    seen = (dist >= 0) & ((dist < window) if window else True)
    out = np.zeros((T, H, v.shape[2]))
    for hd in range(H):
        kv = hd // (H // G)
        s = (q[:, hd] @ k[:, kv].T) * scale - slopes[hd] * dist
        s = np.where(seen, s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(axis=1, keepdims=True)
        out[:, hd] = p @ v[:, kv]
    return out


def attention_mixer(h, w, name, m, first_pos=0, past_k=None, past_v=None):
    """Windowed softmax attention with a distance bias and a query temperature.  ``past_k``/``past_v`` hold the
    keys and values of positions 0 .. first_pos - 1 (None: the rows of h start the sequence).  Returns
    (output rows, all keys, all values)."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = h @ w[f"{name}.q"].T + w[f"{name}.q.b"]
    k = h @ w[f"{name}.k"].T + w[f"{name}.k.b"]
    v = h @ w[f"{name}.v"].T + w[f"{name}.v.b"]
    pos = first_pos + np.arange(T)
    temp = query_temperature(pos, m["q_temp"]["coef"], m["q_temp"]["every"]) if m.get("q_temp") else np.ones(T)
    q = q.reshape(T, H, d) * temp[:, None, None]
    k = k.reshape(T, G, d)
    v = v.reshape(T, G, e)
    if past_k is not None:
        k = np.concatenate([past_k, k], axis=0)
        v = np.concatenate([past_v, v], axis=0)
    window = m["mask"]["size"] if m.get("mask") else None
    out = biased_attention(q, k, v, pos, m["scale"], window, head_slopes(H))
    return out.reshape(T, H * e) @ w[f"{name}.o"].T, k, v


def dense_mlp(h, w, name):
    up = h @ w[f"{name}.up"].T + w[f"{name}.up.b"]
    p, q = w[f"{name}.act"]
    return xielu(up, p, q) @ w[f"{name}.down"].T + w[f"{name}.down.b"]


# -- the model ----------------------------------------------------------------------------------

class Sequence:
    """One sequence's memory between calls of ``forward``: its length, the keys and values of every attention layer
    and the state of every recurrent layer."""

    def __init__(self):
        self.length = 0
        self.kv = {}
        self.state = {}


def forward(cfg, w, tokens, seq: Sequence = None, return_layers=False):
    """Logits [len(tokens), vocab] of ``tokens`` appended to ``seq`` (a fresh sequence when None)."""
    seq = seq if seq is not None else Sequence()
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    pos = seq.length + np.arange(T)
    x = w["embed"][np.asarray(tokens)] + w["pos"][pos]
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}"
        m = dict(layer["mixer"], _eps=eps)
        h = offset_norm(x, w[f"{L}.norm1"], eps)
        if layer["type"] == "gla":
            y, seq.state[i] = gla_mixer(h, w, f"{L}.mix", m, seq.state.get(i))
        elif layer["type"] == "attention":
            pk, pv = seq.kv.get(i, (None, None))
            y, k, v = attention_mixer(h, w, f"{L}.mix", m, seq.length, pk, pv)
            seq.kv[i] = (k, v)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + offset_norm(y, w[f"{L}.norm1b"], eps)
        if layer.get("mlp") is not None:
            h = offset_norm(x, w[f"{L}.norm2"], eps)
            x = x + offset_norm(dense_mlp(h, w, f"{L}.mlp"), w[f"{L}.norm2b"], eps)
        layers.append(x.copy())
    seq.length += T
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(layers)) if return_layers else logits

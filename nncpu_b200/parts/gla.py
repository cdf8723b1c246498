"""Gated linear attention: a recurrent mixer that keeps, per sequence and head, a state S of ``key_dim`` x
``value_dim`` 32-bit floats in the cache's state area instead of keys and values per position.

With h the mixer's input, per head (d = key_dim, e = value_dim):

    q = W_q h * d^(-1/2),  k = W_k h,  v = W_v h,  gate = W_g h
    z = W_a2 (W_a1 h) + b_a2                    (a low-rank projection: decay logits per key channel)
    a = sigmoid(z)^(1/tau)
    S <- diag(a) S + k v^T,   o = S^T q
    out = W_o concat_heads(o / rms(o) * w_norm * silu(gate))

The four projections of h are one product (their rows stacked); products run in the run's element type with
32-bit accumulators and their results stay in float32; the decay (its logarithm and exponential), the
recurrence and the norm are 32-bit in both run types.  The recurrence walks a sequence's tokens in order inside
one kernel, so a prompt cut into portions and a batch of unequal sequences give the same bits; a decode step
(one token per sequence) runs a kernel of its own that streams the state once and adds a column's terms in
another order, which differs by rounding in the last bits.
"""
from __future__ import annotations

import torch

from ..cache import StateRequest
from ..errors import BadFormat, UnsupportedModel
from ..kernels import ops
from ..weights.params import ParamSpec
from .base import Mixer, register_mixer

MAX_KEY_DIM = 512      # a lane of the scan kernel keeps one column of a head's state in registers


@register_mixer("gla")
class GatedLinearAttention(Mixer):
    def __init__(self, spec, reads_other_cache: bool = False):
        if reads_other_cache:
            raise UnsupportedModel(f"{spec.name}: a recurrent mixer keeps no keys and values that another layer could read")
        if spec.key_dim > MAX_KEY_DIM:
            raise UnsupportedModel(f"{spec.name}: {spec.key_dim} key channels a head (at most {MAX_KEY_DIM})")
        self.spec = spec
        self.qk_size = spec.n_heads * spec.key_dim
        self.v_size = spec.n_heads * spec.value_dim

    def state_request(self):
        s = self.spec
        return StateRequest((s.n_heads, s.key_dim, s.value_dim), torch.float32)

    def params(self):
        s = self.spec
        r = s.gate_rank if s.gate_rank > 0 else -1        # -1: whatever the file holds
        return [ParamSpec(f"{s.name}.q", (self.qk_size, s.hidden_size)),
                ParamSpec(f"{s.name}.k", (self.qk_size, s.hidden_size)),
                ParamSpec(f"{s.name}.v", (self.v_size, s.hidden_size)),
                ParamSpec(f"{s.name}.g", (self.v_size, s.hidden_size)),
                ParamSpec(f"{s.name}.o", (s.hidden_size, self.v_size)),
                ParamSpec(f"{s.name}.norm", (s.value_dim,), init=("one_plus_normal", 0.1)),
                ParamSpec(f"{s.name}.a1", (r, s.hidden_size)),
                ParamSpec(f"{s.name}.a2", (self.qk_size, r), init=("normal", 0.2)),
                ParamSpec(f"{s.name}.a2.b", (self.qk_size,), init=("normal", 1.0))]

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        ws = [tensors.pop(f"{s.name}.{n}") for n in ("q", "k", "v", "g")]
        self.w_qkvg = torch.cat(ws, dim=0).contiguous()
        del ws
        self.w_a1, self.w_a2, self.b_a2 = tensors[f"{s.name}.a1"], tensors[f"{s.name}.a2"], tensors[f"{s.name}.a2.b"]
        if self.w_a1.shape[0] != self.w_a2.shape[1]:
            raise BadFormat(f"{s.name}: a1 has {self.w_a1.shape[0]} rows and a2 {self.w_a2.shape[1]} columns")
        self.rank = self.w_a1.shape[0]
        self.w_o, self.w_norm = tensors[f"{s.name}.o"], tensors[f"{s.name}.norm"]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkvg, self.w_a1, self.w_a2, self.w_o))

    def forward(self, ctx, x, residual, cache):
        s, rt = self.spec, self.rt
        n = x.shape[0]
        proj = rt.empty(n, 2 * (self.qk_size + self.v_size), dtype=torch.float32)
        with rt.phase("gla_proj", self.w_qkvg, n):
            rt.linear(x, self.w_qkvg, None, proj)
        low = rt.empty(n, self.rank)
        z = rt.empty(n, self.qk_size, dtype=torch.float32)
        with rt.phase("gla_decay", self.w_a1, n):
            rt.linear(x, self.w_a1, None, low)
            rt.linear(low, self.w_a2, self.b_a2, z)
        gated = rt.empty(n, self.v_size)
        state_bytes = 8.0 * ctx.n_seqs * s.n_heads * s.key_dim * s.value_dim       # read and written once a step
        if ctx.is_decode and s.value_dim <= 1024:
            # one token per sequence: recurrence, norm and gate in one launch that streams the state once
            with rt.phase("gla_scan", nbytes=state_bytes + 4.0 * (proj.numel() + z.numel()) + gated.numel() * gated.element_size()):
                ops.gla_step(proj, z, cache.state, ctx.seq_slots, self.w_norm, s.eps, gated, s.n_heads, s.key_dim,
                             s.value_dim, s.key_dim ** -0.5, s.tau)
        else:
            o = rt.empty(n, self.v_size, dtype=torch.float32)
            with rt.phase("gla_decay"):
                ops.gla_decay(z, s.tau)         # once for all the blocks of the scan that read a token's decays
            with rt.phase("gla_scan", nbytes=state_bytes + 4.0 * (proj.numel() + z.numel() + o.numel()),
                          flops=4.0 * n * s.n_heads * s.key_dim * s.value_dim):
                ops.gla_scan(proj, z, cache.state, ctx.seq_slots, ctx.cu_seqlens, o, ctx.n_seqs, s.n_heads, s.key_dim,
                             s.value_dim, s.key_dim ** -0.5, s.tau, decays_given=True)
            with rt.phase("gla_gate"):
                ops.gla_output(o, proj, self.w_norm, s.eps, gated, s.n_heads, s.key_dim, s.value_dim)
        with rt.phase("gla_out", self.w_o, n):
            rt.linear(gated, self.w_o, None, residual, accumulate=not getattr(ctx, "branch_is_fresh", False))

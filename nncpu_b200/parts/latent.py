"""Latent attention: the keys and values of all heads are products of ONE vector per position, and that vector
is all the cache keeps.

With h the mixer's input, H heads of d query/key lanes and e value lanes, and a latent of r lanes:

    q = W_q h                                  [H, d]
    c = rmsnorm(W_dkv h) * w_norm              [r]          (kept per position)
    k_a = W_uk[a] c,  v_a = W_uv[a] c          per head a
    s_a(i, j) = (q_a(i) . k_a(j)) * scale,  j <= i;  softmax over j;  o_a = sum_j p_a(i, j) v_a(j)
    out = W_o concat_a(sigmoid(g_a) o_a),  g = W_g h         (the gate only with ``head_gate``)

The products with W_uk and W_uv are moved to the query side, so that no key or value of a head is ever made:
q'_a = W_uk[a]^T q_a (r lanes) gives q_a . k_a(j) = q'_a . c(j), and sum_j p(j) v_a(j) = W_uv[a] (sum_j p(j) c(j)).
What runs over the cache is therefore attention of H query heads on one key/value head of r lanes whose values
are its keys: the paged attention kernels of the ordinary attention part, on a cache group that has key pages only.
The projections of h are one product; q, the latent and the gate logits stay float32 until the norm, q' and the
sigmoid have been computed in 32-bit.  No positions enter.
"""
from __future__ import annotations

import torch

from .. import perf
from ..cache import KVRequest
from ..errors import UnsupportedModel
from ..kernels import ops
from ..weights.params import ParamSpec
from .base import Mixer, register_mixer

MAX_LATENT = 1024       # the 32-bit attention kernel keeps a head's output lanes in registers, eight a thread


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    accepts_deferred_norm = True    # x goes to Runtime.linear, which finishes a norm's unfinished output

    def __init__(self, spec, reads_other_cache: bool = False):
        if reads_other_cache:
            raise UnsupportedModel(f"{spec.name}: a latent-attention layer on another layer's cache is not supported")
        if spec.latent_dim > MAX_LATENT:
            raise UnsupportedModel(f"{spec.name}: a latent of {spec.latent_dim} lanes (at most {MAX_LATENT})")
        s = self.spec = spec
        self.q_size = s.n_heads * s.head_dim
        self.gate_size = s.n_heads if s.head_gate else 0
        self.proj_size = self.q_size + s.latent_dim + self.gate_size
        self.out_size = s.n_heads * s.v_head_dim

    def kv_request(self):
        return KVRequest(1, self.spec.latent_dim, keys_only=True)

    def params(self):
        s = self.spec
        p = [ParamSpec(f"{s.name}.q", (self.q_size, s.hidden_size)),
             ParamSpec(f"{s.name}.dkv", (s.latent_dim, s.hidden_size)),
             ParamSpec(f"{s.name}.dkv.norm", (s.latent_dim,), init=("one_plus_normal", 0.1)),
             ParamSpec(f"{s.name}.uk", (self.q_size, s.latent_dim), init=("normal", 0.05)),
             ParamSpec(f"{s.name}.uv", (self.out_size, s.latent_dim), init=("normal", 0.05))]
        if s.head_gate:
            p.append(ParamSpec(f"{s.name}.g", (s.n_heads, s.hidden_size), init=("normal", 0.05)))
        p.append(ParamSpec(f"{s.name}.o", (s.hidden_size, self.out_size)))
        return p

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        ws = [tensors.pop(f"{s.name}.q"), tensors.pop(f"{s.name}.dkv")]
        if s.head_gate:
            ws.append(tensors.pop(f"{s.name}.g"))
        self.w_in = torch.cat(ws, dim=0).contiguous()       # rows: q heads, the latent, the gate logits
        del ws
        self.w_norm = tensors[f"{s.name}.dkv.norm"]
        # head a's W_uk[a] is [d, r]; q' = W_uk[a]^T q needs it as [r, d] (out, in)
        self.w_uk_t = tensors.pop(f"{s.name}.uk").view(s.n_heads, s.head_dim, s.latent_dim).transpose(1, 2).contiguous()
        self.w_uv = tensors[f"{s.name}.uv"].view(s.n_heads, s.v_head_dim, s.latent_dim)
        self.w_o = tensors[f"{s.name}.o"]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_uk_t, self.w_uv, self.w_o))

    def forward(self, ctx, x, residual, cache):
        s, rt = self.spec, self.rt
        n, H, r = x.shape[0], s.n_heads, s.latent_dim
        proj = rt.empty(n, self.proj_size, dtype=torch.float32)
        with rt.phase("attn_qkv", self.w_in, n):
            rt.linear(x, self.w_in, None, proj)
        fast = self._tensor_core_attention(cache)
        lat_dt = torch.bfloat16 if fast else torch.float32
        q_lat, o_lat, heads = rt.empty(n, H * r, dtype=lat_dt), rt.empty(n, H * r, dtype=lat_dt), rt.empty(n, self.out_size)
        # the two per-head products run on the tensor cores where the sizes allow it (the queries are rounded to
        # bfloat16 for that, where the norm's kernel passes over the row anyway), else in 32-bit on the CUDA cores
        q16 = rt.empty(n, self.q_size, dtype=torch.bfloat16)
        absorb_tc = fast and ops.linear_heads_tc_supported(q16, 0, self.w_uk_t, q_lat)
        expand_tc = fast and ops.linear_heads_tc_supported(o_lat, 0, self.w_uv, heads)
        with rt.phase("attn_rope"):
            ops.latent_append(proj, self.q_size, self.w_norm, s.eps, ctx.tok_seq, ctx.tok_pos, cache.block_table,
                              cache.k_pages, q16 if absorb_tc else None)
        with rt.phase("attn_absorb", self.w_uk_t, n):
            if absorb_tc:
                ops.linear_heads_tc(q16, self.w_uk_t, q_lat, rt.workspace)
            else:
                ops.linear_heads(proj, 0, self.w_uk_t, q_lat)
        with self._core_phase(ctx, cache):
            self._attend(ctx, q_lat, cache, o_lat, fast)
        gate = proj if s.head_gate else None
        with rt.phase("attn_expand", self.w_uv, n):
            if expand_tc:
                ops.linear_heads_tc(o_lat, self.w_uv, heads, rt.workspace, gate=gate, gate_col=self.q_size + r)
            else:
                ops.linear_heads(o_lat, 0, self.w_uv, heads, gate=gate, gate_col=self.q_size + r)
        with rt.phase("attn_out", self.w_o, n):
            rt.linear(heads, self.w_o, None, residual, accumulate=not getattr(ctx, "branch_is_fresh", False),
                      then_norm=getattr(ctx, "next_norm", None))

    def _tensor_core_attention(self, cache) -> bool:
        s = self.spec
        return (self.rt.dtype == torch.bfloat16 and cache.k_pages.dtype == torch.bfloat16
                and ops.attention_mma_supported(s.n_heads, 1, s.latent_dim))

    def _core_phase(self, ctx, cache):
        if not perf.enabled():
            return perf._NULL
        s = self.spec
        keys = ctx.span_sum()
        return self.rt.phase("attn_core", nbytes=1.0 * keys * s.latent_dim * cache.k_pages.element_size(),
                             flops=4.0 * keys * s.n_heads * s.latent_dim)

    def _attend(self, ctx, q, cache, out, fast: bool):
        """H query heads on the one key/value head of the latent, values = keys."""
        s, rt = self.spec, self.rt
        H, r = s.n_heads, s.latent_dim
        pages = cache.k_pages
        if not fast:
            ops.attention(q, pages, pages, cache.block_table, ctx.tok_seq, ctx.tok_pos, out, H, 1, r, s.scale)
        elif ctx.is_decode:
            n_splits = ops.attention_decode_splits(ctx.n_tokens, 1, ctx.max_kv_len, rt.sm_count)
            floats = 0 if n_splits <= ops.DECODE_CLUSTER_MAX_SPLITS else ops.attention_decode_scratch_floats(
                ctx.n_tokens, H, 1, r, n_splits)
            scratch = rt.empty(floats, dtype=torch.float32) if floats else None
            ops.attention_decode_mma(q, pages, pages, cache.block_table, ctx.tok_seq, ctx.tok_pos, out, scratch, H, 1, r,
                                     s.scale, 0, n_splits)
        elif ctx.n_tokens >= 32 * ctx.n_seqs and ops.attention_prefill_tc_supported(H, 1, r, q, pages, out):
            ops.attention_prefill_tc(q, pages, pages, cache.block_table, ctx.cu_seqlens, ctx.tok_pos, out,
                                     rt.workspace.status, ctx.n_seqs, H, 1, r, s.scale, 0)
        else:
            ops.attention_prefill_mma(q, pages, pages, cache.block_table, ctx.cu_seqlens, ctx.tok_pos, out, ctx.n_seqs,
                                      H, 1, r, s.scale, 0)

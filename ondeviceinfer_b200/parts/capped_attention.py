"""Grouped-query attention with rotated, unit-normed queries and keys, squashed scores and a window.

Steps of ``forward``: one matrix product for the concatenated q, k, v projections (v heads have a width of their
own); head preparation (``csrc/capped.cu``): rotation of neighbouring-lane pairs, then every q and k head divided
by its root mean square, q to the query buffer, k and v to the token's row of the paged cache (a ring of pages
per sequence when the layer has a window); attention over the cache pages with the scores squashed by
c tanh(score / c) and keys outside the window left out (bfloat16 with heads in steps of 16:
``csrc/attention_capped_mma.cu`` on the tensor cores, a form for prompts and portions and a split-key form for
single tokens; prompts with key and value heads of 64 or 128 lanes: ``csrc/attention_tcgen05.cu``, the kernel of
the plain attention, which takes the window, the ring and the cap as arguments; float32 and other head sizes: the
CUDA-core kernel ``csrc/attention_simt.cu``); the output projection.  Rotation, unit norm, scores and
softmax are fp32 in both compute dtypes.  Every constant (scale, cap, window, eps, rotated lanes, frequency
scaling) is a field of the spec; a field that is None switches its mechanism off.
"""

from __future__ import annotations

import torch

from ..cache import PAGE_SIZE, KVNeed
from ..config.specs import CappedAttentionSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, build_part, register_part
from .attention import TCGEN05_MIN_Q_LEN
from .linear import linear


class CappedAttention(Part):
    graph_safe = True   # no host work that depends on the step's values: may be captured in a CUDA graph
    returns_output = True   # forward(..., residual=None) returns the fp32 output instead of adding it

    def __init__(self, spec: CappedAttentionSpec) -> None:
        super().__init__(spec)
        if spec.num_heads <= 0 or spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError("query heads must be a positive multiple of the key/value heads")
        if not 1 <= spec.head_dim <= 512:
            raise ValueError(f"head_dim={spec.head_dim}: the attention kernels take heads of up to 512 lanes")
        # the attention kernel reads heads four lanes at a time: stored q and k heads are padded with zero lanes
        self.lanes = -(-spec.head_dim // 4) * 4
        if spec.value_dim <= 0:
            raise ValueError("value_dim must be positive")
        if spec.values_are_keys and spec.value_dim != spec.head_dim:
            raise ValueError("values that are the keys have the keys' width")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("window must be positive")
        if spec.softcap is not None and spec.softcap <= 0:
            raise ValueError("softcap must be positive")
        if spec.keep_first < 0 or (spec.keep_first > 0 and spec.window is None):
            raise ValueError("keep_first is a number of first positions kept beside a window")
        if spec.has("q_norm") != spec.has("k_norm") or (spec.has("q_norm") and spec.unit_norm_eps is None):
            raise ValueError("weights of the per-head norm come in a pair and go with unit_norm_eps")
        self.position = build_part(spec.position)
        if self.position.rot_dim > 0 and not getattr(self.position, "interleaved", False):
            raise ValueError("this attention's head preparation rotates neighbouring-lane pairs only")

    # ------------------------------------------------------------------ tensors

    def tensor_decls(self):
        s = self.spec
        q, k, v = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim, s.num_kv_heads * s.value_dim
        decls = [TensorDecl(s.name("q"), (q, s.hidden_size)), TensorDecl(s.name("k"), (k, s.hidden_size))]
        if not s.values_are_keys:
            decls.append(TensorDecl(s.name("v"), (v, s.hidden_size)))
        decls.append(TensorDecl(s.name("o"), (s.hidden_size, s.num_heads * s.value_dim)))
        decls += [TensorDecl(s.name(role), (size,)) for role, size in (("q_bias", q), ("k_bias", k)) if s.has(role)]
        decls += [TensorDecl(s.name(role), (s.head_dim,), "one_plus_normal") for role in ("q_norm", "k_norm") if s.has(role)]
        return decls + self.position.tensor_decls()

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        # q, k and v rows concatenated: one product yields [tokens, nq d + nkv d + nkv dv] (no v rows when the
        # values are the keys)
        rows = [fetch.matrix(s.name("q")), fetch.matrix(s.name("k"))]
        if not s.values_are_keys:
            rows.append(fetch.matrix(s.name("v")))
        self.w_qkv = torch.cat(rows, 0)
        self.w_o = fetch.matrix(s.name("o"))
        # biases (fp32) concatenated like their weights; a projection without one adds zero
        self.b_qkv = None
        if s.has("q_bias") or s.has("k_bias"):
            sizes = (("q_bias", s.num_heads * s.head_dim), ("k_bias", s.num_kv_heads * s.head_dim),
                     ("v_bias", 0 if s.values_are_keys else s.num_kv_heads * s.value_dim))
            self.b_qkv = torch.cat([fetch.vector(s.name(role)) if s.has(role)
                                    else torch.zeros(size, dtype=torch.float32, device=runtime.device)
                                    for role, size in sizes])
        self.q_norm_w = fetch.vector(s.name("q_norm")) if s.has("q_norm") else None
        self.k_norm_w = fetch.vector(s.name("k_norm")) if s.has("k_norm") else None
        self.position.load(fetch, runtime)

    def cache_needs(self):
        s = self.spec
        return (KVNeed(s.num_kv_heads, self.lanes, s.window, value_dim=s.value_dim, keep_first=s.keep_first),)

    # ------------------------------------------------------------------ step

    def forward(self, x, ctx, view, residual):
        """Adds the mixer's output to ``residual`` (fp32); with ``residual`` None returns it as a new fp32 tensor."""
        s = self.spec
        n = x.shape[0]
        group = view.kv_group
        page_start, page_ids = ctx.page_table(group.index)
        tables = self.position.rotary_tables(ctx)
        cos, sin = tables if tables is not None else (None, None)
        q = torch.empty((n, s.num_heads * self.lanes), dtype=x.dtype, device=x.device)
        ops.rot_unit_prep(linear(x, self.w_qkv, bias=self.b_qkv), q, view.keys, view.values, cos, sin, ctx.tok_seq,
                          ctx.tok_pos, page_start, page_ids, nq=s.num_heads, nkv=s.num_kv_heads, d=s.head_dim,
                          dv=s.value_dim, rot_dim=self.position.rot_dim, page_size=PAGE_SIZE, ring_pages=group.ring_pages,
                          write_kv=view.writes_kv, unit_eps=s.unit_norm_eps, d_store=self.lanes,
                          v_from_k=s.values_are_keys, q_weight=self.q_norm_w, k_weight=self.k_norm_w)
        o = self.attend(q, ctx, view, page_start, page_ids)
        if residual is None:
            return linear(o, self.w_o, out_dtype=torch.float32)
        linear(o, self.w_o, residual=residual, track=ctx)
        return None

    def attend(self, q, ctx, view, page_start, page_ids):
        """The attention output [tokens, heads * value_dim]."""
        s = self.spec
        o = torch.empty((ctx.n_tokens, s.num_heads * s.value_dim), dtype=q.dtype, device=q.device)
        tensor_cores = ops.attention_capped_supported(q.dtype, self.lanes, s.value_dim)
        common = dict(n_seqs=ctx.n_seqs, nq=s.num_heads, nkv=s.num_kv_heads, d=self.lanes, dv=s.value_dim, page_size=PAGE_SIZE,
                      ring_pages=view.kv_group.ring_pages, window=s.window or 0, scale=s.scale, softcap=s.softcap or 0.0,
                      sink=s.sink, keep=s.keep_first)
        if (tensor_cores and ctx.max_q_len > TCGEN05_MIN_Q_LEN and self.lanes == s.value_dim
                and self.lanes in ops.TCGEN05_ATTENTION_HEAD_DIMS):
            # bf16 prompts with heads of 64 or 128 lanes: scores and outputs in tensor memory (tcgen05)
            ops.attention_tcgen05(q, view.keys, view.values, o, ctx.cu_q, ctx.past, page_start, page_ids, n_seqs=ctx.n_seqs,
                                  max_q_len=ctx.max_q_len, nq=s.num_heads, nkv=s.num_kv_heads, d=self.lanes, page_size=PAGE_SIZE,
                                  scale=s.scale, window=s.window or 0, ring_pages=view.kv_group.ring_pages,
                                  softcap=s.softcap or 0.0, sink=s.sink, keep=s.keep_first)
            return o
        if tensor_cores and ctx.max_q_len > 1:
            # other bf16 prompts and portions: the mma.sync form
            ops.attention_capped(q, view.keys, view.values, o, ctx.cu_q, ctx.past, page_start, page_ids,
                                 max_q_len=ctx.max_q_len, **common)
            return o
        splits, partial = 1, None
        if ctx.max_q_len == 1:
            # single tokens: cut the visible keys so that enough blocks run side by side
            block_rows = s.num_kv_heads * ((s.num_heads // s.num_kv_heads + 15) // 16)
            keys = ctx.max_kv_len if s.window is None else min(ctx.max_kv_len, s.window + s.keep_first)
            if tensor_cores:
                tiles = (keys + 63) // 64 + (1 if s.window is not None else 0)      # a window may straddle one tile more
                tiles += 1 if s.keep_first > 0 else 0                               # and so may the kept first keys
                splits = max(1, min(32, 296 // max(ctx.n_seqs * block_rows, 1), tiles))
            else:
                splits = max(1, min(32, 296 // max(ctx.n_seqs * block_rows, 1), (keys + 255) // 256))
            if splits > 1:
                partial = torch.empty((ctx.n_tokens * s.num_heads * splits * (s.value_dim + 2),), dtype=torch.float32,
                                      device=q.device)
        if tensor_cores and ctx.max_q_len == 1:
            ops.attention_capped_decode(q, view.keys, view.values, o, ctx.cu_q, ctx.past, page_start, page_ids,
                                        splits=splits, partial=partial, **common)
            return o
        ops.attention_simt(q, view.keys, view.values, o, ctx.cu_q, ctx.past, page_start, page_ids,
                           max_q_len=ctx.max_q_len, splits=splits, partial=partial, **common)
        return o


register_part(CappedAttentionSpec, CappedAttention)

"""Latent attention: causal attention over a compressed cache of one latent row per position.

The cache row of a position is ``[c | k_rot]``: the normed latent (``kv_rank`` lanes) and the rotated key lanes
that all heads share.  Keys and values are never expanded.  Since a head's plain key is ``W_uk c`` and its
value ``W_uv c``, the score ``q_plain . W_uk c + q_rot . k_rot`` equals ``[W_uk^T q_plain | q_rot] . [c | k_rot]``
and the output ``W_uv sum_j p_j c_j``: the key up-projection is folded into the query, attention runs with one
shared key/value row per position (the value being the row's first ``kv_rank`` lanes), and the value
up-projection is applied to the attention's output.  Steps of ``forward``:

1. one product for the query and the down projection;
2. head preparation (``csrc/latent.cu``): latent norm, rotation, cache write, rotated query lanes;
3. a product per head that folds ``W_uk`` into the plain query lanes (``csrc/grouped_gemm.cu``);
4. attention over the cache pages, split over the keys for single-token steps: on the tensor cores
   (``csrc/attention_latent_mma.cu``) for bfloat16 rows in steps of 16 lanes, else ``csrc/attention_simt.cu`` built
   for shared rows;
5. a product per head with ``W_uv``, then the output projection with the residual add.

A bfloat16 step whose sequences all start (prompts) takes the other way round instead, because whole heads are
what the tensor-core attention kernels take: keys and values are up-projected for the step's tokens (two
products), laid out as heads of ``head_lanes`` lanes in pages of the step's own (``latent_expand``), and the
prefill kernels for ordinary heads run on them; the output projection reads those padded heads through a copy
of its weight with zero columns for the padding.  The cache still receives only the latent rows.

Options of the spec: queries through a latent of their own (its norm is ``ops.slice_norm`` on a slice of the first
product, then a second product), a window (an argument of every attention kernel used; the cache is then a ring of
pages), an output gate (``ops.gate_heads`` on the heads before the output projection), and a layer without a down
projection that reads the rows another layer execution cached (in the whole-heads form it takes the step's latent
rows from the step's context, where the layer that wrote them left them).

Scores, softmax, the latent norms and the angles are fp32 in both compute dtypes.
"""

from __future__ import annotations

import torch

from ..cache import PAGE_SIZE, KVNeed
from ..config.specs import LatentAttentionSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, build_part, register_part
from .linear import linear

WHOLE_HEADS_MIN_TOKENS = 32      # shorter prompts stay with the kernel over the latent rows
WHOLE_HEADS_MAX_LANES = 256      # the widest head of the tensor-core prefill kernels


class LatentAttention(Part):
    graph_safe = True   # no host work that depends on the step's values
    returns_output = True   # forward(..., residual=None) returns the fp32 output instead of adding it

    def __init__(self, spec: LatentAttentionSpec) -> None:
        super().__init__(spec)
        for key in ("num_heads", "qk_dim", "v_dim", "kv_rank"):
            if getattr(spec, key) <= 0:
                raise ValueError(f"{key} must be positive, got {getattr(spec, key)}")
        if spec.rot_dim < 0:
            raise ValueError("rot_dim must not be negative")
        if spec.q_rank is not None and spec.q_rank <= 0:
            raise ValueError("q_rank must be positive")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("window must be positive")
        self.position = build_part(spec.position)
        if self.position.rot_dim > spec.rot_dim:
            raise ValueError("the position encoding rotates more lanes than the heads have rotated lanes")
        # width of a cache row and of an absorbed query: the attention kernels read rows 16 lanes at a time on the
        # tensor cores (which take latents in steps of 16) and four at a time otherwise, so the lanes are rounded up
        # and the ones beyond kv_rank + rot_dim stay zero in the cache and in the query
        step = 16 if spec.kv_rank % 16 == 0 else 4
        self.row = -(-(spec.kv_rank + spec.rot_dim) // step) * step
        self.padded = self.row != spec.kv_rank + spec.rot_dim
        # lanes of a whole head (query/key: plain + rotated; value), in the steps of 16 the prefill kernels take
        self.head_lanes = -(-max(spec.qk_dim + spec.rot_dim, spec.v_dim) // 16) * 16

    def tensor_decls(self):
        s = self.spec
        q = s.num_heads * (s.qk_dim + s.rot_dim)
        if s.q_rank is None:
            decls = [TensorDecl(s.name("q"), (q, s.hidden_size))]
        else:
            decls = [TensorDecl(s.name("dq"), (s.q_rank, s.hidden_size)),
                     TensorDecl(s.name("dq_norm"), (s.q_rank,), "one_plus_normal"),
                     TensorDecl(s.name("uq"), (q, s.q_rank))]
        if s.own_kv:
            decls += [TensorDecl(s.name("dkv"), (s.kv_rank + s.rot_dim, s.hidden_size)),
                      TensorDecl(s.name("dkv_norm"), (s.kv_rank,), "one_plus_normal")]
        decls += [TensorDecl(s.name("uk"), (s.num_heads * s.qk_dim, s.kv_rank)),
                  TensorDecl(s.name("uv"), (s.num_heads * s.v_dim, s.kv_rank))]
        if s.gated:
            decls.append(TensorDecl(s.name("g"), (s.num_heads * (1 if s.gate_per_head else s.v_dim), s.hidden_size)))
        return decls + [TensorDecl(s.name("o"), (s.hidden_size, s.num_heads * s.v_dim))] + self.position.tensor_decls()

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        # One product for everything that reads the layer's input.  Queries without a latent of their own:
        # [q | down projection] (the gate, if any, is a product of its own).  Queries through a latent:
        # [down projection | query latent | gate], the down projection first so that its lanes start a row.
        self.w_gate = self.w_uq = self.q_norm = None
        down = [fetch.matrix(s.name("dkv"))] if s.own_kv else []
        self.gate_in_first = False
        if s.q_rank is None:
            rows = [fetch.matrix(s.name("q"))] + down
            if s.gated and s.gate_per_head:
                # a gate of one row per head is too small for a product of its own: its rows follow the others,
                # with zero rows up to a multiple of eight so that the product's rows stay 16-byte aligned
                g = fetch.matrix(s.name("g"))
                rows += [g, torch.zeros(((-s.num_heads) % 8, s.hidden_size), dtype=g.dtype, device=g.device)]
                self.gate_in_first = True
            elif s.gated:
                self.w_gate = fetch.matrix(s.name("g"))
            self.w_in = torch.cat(rows, 0)
        else:
            self.w_in = torch.cat(down + [fetch.matrix(s.name("dq"))] + ([fetch.matrix(s.name("g"))] if s.gated else []), 0)
            self.w_uq = fetch.matrix(s.name("uq"))
            self.q_norm = fetch.vector(s.name("dq_norm"))
        self.latent_norm = fetch.vector(s.name("dkv_norm")) if s.own_kv else None
        # per head: [kv_rank, qk_dim] so that q_plain W gives the query in latent lanes; [v_dim, kv_rank] as stored
        self.w_uk_t = fetch.matrix(s.name("uk")).view(s.num_heads, s.qk_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = fetch.matrix(s.name("uv")).view(s.num_heads, s.v_dim, s.kv_rank).contiguous()
        self.w_o = fetch.matrix(s.name("o"))
        self.w_uk = self.w_uv_rows = self.w_o_padded = None
        if runtime.dtype == torch.bfloat16 and self.head_lanes <= WHOLE_HEADS_MAX_LANES:
            self.w_uk = fetch.matrix(s.name("uk"))
            self.w_uv_rows = self.w_uv.view(s.num_heads * s.v_dim, s.kv_rank)
            padded = torch.zeros((s.hidden_size, s.num_heads, self.head_lanes), dtype=self.w_o.dtype, device=self.w_o.device)
            padded[:, :, :s.v_dim] = self.w_o.view(s.hidden_size, s.num_heads, s.v_dim)
            self.w_o_padded = padded.view(s.hidden_size, s.num_heads * self.head_lanes)
        self.position.load(fetch, runtime)

    def cache_needs(self):
        return (KVNeed(1, self.row, self.spec.cache_window, value_plane=False),)

    def forward(self, x, ctx, view, residual):
        """Adds the mixer's output to ``residual`` (fp32); with ``residual`` None returns it as a new fp32 tensor."""
        s = self.spec
        n = x.shape[0]
        group = view.kv_group
        page_start, page_ids = ctx.page_table(group.index)
        proj = linear(x, self.w_in)
        gate, gate_col, down = None, 0, None
        if s.q_rank is None:
            queries = proj          # with the down projection behind the heads, if the layer has one
            if self.gate_in_first:
                gate, gate_col = proj, s.num_heads * (s.qk_dim + s.rot_dim) + (s.kv_rank + s.rot_dim if s.own_kv else 0)
            elif s.gated:
                gate = linear(x, self.w_gate)
        else:
            at = s.kv_rank + s.rot_dim if s.own_kv else 0
            latent_q = torch.empty((n, s.q_rank), dtype=proj.dtype, device=proj.device)
            ops.slice_norm(proj, self.q_norm, s.norm_eps, latent_q, col=at)
            queries = linear(latent_q, self.w_uq)
            down = proj if s.own_kv else None
            gate, gate_col = (proj, at + s.q_rank) if s.gated else (None, 0)
        tables = self.position.rotary_tables(ctx)
        cos, sin = tables if tables is not None else (None, None)
        q_abs = (torch.zeros if self.padded else torch.empty)((n, s.num_heads * self.row), dtype=proj.dtype,
                                                              device=proj.device)
        # a bfloat16 step whose sequences all start: whole heads for the tensor-core kernels, if this layer has the
        # step's latent rows at hand (its own, or the ones that the layer whose cache it reads left on the context)
        step_whole = (proj.dtype == torch.bfloat16 and ctx.max_q_len >= WHOLE_HEADS_MIN_TOKENS
                      and not any(ctx.past_lens) and not torch.cuda.is_current_stream_capturing())
        shared_key = ("latent rows of the step", view.keys.data_ptr())
        latent = key_rot = None
        if step_whole and s.own_kv:
            latent = torch.empty((n, s.kv_rank), dtype=proj.dtype, device=proj.device)
            key_rot = torch.empty((n, s.rot_dim), dtype=proj.dtype, device=proj.device)
        ops.latent_prep(queries, q_abs, view.keys, self.latent_norm, cos, sin, ctx.tok_seq, ctx.tok_pos, page_start,
                        page_ids, heads=s.num_heads, d=s.qk_dim, r=s.rot_dim, R=s.kv_rank,
                        rot_dims=self.position.rot_dim if cos is not None else 0,
                        interleaved=getattr(self.position, "interleaved", False), page_size=PAGE_SIZE,
                        ring_pages=group.ring_pages, write_cache=s.own_kv and view.writes_kv, eps=s.norm_eps,
                        latent_out=latent, key_rot_out=key_rot, row=self.row, down=down, has_down=s.own_kv,
                        trailing=-(-s.num_heads // 8) * 8 if self.gate_in_first else 0)
        if step_whole:
            if s.own_kv and view.writes_kv:
                ctx.memo(shared_key, lambda: (latent, key_rot))
            elif not s.own_kv:
                latent, key_rot = ctx.memo(shared_key, lambda: (None, None))
        if step_whole and self.w_o_padded is not None and latent is not None:
            out, w_o = self._attend_whole_heads(queries, q_abs, latent, key_rot, ctx), self.w_o_padded
            lanes = self.head_lanes
        else:
            ops.grouped_gemm_heads(queries, self.w_uk_t, q_abs, a_col=0, a_stride=s.qk_dim + s.rot_dim, c_col=0,
                                   c_stride=self.row, K=s.qk_dim)
            latent_out = self.attend(q_abs, ctx, view, page_start, page_ids)
            out = torch.empty((n, s.num_heads * s.v_dim), dtype=proj.dtype, device=proj.device)
            ops.grouped_gemm_heads(latent_out, self.w_uv, out, a_col=0, a_stride=s.kv_rank, c_col=0,
                                   c_stride=s.v_dim, K=s.kv_rank)
            w_o, lanes = self.w_o, s.v_dim
        if s.gated:
            ops.gate_heads(out, gate, heads=s.num_heads, dv=s.v_dim, lanes=lanes, col=gate_col, per_head=s.gate_per_head)
        if residual is None:
            return linear(out, w_o, out_dtype=torch.float32)
        linear(out, w_o, residual=residual, track=ctx)
        return None

    def _attend_whole_heads(self, proj, q_abs, latent, key_rot, ctx):
        """Prompts from their first token on: attention over up-projected heads in pages of the step's own; returns
        the padded heads [tokens, heads * head_lanes]."""
        s, n, lanes, dev = self.spec, proj.shape[0], self.head_lanes, proj.device

        def pages_of_the_step():
            counts = [-(-t // PAGE_SIZE) for t in ctx.q_lens]
            starts = [0]
            for c in counts:
                starts.append(starts[-1] + c)
            table = torch.tensor(starts + list(range(starts[-1])) + [0] * ctx.n_seqs, dtype=torch.int32).to(dev)
            return (table[:ctx.n_seqs + 1], table[ctx.n_seqs + 1:ctx.n_seqs + 1 + starts[-1]],
                    table[ctx.n_seqs + 1 + starts[-1]:], starts[-1])

        page_start, page_ids, no_past, n_pages = ctx.memo("pages of a step whose sequences all start", pages_of_the_step)
        k_plain = linear(latent, self.w_uk)
        values = linear(latent, self.w_uv_rows)
        # zeros: a page's rows beyond its sequence's end are multiplied by weights of zero
        pools = torch.zeros((2, n_pages, s.num_heads, PAGE_SIZE, lanes), dtype=proj.dtype, device=dev)
        q_full = torch.empty((n, s.num_heads * lanes), dtype=proj.dtype, device=dev)
        ops.latent_expand(proj, q_abs, k_plain, key_rot, values, q_full, pools[0], pools[1], ctx.tok_seq, ctx.cu_q,
                          page_start, heads=s.num_heads, d=s.qk_dim, r=s.rot_dim, R=s.kv_rank, dv=s.v_dim, Dh=lanes,
                          page_size=PAGE_SIZE, row=self.row)
        out = torch.empty_like(q_full)
        sizes = dict(n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, nq=s.num_heads, nkv=s.num_heads, d=lanes,
                     page_size=PAGE_SIZE, scale=s.scale)
        window = s.window or 0
        if lanes in ops.TCGEN05_ATTENTION_HEAD_DIMS:
            ops.attention_tcgen05(q_full, pools[0], pools[1], out, ctx.cu_q, no_past, page_start, page_ids, window=window,
                                  ring_pages=0, **sizes)
        elif window > 0:
            ops.attention_capped(q_full, pools[0], pools[1], out, ctx.cu_q, no_past, page_start, page_ids, dv=lanes,
                                 ring_pages=0, window=window, **sizes)
        else:
            ops.attention_mma(q_full, pools[0], pools[1], out, ctx.cu_q, no_past, page_start, page_ids, **sizes)
        return out

    def attend(self, q_abs, ctx, view, page_start, page_ids):
        """[tokens, heads * kv_rank]: per head the softmax-weighted sum of the latents it sees."""
        s = self.spec
        out = torch.empty((ctx.n_tokens, s.num_heads * s.kv_rank), dtype=q_abs.dtype, device=q_abs.device)
        tensor_cores = ops.attention_latent_supported(q_abs.dtype, self.row, s.kv_rank, PAGE_SIZE)
        splits, partial = 1, None
        if ctx.max_q_len == 1:
            # single tokens: cut long key ranges so that enough blocks run side by side (a block of the tensor-core
            # kernel fills a multiprocessor; two of the other kernel's fit)
            blocks = ctx.n_seqs * ((s.num_heads + 15) // 16)
            keys = ctx.max_kv_len if s.window is None else min(ctx.max_kv_len, s.window + PAGE_SIZE)
            room = 148 if tensor_cores else 592
            splits = max(1, min(32, room // max(blocks, 1), (keys + 63) // 64))
            if splits > 1:
                partial = torch.empty((ctx.n_tokens * s.num_heads * splits * (s.kv_rank + 2),), dtype=torch.float32,
                                      device=q_abs.device)
        if tensor_cores:
            ops.attention_latent(q_abs, view.keys, out, ctx.cu_q, ctx.past, page_start, page_ids, n_seqs=ctx.n_seqs,
                                 max_q_len=ctx.max_q_len, nq=s.num_heads, d=self.row, dv=s.kv_rank, page_size=PAGE_SIZE,
                                 ring_pages=view.kv_group.ring_pages, window=s.window or 0, scale=s.scale, splits=splits,
                                 partial=partial)
            return out
        ops.attention_simt(q_abs, view.keys, None, out, ctx.cu_q, ctx.past, page_start, page_ids, n_seqs=ctx.n_seqs,
                           max_q_len=ctx.max_q_len, nq=s.num_heads, nkv=1, d=self.row, dv=s.kv_rank, shared_kv=True,
                           page_size=PAGE_SIZE, ring_pages=view.kv_group.ring_pages, window=s.window or 0, scale=s.scale,
                           splits=splits, partial=partial)
        return out


register_part(LatentAttentionSpec, LatentAttention)

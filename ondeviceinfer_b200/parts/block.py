"""Arrangement of norms, mixer and feed-forward in a layer."""

from __future__ import annotations

import torch

from ..cache import StateNeed
from ..config.specs import ParallelBlockSpec, PreNormBlockSpec, ReinjectSpec, SandwichBlockSpec, ScaledParallelBlockSpec
from ..weights.tensors import TensorDecl
from .base import Part, build_part, register_part


class PreNormBlock(Part):
    """h += mixer(norm(h)); h += feed_forward(norm(h))  (ondeviceinfer/model.py:49-63); the second half is
    left out for a spec without a feed-forward."""

    finishes_residual_adds = True     # its norms take over a residual add that a product left pending

    def __init__(self, spec: PreNormBlockSpec) -> None:
        super().__init__(spec)
        self.mixer_norm = build_part(spec.mixer_norm)
        self.mixer = build_part(spec.mixer)
        # a layer without a feed-forward has neither the part nor its norm
        self.ffn_norm = build_part(spec.ffn_norm) if spec.ffn is not None else None
        self.ffn = build_part(spec.ffn) if spec.ffn is not None else None

    def _children(self):
        return tuple(part for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if part is not None)

    def tensor_decls(self):
        return [d for part in self._children() for d in part.tensor_decls()]

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        for part in self._children():
            part.load(fetch, runtime)

    def cache_needs(self):
        return tuple(self.mixer.cache_needs())

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self._children())

    @staticmethod
    def _normed(norm, consumer, hidden, ctx):
        """norm(hidden); left to the consumer's first product when the product that wrote ``hidden``
        has left the rows' sums of squares in ``ctx.residual_sumsq`` and both sides know how."""
        known = getattr(ctx, "residual_sumsq", None)
        ctx.residual_sumsq = None
        pending = getattr(ctx, "pending_residual_add", None)
        if pending is not None:
            # a product of the part before is still to be added to the stream: in this norm's pass if it is
            # this stream and the norm knows how, else now
            if len(pending) == 2 and pending[0] is hidden and getattr(norm, "adds", False):
                ctx.pending_residual_add = None
                return norm(hidden, add=pending[1])
            from .linear import flush_residual_add
            flush_residual_add(ctx)
        if known is not None and known[0] is hidden and getattr(norm, "lazy", None) is not None and getattr(consumer, "takes_lazy_norm", False):
            return norm.lazy(hidden, known[1])
        return norm(hidden)

    def forward(self, hidden, ctx, view) -> None:
        # This block finishes residual adds that its parts' last products leave pending (in the norm that follows,
        # here or in the next block; the model flushes the last one): it says so, and only then is an add deferred.
        ctx.defers_residual_add = True
        self.mixer.forward(self._normed(self.mixer_norm, self.mixer, hidden, ctx), ctx, view, hidden)
        if self.ffn is not None:
            self.ffn.forward(self._normed(self.ffn_norm, self.ffn, hidden, ctx), ctx, hidden)


class SandwichBlock(Part):
    """h += post_norm(mixer(norm(h))); h += post_norm(feed_forward(norm(h))): a norm on both sides of each sublayer.

    A sublayer's output is taken in fp32, normed in fp32 and added to the fp32 stream in one kernel
    (``ops.rmsnorm_add``), or, when the next sublayer's norm follows at once, together with that norm
    (``ops.rmsnorm_add_norm``): the block leaves the add pending on the step's context (``(hidden, output, weight,
    eps)``), the next norm of this or the following block of this kind finishes it, and the model flushes what is
    left.  A part that says ``returns_output`` (its ``forward`` returns the output when given no residual) is
    asked for that; any other part adds into a zeroed fp32 buffer, as the part interface says, so every
    registered mixer and feed-forward fits."""

    finishes_residual_adds = True     # its norms take over an add that the block before left pending

    def __init__(self, spec: SandwichBlockSpec) -> None:
        super().__init__(spec)
        self.mixer_norm = build_part(spec.mixer_norm)
        self.mixer = build_part(spec.mixer)
        self.mixer_post_norm = build_part(spec.mixer_post_norm)
        has = spec.ffn is not None
        self.ffn_norm = build_part(spec.ffn_norm) if has else None
        self.ffn = build_part(spec.ffn) if has else None
        self.ffn_post_norm = build_part(spec.ffn_post_norm) if has else None
        for norm in (self.mixer_post_norm, self.ffn_post_norm):
            if norm is not None and not hasattr(norm.spec, "eps"):
                raise TypeError("the norm after a sublayer must be an RMS norm (a weight and eps)")

    def _children(self):
        return tuple(part for part in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.ffn_norm, self.ffn,
                                       self.ffn_post_norm) if part is not None)

    def tensor_decls(self):
        return [d for part in self._children() for d in part.tensor_decls()]

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        for part in self._children():
            part.load(fetch, runtime)

    def cache_needs(self):
        return tuple(self.mixer.cache_needs())

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self._children())

    @staticmethod
    def _branch(part, hidden, call):
        """The fp32 output of a sublayer: ``call(residual)`` runs it."""
        if getattr(part, "returns_output", False):
            return call(None)
        branch = torch.zeros_like(hidden)
        call(branch)
        return branch

    @staticmethod
    def _normed(norm, hidden, ctx):
        """norm(hidden) for the next sublayer; a sublayer output that is still to be normed and added to this
        stream is finished in the same kernel when the norm allows it, else beforehand."""
        from ..kernels import ops
        from .linear import flush_residual_add
        pending = getattr(ctx, "pending_residual_add", None)
        if (pending is not None and len(pending) == 4 and pending[0] is hidden
                and getattr(norm.spec, "scale_in_fp32", False) and hasattr(norm, "weight")):
            out = torch.empty(hidden.shape, dtype=norm.runtime.dtype, device=hidden.device)
            if ops.rmsnorm_add_norm(hidden, pending[1], pending[2], pending[3], norm.weight, norm.spec.eps, out):
                ctx.pending_residual_add = None
                return out
        flush_residual_add(ctx)
        return norm(hidden)

    def forward(self, hidden, ctx, view) -> None:
        ctx.defers_residual_add = False        # the parts' own products add (or return) at once
        normed = self._normed(self.mixer_norm, hidden, ctx)
        out = self._branch(self.mixer, hidden, lambda r: self.mixer.forward(normed, ctx, view, r))
        ctx.pending_residual_add = (hidden, out, self.mixer_post_norm.weight, self.mixer_post_norm.spec.eps)
        if self.ffn is not None:
            normed = self._normed(self.ffn_norm, hidden, ctx)
            out = self._branch(self.ffn, hidden, lambda r: self.ffn.forward(normed, ctx, r))
            ctx.pending_residual_add = (hidden, out, self.ffn_post_norm.weight, self.ffn_post_norm.spec.eps)
        ctx.residual_sumsq = None


class ParallelBlock(Part):
    """h = norm(x); x += m (mixer(h + conv(h)) + feed_forward(h)): one norm whose output both sublayers read, a
    short causal convolution over time in front of the mixer, one scaled add.

    ``ops.canon_norm`` makes h and h + conv(h) in one pass over the stream (the norm's weight is one number);
    the rows of h before a sequence's first token of the step come from the sequence's state, the fp32 h of its
    last taps - 1 positions (a :class:`~ondeviceinfer_b200.cache.StateNeed` of the block, zero when a sequence
    starts), which the same launch moves on for a sequence that brings one token and ``ops.canon_state`` for the
    others.  The mixer's fp32 output (a part that says ``returns_output``
    returns it; any other adds into a zeroed buffer) takes the feed-forward's as its residual add, and
    ``ops.scaled_add`` adds the sum to the stream."""

    def __init__(self, spec: ParallelBlockSpec) -> None:
        super().__init__(spec)
        self.norm = build_part(spec.norm)
        self.mixer = build_part(spec.mixer)
        self.ffn = build_part(spec.ffn) if spec.ffn is not None else None
        if not (getattr(spec.norm, "scalar_weight", False) and getattr(spec.norm, "scale_in_fp32", False)):
            raise TypeError("this block's norm has one number as its weight and scales in fp32")
        if spec.conv_taps < 1 or (spec.conv_name is None and spec.conv_taps != 1):
            raise ValueError("conv_taps is at least 1, and 1 without a convolution")
        if spec.conv_taps > 64:
            raise ValueError(f"the convolution kernels take up to 64 taps, got {spec.conv_taps}")
        self.taps = spec.conv_taps if spec.conv_name is not None else 1

    def _children(self):
        return tuple(part for part in (self.norm, self.mixer, self.ffn) if part is not None)

    def tensor_decls(self):
        decls = [d for part in self._children() for d in part.tensor_decls()]
        if self.spec.conv_name is not None:
            decls.append(TensorDecl(self.spec.conv_name, (self.spec.hidden_size, self.spec.conv_taps)))
        return decls

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        for part in self._children():
            part.load(fetch, runtime)
        if self.spec.conv_name is not None:
            self.taps_w = fetch.vector(self.spec.conv_name)
        else:       # no convolution: one tap of zero, h + 0 h
            self.taps_w = torch.zeros((self.spec.hidden_size, 1), dtype=torch.float32, device=runtime.device)

    def _state_need(self):
        return StateNeed((self.taps - 1, self.spec.hidden_size), torch.float32, "conv before the mixer")

    def cache_needs(self):
        needs = tuple(self.mixer.cache_needs())
        return needs + ((self._state_need(),) if self.taps > 1 else ())

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self._children())

    def forward(self, hidden, ctx, view) -> None:
        ctx.defers_residual_add = False        # the parts' own products add (or return) at once
        ctx.residual_sumsq = None
        state = view.states[-1] if self.taps > 1 else None      # the block's need is the last one it names
        n = hidden.shape[0]
        h = torch.empty((n, self.spec.hidden_size), dtype=self.runtime.dtype, device=hidden.device)
        hc = torch.empty_like(h)
        eps = self.norm.spec.eps
        from ..kernels import ops
        ops.canon_norm(hidden, self.norm.scalar, eps, self.taps_w, state, ctx.tok_seq, ctx.cu_q, ctx.slots, h, hc)
        if ctx.max_q_len > 1:       # the state of a sequence that brings one token moved on in the launch above
            ops.canon_state(hidden, self.norm.scalar, eps, self.taps_w, state, ctx.tok_seq, ctx.cu_q, ctx.slots)
        if getattr(self.mixer, "returns_output", False):
            branch = self.mixer.forward(hc, ctx, view, None)
        else:
            branch = torch.zeros_like(hidden)
            self.mixer.forward(hc, ctx, view, branch)
        if self.ffn is not None:
            self.ffn.forward(h, ctx, branch)
        ctx.residual_sumsq = None
        ops.scaled_add(hidden, branch, self.spec.residual_mult)


class ScaledParallelBlock(Part):
    """x <- x + s1 * mixer(norm1(x)) + s2 * feed_forward(norm2(x)), then an optional part that adds to the new stream.

    Both norms read the same rows, so ``ops.dual_norm`` makes them in one pass from one sum of squares (the norms
    must be RMS norms of one eps that scale in fp32).  Each sublayer's fp32 output (a part that says
    ``returns_output`` returns it; any other adds into a zeroed buffer) is multiplied lane by lane by its stored
    vector and added in ``ops.scaled_add2``, which also leaves the new rows in the compute dtype for the part after
    (``after.wants_copy``).  Norms, scales and sums are fp32 in both compute dtypes."""

    def __init__(self, spec: ScaledParallelBlockSpec) -> None:
        super().__init__(spec)
        self.mixer_norm = build_part(spec.mixer_norm)
        self.mixer = build_part(spec.mixer)
        has = spec.ffn is not None
        if has != (spec.ffn_norm is not None) or has != (spec.ffn_scale_name is not None):
            raise ValueError("a feed-forward comes with its norm and its scale, or none of the three")
        self.ffn_norm = build_part(spec.ffn_norm) if has else None
        self.ffn = build_part(spec.ffn) if has else None
        self.after = build_part(spec.after) if spec.after is not None else None
        for norm in (spec.mixer_norm, spec.ffn_norm):
            if norm is not None and not (getattr(norm, "scale_in_fp32", False) and not getattr(norm, "scalar_weight", False)):
                raise TypeError("this block's norms are RMS norms with a weight per lane that scale in fp32")
        self.one_pass = has and spec.mixer_norm.eps == spec.ffn_norm.eps

    def _children(self):
        return tuple(part for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.after) if part is not None)

    def tensor_decls(self):
        s = self.spec
        decls = [d for part in self._children() for d in part.tensor_decls()]
        decls.append(TensorDecl(s.mixer_scale_name, (s.hidden_size,), "one_plus_normal"))
        if self.ffn is not None:
            decls.append(TensorDecl(s.ffn_scale_name, (s.hidden_size,), "one_plus_normal"))
        return decls

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        for part in self._children():
            part.load(fetch, runtime)
        self.mixer_scale = fetch.vector(self.spec.mixer_scale_name)
        self.ffn_scale = fetch.vector(self.spec.ffn_scale_name) if self.ffn is not None else None

    def cache_needs(self):
        return tuple(self.mixer.cache_needs())

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self._children())

    def forward(self, hidden, ctx, view) -> None:
        from ..kernels import ops
        ctx.defers_residual_add = False        # the parts' own products add (or return) at once
        ctx.residual_sumsq = None
        if self.one_pass:
            h1 = torch.empty(hidden.shape, dtype=self.runtime.dtype, device=hidden.device)
            h2 = torch.empty_like(h1)
            ops.dual_norm(hidden, self.mixer_norm.weight, self.ffn_norm.weight, self.mixer_norm.spec.eps, h1, h2)
        else:
            h1 = self.mixer_norm(hidden)
            h2 = self.ffn_norm(hidden) if self.ffn is not None else None
        if getattr(self.mixer, "returns_output", False):
            mixed = self.mixer.forward(h1, ctx, view, None)
        else:
            mixed = torch.zeros_like(hidden)
            self.mixer.forward(h1, ctx, view, mixed)
        fed = None
        if self.ffn is not None:
            if getattr(self.ffn, "returns_output", False):
                fed = self.ffn.forward(h2, ctx, None)
            else:
                fed = torch.zeros_like(hidden)
                self.ffn.forward(h2, ctx, fed)
        ctx.residual_sumsq = None
        copy = None
        if self.after is not None and getattr(self.after, "wants_copy", False):
            copy = torch.empty(hidden.shape, dtype=self.runtime.dtype, device=hidden.device)
        ops.scaled_add2(hidden, mixed, self.mixer_scale, fed, self.ffn_scale, copy)
        if self.after is not None:
            if copy is not None:
                self.after.forward(hidden, ctx, copy)
            else:
                self.after.forward(hidden, ctx)


class Reinject(Part):
    """h <- W [h ; e] + steps[index], e the embedding's output (``ctx.embedded``): what opens a pass of a looped
    stack.  It keeps no cache and returns the new stream (the model goes on with what a layer returns)."""

    graph_safe = True
    reads_embedding = True      # the model keeps the embedding's output on the step's context for it

    def tensor_decls(self):
        s = self.spec
        return [TensorDecl(s.weight_name, (s.hidden_size, 2 * s.hidden_size)),
                TensorDecl(s.steps_name, (s.num_steps, s.hidden_size))]

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        self.weight = fetch.matrix(self.spec.weight_name)
        self.step = fetch.vector(self.spec.steps_name)[self.spec.index].contiguous()

    def cache_needs(self):
        return ()

    def forward(self, hidden, ctx, view):
        from ..kernels import ops
        from .linear import linear
        both = torch.empty((hidden.shape[0], 2 * self.spec.hidden_size), dtype=self.runtime.dtype, device=hidden.device)
        ops.concat_cast(hidden, ctx.embedded, both)
        ctx.residual_sumsq = None
        return linear(both, self.weight, bias=self.step, out_dtype=torch.float32)


register_part(PreNormBlockSpec, PreNormBlock)
register_part(SandwichBlockSpec, SandwichBlock)
register_part(ParallelBlockSpec, ParallelBlock)
register_part(ScaledParallelBlockSpec, ScaledParallelBlock)
register_part(ReinjectSpec, Reinject)

"""A selective state-space mixer with one scalar decay per head: a recurrent mixer whose cache is a matrix state
per head and the last inputs of its short convolution.

Steps of ``forward``: one product for [z | x | B | C | dt]; then ``ops.ssd_mix`` (``csrc/ssd.cu``: the convolution
over x, B and C with SiLU and its state, step sizes and decays, the recurrence over each sequence's tokens in order,
the gate by silu(z) and the RMS norm in equal parts); then the output projection.

The state [heads, state_dim, head_dim] and the convolution inputs [taps - 1, channels] are fp32 rows of the cache's
state groups, zero when a sequence starts, advanced over all tokens that a sequence brings in a step, so a prompt,
its portions and single tokens go through the same kernels.  Everything between the two projections is fp32.
"""

from __future__ import annotations

import torch

from ..cache import StateNeed
from ..config.specs import StateSpaceSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import linear


class StateSpace(Part):
    graph_safe = True   # no host work that depends on the step's values
    returns_output = True   # forward(..., residual=None) returns the fp32 output instead of adding it

    def __init__(self, spec: StateSpaceSpec) -> None:
        super().__init__(spec)
        for key in ("num_heads", "head_dim", "state_dim", "groups", "conv_taps", "norm_groups"):
            if getattr(spec, key) <= 0:
                raise ValueError(f"{key} must be positive, got {getattr(spec, key)}")
        if spec.num_heads % spec.groups != 0:
            raise ValueError("heads must be divisible by groups")
        self.inner = spec.num_heads * spec.head_dim
        if self.inner % spec.norm_groups != 0:
            raise ValueError("the output norm's parts must divide heads * head_dim")
        if spec.state_dim > ops.SSD_MAX_STATE or spec.conv_taps > ops.SSD_MAX_TAPS:
            raise ValueError(f"the state-space kernels take states up to {ops.SSD_MAX_STATE} and up to {ops.SSD_MAX_TAPS} taps")
        self.channels = self.inner + 2 * spec.groups * spec.state_dim

    def tensor_decls(self):
        s = self.spec
        return [TensorDecl(s.name("in"), (self.inner + self.channels + s.num_heads, s.hidden_size)),
                TensorDecl(s.name("conv"), (self.channels, s.conv_taps)),
                TensorDecl(s.name("conv_bias"), (self.channels,)),
                TensorDecl(s.name("dt_bias"), (s.num_heads,)), TensorDecl(s.name("A_log"), (s.num_heads,)),
                TensorDecl(s.name("D"), (s.num_heads,), "one_plus_normal"),
                TensorDecl(s.name("norm"), (self.inner,), "one_plus_normal"),
                TensorDecl(s.name("o"), (s.hidden_size, self.inner))]

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        self.w_in = fetch.matrix(s.name("in"))
        self.conv_w = fetch.vector(s.name("conv"))
        self.conv_b = fetch.vector(s.name("conv_bias"))
        self.dt_bias = fetch.vector(s.name("dt_bias"))
        self.a_log = fetch.vector(s.name("A_log"))
        self.d_skip = fetch.vector(s.name("D"))
        self.out_norm = fetch.vector(s.name("norm"))
        self.w_o = fetch.matrix(s.name("o"))

    def cache_needs(self):
        s = self.spec
        needs = [StateNeed((s.num_heads, s.state_dim, s.head_dim), torch.float32, "state-space state")]
        if s.conv_taps > 1:
            needs.append(StateNeed((s.conv_taps - 1, self.channels), torch.float32, "state-space convolution inputs"))
        return tuple(needs)

    def forward(self, x, ctx, view, residual):
        """Adds the mixer's output to ``residual`` (fp32); with ``residual`` None returns it as a new fp32 tensor."""
        s = self.spec
        proj = linear(x, self.w_in)
        out = torch.empty((x.shape[0], self.inner), dtype=proj.dtype, device=proj.device)
        ops.ssd_mix(proj, self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.d_skip, self.out_norm,
                    view.states[1] if s.conv_taps > 1 else None, view.states[0], out, ctx.cu_q, ctx.tok_seq, ctx.slots,
                    n_seqs=ctx.n_seqs, heads=s.num_heads, head_dim=s.head_dim, state_dim=s.state_dim, groups=s.groups,
                    norm_groups=s.norm_groups, eps=s.norm_eps)
        if residual is None:
            return linear(out, self.w_o, out_dtype=torch.float32)
        linear(out, self.w_o, residual=residual, track=ctx)
        return None


register_part(StateSpaceSpec, StateSpace)

"""Dense gated feed-forward (ondeviceinfer/layers.py:86-113 of UESlubei/ondeviceinfer)."""

from __future__ import annotations

import torch

from ..config.specs import ClampedGatedMLPSpec, GatedMLPSpec, MLPSpec, PolyNormMLPSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import activated_linear, gated_linear, linear


class GatedMLP(Part):
    graph_safe = True   # no host work that depends on the step's values: may be captured in a CUDA graph
    takes_lazy_norm = True   # x may be a NormedRows: its first product makes the normed operand itself

    """down(silu(gate(x)) * up(x)).  The gate and up matrices are concatenated at load so
    that one matrix product yields both; the activation is taken in fp32 and rounded once."""

    def __init__(self, spec: GatedMLPSpec) -> None:
        super().__init__(spec)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not implemented (silu is)")

    def tensor_decls(self):
        s = self.spec
        return [TensorDecl(s.name("gate"), (s.intermediate_size, s.hidden_size)),
                TensorDecl(s.name("up"), (s.intermediate_size, s.hidden_size)),
                TensorDecl(s.name("down"), (s.hidden_size, s.intermediate_size))]

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        self.w_gate_up = torch.cat([fetch.matrix(s.name("gate")), fetch.matrix(s.name("up"))], 0)
        self.w_down = fetch.matrix(s.name("down"))

    def forward(self, x, ctx, residual) -> None:
        linear(gated_linear(x, self.w_gate_up), self.w_down, residual=residual, track=ctx)


class PlainMLP(Part):
    """down(act(up(x))) without a gate; the activation (the exact GELU or its tanh form) is taken in fp32 and
    rounded once (in the epilogue of the up product where the tensor-core kernels have it)."""

    graph_safe = True
    returns_output = True   # forward(..., residual=None) returns the fp32 output instead of adding it

    def __init__(self, spec: MLPSpec) -> None:
        super().__init__(spec)
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} is not implemented ({sorted(ops.ACTIVATIONS)} are)")

    def tensor_decls(self):
        s = self.spec
        return [TensorDecl(s.name("up"), (s.intermediate_size, s.hidden_size)),
                TensorDecl(s.name("down"), (s.hidden_size, s.intermediate_size))]

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        self.w_up = fetch.matrix(self.spec.name("up"))
        self.w_down = fetch.matrix(self.spec.name("down"))

    def forward(self, x, ctx, residual):
        """Adds to ``residual`` (fp32); with ``residual`` None returns the output as a new fp32 tensor."""
        act = activated_linear(x, self.w_up, self.spec.activation)
        if residual is None:
            return linear(act, self.w_down, out_dtype=torch.float32)
        linear(act, self.w_down, residual=residual, track=ctx)
        return None


class PolyNormMLP(Part):
    """down(act(up x + b_up)) + b_down with act(z) = a N(z) + b N(z^2) + c N(z^3) + e, N the division of a token's
    row of z by its root mean square.  The biases join their products' fp32 sums; the activation takes z in the
    compute dtype, works in fp32 and rounds once (``csrc/parallel.cu``)."""

    graph_safe = True
    returns_output = True   # forward(..., residual=None) returns the fp32 output instead of adding it

    def tensor_decls(self):
        s = self.spec
        return [TensorDecl(s.name("up"), (s.intermediate_size, s.hidden_size)),
                TensorDecl(s.name("up_bias"), (s.intermediate_size,)),
                TensorDecl(s.name("down"), (s.hidden_size, s.intermediate_size)),
                TensorDecl(s.name("down_bias"), (s.hidden_size,)),
                TensorDecl(s.name("act"), (4,), "one_plus_normal")]

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        self.w_up, self.b_up = fetch.matrix(s.name("up")), fetch.vector(s.name("up_bias"))
        self.w_down, self.b_down = fetch.matrix(s.name("down")), fetch.vector(s.name("down_bias"))
        self.coef = fetch.vector(s.name("act"))

    def forward(self, x, ctx, residual):
        """Adds to ``residual`` (fp32); with ``residual`` None returns the output as a new fp32 tensor."""
        z = linear(x, self.w_up, bias=self.b_up)
        act = torch.empty_like(z)
        ops.poly_norm(z, self.coef, self.spec.eps, act)
        if residual is None:
            return linear(act, self.w_down, bias=self.b_down, out_dtype=torch.float32)
        linear(act, self.w_down, bias=self.b_down, residual=residual)
        return None


class ClampedGatedMLP(Part):
    """down(g * sigmoid(alpha g) * (u + 1)) with g = min(gate x, limit), u = clamp(up x, -limit, limit), biases on the
    projections that the spec names one for.  Gate and up rows are concatenated at load: one product (the biases join
    its fp32 sums), then ``ops.gated_clamp`` (fp32 arithmetic, one rounding), then the down product."""

    graph_safe = True
    returns_output = True   # forward(..., residual=None) returns the fp32 output instead of adding it

    def __init__(self, spec: ClampedGatedMLPSpec) -> None:
        super().__init__(spec)
        if spec.limit <= 0:
            raise ValueError("limit must be positive")

    def tensor_decls(self):
        s = self.spec
        decls = [TensorDecl(s.name("gate"), (s.intermediate_size, s.hidden_size)),
                 TensorDecl(s.name("up"), (s.intermediate_size, s.hidden_size)),
                 TensorDecl(s.name("down"), (s.hidden_size, s.intermediate_size))]
        sizes = (("gate_bias", s.intermediate_size), ("up_bias", s.intermediate_size), ("down_bias", s.hidden_size))
        return decls + [TensorDecl(s.name(role), (size,)) for role, size in sizes if s.has(role)]

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        self.w_gate_up = torch.cat([fetch.matrix(s.name("gate")), fetch.matrix(s.name("up"))], 0)
        self.w_down = fetch.matrix(s.name("down"))
        self.b_gate_up = None
        if s.has("gate_bias") or s.has("up_bias"):       # a projection without a bias adds zero
            self.b_gate_up = torch.cat([fetch.vector(s.name(role)) if s.has(role)
                                        else torch.zeros(s.intermediate_size, dtype=torch.float32, device=runtime.device)
                                        for role in ("gate_bias", "up_bias")])
        self.b_down = fetch.vector(s.name("down_bias")) if s.has("down_bias") else None

    def forward(self, x, ctx, residual):
        """Adds to ``residual`` (fp32); with ``residual`` None returns the output as a new fp32 tensor."""
        s = self.spec
        act = torch.empty((x.shape[0], s.intermediate_size), dtype=x.dtype, device=x.device)
        ops.gated_clamp(linear(x, self.w_gate_up, bias=self.b_gate_up), act, s.limit, s.alpha)
        if residual is None:
            return linear(act, self.w_down, bias=self.b_down, out_dtype=torch.float32)
        linear(act, self.w_down, bias=self.b_down, residual=residual)
        return None


register_part(ClampedGatedMLPSpec, ClampedGatedMLP)
register_part(GatedMLPSpec, GatedMLP)
register_part(PolyNormMLPSpec, PolyNormMLP)
register_part(MLPSpec, PlainMLP)

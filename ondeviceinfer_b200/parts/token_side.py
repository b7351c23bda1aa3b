"""A per-layer input that is looked up by token id and added to the stream after a layer.

e = a layer's lanes of the token's row of a table that all layers share; g = gelu_tanh(gate x) * e; y = proj g;
x <- x + y / sqrt(mean(y^2) + eps) * weight.  Steps: the gate's product on the stream in the compute dtype (the block
hands over the copy that its own add made, or the part casts one), ``ops.gated_lookup`` (activation, lookup and
product in one kernel), the projection with fp32 output, and ``ops.rmsnorm_add`` (norm and add in one fp32 pass).
"""

from __future__ import annotations

import torch

from ..config.specs import TokenSideInputSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import linear


class TokenSideInput(Part):
    graph_safe = True
    wants_copy = True       # forward takes the stream once more in the compute dtype, if the caller has it

    def __init__(self, spec: TokenSideInputSpec) -> None:
        super().__init__(spec)
        if spec.dim <= 0 or spec.col < 0 or spec.col + spec.dim > spec.table_width:
            raise ValueError("the layer's lanes lie outside the table's rows")

    def tensor_decls(self):
        s = self.spec
        return [TensorDecl(s.table_name, (s.vocab_size, s.table_width)), TensorDecl(s.gate_name, (s.dim, s.hidden_size)),
                TensorDecl(s.proj_name, (s.hidden_size, s.dim)), TensorDecl(s.norm_name, (s.hidden_size,), "one_plus_normal")]

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        self.table = fetch.matrix(s.table_name)       # one tensor for all layers: the loader hands out one per name
        self.w_gate = fetch.matrix(s.gate_name)
        self.w_proj = fetch.matrix(s.proj_name)
        self.weight = fetch.vector(s.norm_name)

    def forward(self, hidden: torch.Tensor, ctx, copy=None) -> None:
        """``hidden`` is the fp32 stream, changed in place; ``copy`` the same rows in the compute dtype or None."""
        s = self.spec
        if copy is None:
            copy = torch.empty(hidden.shape, dtype=self.runtime.dtype, device=hidden.device)
            ops.cast_rows(hidden, copy)
        z = linear(copy, self.w_gate)
        g = torch.empty_like(z)
        ops.gated_lookup(z, self.table, ctx.token_ids, g, s.col)
        y = linear(g, self.w_proj, out_dtype=torch.float32)
        ops.rmsnorm_add(hidden, y, self.weight, s.eps)


register_part(TokenSideInputSpec, TokenSideInput)

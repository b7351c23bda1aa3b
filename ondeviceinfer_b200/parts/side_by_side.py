"""Two mixers on the same input, side by side: the result is left_scale * left + right_scale * right.

Each of the two is any registered mixer and keeps what it would keep alone: the part names the needs of the left one
and then those of the right one, and hands each a view of the layer's cache with its own share (at most one of the
two may keep keys and values; fixed-size states are told apart by their order).  Both outputs are taken in fp32 (a
part that says ``returns_output`` returns it, any other adds into a zeroed buffer) and summed by ``ops.weighted_sum``.
"""

from __future__ import annotations

import torch

from ..cache import CacheView, KVNeed, StateNeed
from ..config.specs import SideBySideMixersSpec
from ..kernels import ops
from .base import Part, build_part, register_part


class SideBySideMixers(Part):
    returns_output = True   # forward(..., residual=None) returns the fp32 output instead of adding it

    def __init__(self, spec: SideBySideMixersSpec) -> None:
        super().__init__(spec)
        self.left = build_part(spec.left)
        self.right = build_part(spec.right)
        needs = [tuple(self.left.cache_needs()), tuple(self.right.cache_needs())]
        if sum(any(isinstance(n, KVNeed) for n in side) for side in needs) > 1:
            raise ValueError("only one of two mixers side by side may keep keys and values")
        self.n_left_states = sum(isinstance(n, StateNeed) for n in needs[0])

    def tensor_decls(self):
        return list(self.left.tensor_decls()) + list(self.right.tensor_decls())

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        self.left.load(fetch, runtime)
        self.right.load(fetch, runtime)

    def cache_needs(self):
        return tuple(self.left.cache_needs()) + tuple(self.right.cache_needs())

    @property
    def graph_safe(self) -> bool:
        return getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False)

    @staticmethod
    def _share(view, states):
        return CacheView(kv_group=view.kv_group, keys=view.keys, values=view.values, writes_kv=view.writes_kv,
                         state=states[0] if states else None, states=tuple(states))

    @staticmethod
    def _output(part, x, ctx, view):
        if getattr(part, "returns_output", False):
            return part.forward(x, ctx, view, None)
        out = torch.zeros((x.shape[0], part.spec.hidden_size), dtype=torch.float32, device=x.device)
        part.forward(x, ctx, view, out)
        return out

    def forward(self, x, ctx, view, residual):
        """Adds the weighted sum to ``residual`` (fp32); with ``residual`` None returns it as a new fp32 tensor."""
        s = self.spec
        left = self._output(self.left, x, ctx, self._share(view, view.states[:self.n_left_states]))
        right = self._output(self.right, x, ctx, self._share(view, view.states[self.n_left_states:]))
        ctx.residual_sumsq = None
        ops.weighted_sum(left, left, right, s.left_scale, s.right_scale)
        if residual is None:
            return left
        ops.residual_add(residual, left)
        return None


register_part(SideBySideMixersSpec, SideBySideMixers)

"""RMSNorm part (ondeviceinfer/layers.py:9-33 of UESlubei/ondeviceinfer)."""

from __future__ import annotations

import torch

from ..config.specs import RMSNormSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import NormedRows


class RMSNorm(Part):
    graph_safe = True   # no host work that depends on the step's values: may be captured in a CUDA graph
    adds = True         # __call__ takes `add`: a pending residual add done in the norm's own pass

    """weight * cast(x * rsqrt(mean(x^2) + eps)): statistics in fp32, cast to the compute
    dtype before the multiplication by the weight.  With ``scale_in_fp32`` the row is scaled in fp32 and
    rounded once; ``weight_offset`` is added to the stored weight (in fp32, at load)."""

    def __init__(self, spec: RMSNormSpec) -> None:
        super().__init__(spec)
        if spec.scale_in_fp32:
            self.lazy = None      # the product prologue that norms rows itself rounds before it scales

    def tensor_decls(self):
        return [TensorDecl(self.spec.weight_name, () if self.spec.scalar_weight else (self.spec.size,),
                           "one_plus_normal" if self.spec.weight_offset == 0.0 else "normal")]

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        self.weight = fetch.vector(self.spec.weight_name)
        if self.spec.weight_offset != 0.0:
            self.weight = self.weight + self.spec.weight_offset
        if self.spec.scalar_weight:
            # one number for all coordinates: kept as it is for kernels that take it so, and laid out as a row
            # for the norm kernels that take a weight per coordinate
            self.scalar = self.weight.reshape(1).contiguous()
            self.weight = self.scalar.expand(self.spec.size).contiguous()

    def lazy(self, x: torch.Tensor, parts: torch.Tensor):
        """The norm of the whole of ``x`` as a :class:`~ondeviceinfer_b200.parts.linear.NormedRows`:
        ``parts`` [pieces, tokens] are sums of squares of pieces of each row, left by the product that
        wrote ``x``.  For a consumer that says ``takes_lazy_norm``."""
        return NormedRows(x, self.weight, self.spec.eps, parts, self.runtime.dtype)

    def __call__(self, x: torch.Tensor, rows=None, add=None, out_dtype=None) -> torch.Tensor:
        """``add`` (optional, without ``rows``): a product still to be added to ``x``; it is added in place in
        the same pass when the kernel can, else beforehand.  ``out_dtype`` (a norm with ``scale_in_fp32`` only):
        float32 keeps the result in 32 bits whatever the compute dtype."""
        n = x.shape[0] if rows is None else rows.numel()
        if out_dtype is not None and out_dtype != self.runtime.dtype and not self.spec.scale_in_fp32:
            raise ValueError("only a norm that scales in fp32 gives its result in another dtype")
        out = torch.empty((n, self.spec.size), dtype=out_dtype or self.runtime.dtype, device=x.device)
        if add is not None and (self.spec.scale_in_fp32 or
                                not (rows is None and ops.rmsnorm_adds(x, self.weight, out, add))):
            ops.residual_add(x, add)
            add = None
        if self.spec.scale_in_fp32:
            ops.rmsnorm_scaled(x, self.weight, self.spec.eps, out, rows)
        else:
            ops.rmsnorm(x, self.weight, self.spec.eps, out, rows, add=add)
        return out


register_part(RMSNormSpec, RMSNorm)

"""The two ends of a decoder as parts: the token embedding and the output head.

Like every part they are chosen by the type of their spec, so an architecture whose ends differ (a scaled
embedding, learned positions added to it, logits with a soft cap, several heads) brings a spec and a class
of its own and registers them; the model only calls ``embedding.forward(ctx)`` and
``head.forward(rows, ctx)``.

Reference: ``nn.Embedding`` lookup without scaling (ondeviceinfer/model.py:77-82,100) and a bias-free
``lm_head`` (ondeviceinfer/model.py:138-144,163), tied to the embedding table when the configuration says
so (ondeviceinfer/weights.py:77-78).
"""

from __future__ import annotations

import torch

from ..config.specs import EmbeddingSpec, HeadSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, build_part, register_part
from .linear import linear


class TokenEmbedding(Part):
    """hidden[t, :] = table[token[t], :], widened into the fp32 residual stream; with a norm in the spec the rows
    then pass it, in fp32 (a norm that scales in fp32).  With ``sinusoid_base`` in the spec the rows are multiplied
    by ``scale`` and get an absolute sinusoidal position vector in the same kernel: the frequencies
    base^(-2i / hidden) are computed here in double and rounded once, the angle position * frequency and its sine
    and cosine are fp32 on the device."""

    graph_safe = True

    def __init__(self, spec) -> None:
        super().__init__(spec)
        self.norm = build_part(spec.norm) if getattr(spec, "norm", None) is not None else None

    def tensor_decls(self):
        decls = [TensorDecl(self.spec.weight_name, (self.spec.vocab_size, self.spec.hidden_size))]
        return decls + (self.norm.tensor_decls() if self.norm is not None else [])

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        self.table = fetch.matrix(self.spec.weight_name)
        if self.norm is not None:
            self.norm.load(fetch, runtime)
        self.scale = float(getattr(self.spec, "scale", 1.0))
        base = getattr(self.spec, "sinusoid_base", None)
        self.inv_freq = None
        if base is not None:
            H = self.spec.hidden_size
            self.inv_freq = torch.tensor([float(base) ** (-2.0 * i / H) for i in range((H + 1) // 2)],
                                         dtype=torch.float64).to(torch.float32).to(runtime.device)
        elif self.scale != 1.0:
            raise ValueError("a scaled embedding without positions is not implemented")

    def forward(self, ctx) -> torch.Tensor:
        hidden = torch.empty((ctx.n_tokens, self.spec.hidden_size), dtype=torch.float32, device=self.runtime.device)
        if self.inv_freq is not None:
            ops.embed_sinusoid(self.table, ctx.token_ids, ctx.tok_pos, self.inv_freq, hidden, self.scale)
        else:
            ops.embed(self.table, ctx.token_ids, hidden)
        if self.norm is not None:
            return self.norm(hidden, out_dtype=torch.float32)
        return hidden


class OutputHead(Part):
    """logits = rows W^T in fp32, squashed by ``softcap`` if the spec has one.  A tied head binds the embedding's tensor (the loader hands out one tensor
    per name, so the table is held once) and declares nothing of its own."""

    graph_safe = True

    def tensor_decls(self):
        if self.spec.tied:
            return []
        return [TensorDecl(self.spec.weight_name, (self.spec.vocab_size, self.spec.hidden_size))]

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        self.weight = fetch.matrix(self.spec.weight_name)
        if tuple(self.weight.shape) != (self.spec.vocab_size, self.spec.hidden_size):
            raise ValueError(f"the head's weight {self.spec.weight_name!r} is {tuple(self.weight.shape)}, expected "
                             f"{(self.spec.vocab_size, self.spec.hidden_size)}")

    def forward(self, rows: torch.Tensor, ctx) -> torch.Tensor:
        """``rows`` [wanted, hidden] in the compute dtype (already normed) -> fp32 logits [wanted, vocab]."""
        logits = linear(rows, self.weight, out_dtype=torch.float32)
        if self.spec.softcap is not None:
            ops.softcap(logits, self.spec.softcap)        # c tanh(logits / c), in fp32
        return logits


register_part(EmbeddingSpec, TokenEmbedding)
register_part(HeadSpec, OutputHead)

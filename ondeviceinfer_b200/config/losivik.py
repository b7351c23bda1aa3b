"""Typed configuration of the Losivik decoder, read from its own ``config.json`` keys.

``config.json`` holds ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``token_side.dim`` and a list
``layers``; each entry has ``type`` (``latent_attention`` or ``parallel``), the mixer's sizes and constants under
``mixer`` and its feed-forward under ``mlp`` (null: none).

* ``latent_attention``: ``heads``, ``dim``, ``vdim``, ``kv_rank``, ``scale``, optionally ``mask.size``.  No rotated
  lanes: a head's key and value are up-projections of one normed latent row per position; a sigmoid gate with one
  number per head, computed from the mixer's input, multiplies the head's output.
* ``parallel``: two mixers on the same input, ``left_scale`` * left + ``right_scale`` * right.  ``left``: grouped
  attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``) with an RMS norm per query and key head whose
  weight the heads share, no rotation, and a window that keeps a sequence's first tokens (``mask.size``,
  ``mask.keep_first``).  ``right``: a state-space mixer (``heads``, ``vdim``, ``state``, ``groups``, ``conv``,
  ``norm_groups``).
* ``mlp.kind`` ``dense``: gated and clamped, with biases (``ff``, ``limit``).  ``moe``: ``router.experts`` ungated
  experts of ``expert.ff`` lanes with the squared ReLU, ``router.top`` chosen by the largest sigmoid scores, which
  multiply the experts' inputs; ``shared.ff``: one more expert that every token takes.

Every layer is x <- x + ls1 * mixer(norm1(x)) + ls2 * ff(norm2(x)) with RMS norms that multiply by one plus their
stored weight, followed by a per-layer input looked up by token id (``side.*``).  The embedding is scaled and gets sinusoidal
positions; the head is the embedding table.  A key that is absent switches its mechanism off.
Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1|norm2|ls1|ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``l<i>.side.gate|proj|norm``, ``final.norm``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .specs import (CappedAttentionSpec, ClampedGatedMLPSpec, EmbeddingSpec, HeadSpec, LatentAttentionSpec, ModelPlan,
                    NoPositionSpec, OrderEntry, RMSNormSpec, RoutedExpertsSpec, ScaledParallelBlockSpec,
                    SideBySideMixersSpec, StateSpaceSpec, TokenSideInputSpec, names)

MIXERS = ("latent_attention", "parallel")
FEED_FORWARDS = ("dense", "moe")
SINUSOID_BASE = 10000.0      # fixed by the design
GATE_ALPHA = 1.702           # fixed by the design: y = g sigmoid(1.702 g) (u + 1)


def _need(raw: Mapping[str, Any], key: str, where: str):
    if not isinstance(raw, Mapping) or key not in raw:
        raise KeyError(f"config.json: {where} lacks {key!r}")
    return raw[key]


@dataclass(frozen=True)
class LosivikConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]     # the entries of config.json["layers"], as read
    embedding_scale: float = 1.0
    side_dim: Optional[int] = None            # None: no per-layer token input

    architecture = "Losivik"

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LosivikConfig":
        layers = _need(raw, "layers", "the model")
        if not isinstance(layers, list) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        side = raw.get("token_side")
        config = cls(vocab_size=int(_need(raw, "vocab", "the model")), hidden_size=int(_need(raw, "width", "the model")),
                     norm_eps=float(_need(_need(raw, "norm", "the model"), "eps", "norm")),
                     layers=tuple(copy.deepcopy(layer) for layer in layers),
                     embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                     side_dim=None if side is None else int(_need(side, "dim", "token_side")))
        config.validate()
        return config

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
               "layers": [copy.deepcopy(dict(layer)) for layer in self.layers], "norm": {"eps": self.norm_eps},
               "vocab": self.vocab_size, "width": self.hidden_size}
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        return out

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or self.norm_eps <= 0:
            raise ValueError("vocab, width and norm.eps must be positive")
        if self.side_dim is not None and self.side_dim <= 0:
            raise ValueError("token_side.dim must be positive")
        for i, layer in enumerate(self.layers):
            if layer.get("type") not in MIXERS:
                raise ValueError(f"layers[{i}].type is {layer.get('type')!r}; known: {MIXERS}")
            f = layer.get("mlp")
            if f is not None and f.get("kind") not in FEED_FORWARDS:
                raise ValueError(f"layers[{i}].mlp.kind is {f.get('kind')!r}; known: {FEED_FORWARDS}")
            m = _need(layer, "mixer", f"layers[{i}]")
            if layer["type"] == "parallel":
                for side in ("left", "right"):
                    _need(m, side, f"layers[{i}].mixer")
                mask = m["left"].get("mask") or {}
                if mask.get("keep_first") and mask.get("size") is None:
                    raise ValueError(f"layers[{i}].mixer.left.mask.keep_first goes with mask.size")

    @property
    def stop_token_ids(self) -> tuple:
        return ()

    # ------------------------------------------------------------------ the plan

    def _norm(self, name: str) -> RMSNormSpec:
        return RMSNormSpec(self.hidden_size, self.norm_eps, name, weight_offset=1.0, scale_in_fp32=True)

    @staticmethod
    def _window(m: Mapping[str, Any]) -> Optional[int]:
        size = (m.get("mask") or {}).get("size")
        return None if size is None else int(size)

    def _latent(self, m: Mapping[str, Any], where: str, p: str) -> LatentAttentionSpec:
        return LatentAttentionSpec(
            hidden_size=self.hidden_size, num_heads=int(_need(m, "heads", where)), qk_dim=int(_need(m, "dim", where)),
            rot_dim=0, v_dim=int(_need(m, "vdim", where)), kv_rank=int(_need(m, "kv_rank", where)),
            scale=float(_need(m, "scale", where)), norm_eps=self.norm_eps, position=NoPositionSpec(), prefix=p,
            names=names(q="q", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", g="g", o="o"), window=self._window(m),
            gated=True, gate_per_head=True)

    def _left(self, m: Mapping[str, Any], where: str, p: str) -> CappedAttentionSpec:
        heads = int(_need(m, "heads", where))
        dim = int(_need(m, "dim", where))
        return CappedAttentionSpec(
            hidden_size=self.hidden_size, num_heads=heads, num_kv_heads=int(m.get("kv_heads", heads)), head_dim=dim,
            value_dim=int(m.get("vdim", dim)), scale=float(_need(m, "scale", where)), position=NoPositionSpec(), prefix=p,
            names=names(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm"), window=self._window(m),
            unit_norm_eps=self.norm_eps, keep_first=int((m.get("mask") or {}).get("keep_first") or 0))

    def _right(self, m: Mapping[str, Any], where: str, p: str) -> StateSpaceSpec:
        return StateSpaceSpec(
            hidden_size=self.hidden_size, num_heads=int(_need(m, "heads", where)), head_dim=int(_need(m, "vdim", where)),
            state_dim=int(_need(m, "state", where)), groups=int(m.get("groups", 1)), conv_taps=int(m.get("conv", 1)),
            norm_groups=int(m.get("norm_groups", 1)), norm_eps=self.norm_eps, prefix=p,
            names=names(**{"in": "in"}, conv="conv", conv_bias="conv.b", dt_bias="dt_bias", A_log="A_log", D="D",
                        norm="norm", o="o"))

    def _mixer(self, i: int, layer: Mapping[str, Any]):
        m, where, p = layer["mixer"], f"layers[{i}].mixer", f"l{i}.mix."
        if layer["type"] == "latent_attention":
            return self._latent(m, where, p)
        return SideBySideMixersSpec(left=self._left(m["left"], where + ".left", p + "left."),
                                    right=self._right(m["right"], where + ".right", p + "right."),
                                    left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0)))

    def _mlp(self, i: int, layer: Mapping[str, Any]):
        f = layer.get("mlp")
        if f is None:
            return None
        where, p = f"layers[{i}].mlp", f"l{i}.mlp."
        if f["kind"] == "dense":
            return ClampedGatedMLPSpec(
                self.hidden_size, int(_need(f, "ff", where)), float(_need(f, "limit", where)), p,
                names(gate="gate", up="up", down="down", gate_bias="gate.b", up_bias="up.b", down_bias="down.b"),
                alpha=GATE_ALPHA)
        router, expert = _need(f, "router", where), _need(f, "expert", where)
        shared = f.get("shared") or {}
        return RoutedExpertsSpec(
            hidden_size=self.hidden_size, expert_size=int(_need(expert, "ff", where + ".expert")),
            num_experts=int(_need(router, "experts", where + ".router")), num_identity=0,
            top_k=int(_need(router, "top", where + ".router")), num_groups=1, keep_groups=1, limit=0.0, prefix=p,
            has_correction=False, shared_size=int(shared.get("ff", 0)), scoring="sigmoid", expert_form="relu2",
            weight_on_input=True)

    def _side(self, i: int) -> Optional[TokenSideInputSpec]:
        if self.side_dim is None:
            return None
        return TokenSideInputSpec(
            hidden_size=self.hidden_size, vocab_size=self.vocab_size, dim=self.side_dim,
            table_width=self.side_dim * len(self.layers), col=i * self.side_dim, table_name="side.embed",
            gate_name=f"l{i}.side.gate", proj_name=f"l{i}.side.proj", norm_name=f"l{i}.side.norm", eps=self.norm_eps)

    def to_plan(self) -> ModelPlan:
        layers: List[ScaledParallelBlockSpec] = []
        ignored: List[str] = []
        for i, layer in enumerate(self.layers):
            mlp = self._mlp(i, layer)
            layers.append(ScaledParallelBlockSpec(
                mixer_norm=self._norm(f"l{i}.norm1"), mixer=self._mixer(i, layer),
                ffn_norm=self._norm(f"l{i}.norm2") if mlp is not None else None, ffn=mlp, hidden_size=self.hidden_size,
                mixer_scale_name=f"l{i}.ls1", ffn_scale_name=f"l{i}.ls2" if mlp is not None else None,
                after=self._side(i)))
            if mlp is None:       # a layer without a feed-forward may still store what belongs to one
                ignored += [f"l{i}.norm2", f"l{i}.ls2"]
        plan = ModelPlan(
            embedding=EmbeddingSpec(self.vocab_size, self.hidden_size, "embed", scale=self.embedding_scale,
                                    sinusoid_base=SINUSOID_BASE),
            layers=tuple(layers), order=tuple(OrderEntry(layer=i) for i in range(len(layers))),
            final_norm=self._norm("final.norm"), head=HeadSpec(self.vocab_size, self.hidden_size, None),
            ignored_tensors=tuple(ignored))
        plan.validate()
        return plan

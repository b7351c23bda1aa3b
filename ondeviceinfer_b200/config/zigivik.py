"""Typed configuration of the Zigivik decoder, read from its own ``config.json`` keys.

``config.json`` holds ``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``canon.taps`` and a list ``layers``;
each entry has ``type`` (``attention`` or ``latent_attention``), the mixer's sizes and constants under ``mixer`` and
its feed-forward under ``mlp`` (null: none; ``kind`` ``dense`` with ``ff``).

* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot.base|dims``, optionally ``mask.size``.
  Projections q and k with biases; the values are the keys before their rotation; neighbouring lanes rotate; the
  softmax has one more term of score zero.
* ``latent_attention``: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``q_rank``, ``scale``,
  ``rot.base|dims|scaling`` (``factor``, ``original``, ``fast``, ``slow``), ``mask.size``, and ``kv_from: j`` for a
  layer without a down projection that reads the rows layer j cached.  Half-split lanes rotate; ordinary softmax;
  a sigmoid gate on the heads.

Every layer is h = norm(x); x += residual_mult (mixer(h + conv(h)) + ff(h)) with a norm whose weight is one number
and a causal convolution of ``canon.taps`` taps per channel.  The embedding's rows pass a norm of that kind too.
A key that is absent switches its mechanism off (no window, no frequency scaling, no convolution, multiplier one).
Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.canon1``, ``l<i>.mix.q|k|o`` (+ ``.b``) or
``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o``, ``l<i>.mlp.up|down`` (+ ``.b``), ``l<i>.mlp.act``, ``final.norm``,
``head``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .specs import (CappedAttentionSpec, EmbeddingSpec, HeadSpec, LatentAttentionSpec, ModelPlan, NoPositionSpec,
                    OrderEntry, ParallelBlockSpec, PolyNormMLPSpec, RMSNormSpec, RotarySpec, names)

MIXERS = ("attention", "latent_attention")
FEED_FORWARDS = ("dense",)


def _need(raw: Mapping[str, Any], key: str, where: str):
    if not isinstance(raw, Mapping) or key not in raw:
        raise KeyError(f"config.json: {where} lacks {key!r}")
    return raw[key]


@dataclass(frozen=True)
class ZigivikConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]     # the entries of config.json["layers"], as read
    residual_mult: float = 1.0
    conv_taps: Optional[int] = None           # None: no convolution in front of the mixers

    architecture = "Zigivik"

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZigivikConfig":
        layers = _need(raw, "layers", "the model")
        if not isinstance(layers, list) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        canon = raw.get("canon")
        config = cls(vocab_size=int(_need(raw, "vocab", "the model")), hidden_size=int(_need(raw, "width", "the model")),
                     norm_eps=float(_need(_need(raw, "norm", "the model"), "eps", "norm")),
                     layers=tuple(copy.deepcopy(layer) for layer in layers),
                     residual_mult=float(raw.get("residual_mult", 1.0)),
                     conv_taps=None if canon is None else int(_need(canon, "taps", "canon")))
        config.validate()
        return config

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "layers": [copy.deepcopy(dict(layer)) for layer in self.layers],
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab_size,
               "width": self.hidden_size}
        if self.conv_taps is not None:
            out["canon"] = {"taps": self.conv_taps}
        return out

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or self.norm_eps <= 0:
            raise ValueError("vocab, width and norm.eps must be positive")
        if self.conv_taps is not None and self.conv_taps < 1:
            raise ValueError("canon.taps must be at least 1")
        for i, layer in enumerate(self.layers):
            if layer.get("type") not in MIXERS:
                raise ValueError(f"layers[{i}].type is {layer.get('type')!r}; known: {MIXERS}")
            f = layer.get("mlp")
            if f is not None and f.get("kind") not in FEED_FORWARDS:
                raise ValueError(f"layers[{i}].mlp.kind is {f.get('kind')!r}; known: {FEED_FORWARDS}")
            m = _need(layer, "mixer", f"layers[{i}]")
            source = m.get("kv_from")
            if source is not None:
                if layer["type"] != "latent_attention":
                    raise ValueError(f"layers[{i}]: only a latent_attention layer reads another layer's cache rows")
                if not (isinstance(source, int) and 0 <= source < i):
                    raise ValueError(f"layers[{i}].mixer.kv_from names layer {source!r}, which is not an earlier layer")
                other = self.layers[source]
                if other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layers[{i}].mixer.kv_from names layer {source}, which caches no rows of its own")
                for key in ("kv_rank", "rot_dim"):
                    if int(other["mixer"].get(key, -1)) != int(m.get(key, -2)):
                        raise ValueError(f"layers[{i}] reads the cache rows of layer {source}, whose {key} differs")
                if other["mixer"].get("rot") != m.get("rot"):
                    raise ValueError(f"layers[{i}] reads the cache rows of layer {source}, whose rotation differs")
            if layer["type"] == "attention" and int(m.get("vdim", m.get("dim", 0))) != int(m.get("dim", 0)):
                raise ValueError(f"layers[{i}]: the values of an attention layer are its keys, so vdim equals dim")

    @property
    def stop_token_ids(self) -> tuple:
        return ()

    # ------------------------------------------------------------------ the plan

    def _norm(self, name: str) -> RMSNormSpec:
        return RMSNormSpec(self.hidden_size, self.norm_eps, name, scale_in_fp32=True, scalar_weight=True)

    @staticmethod
    def _window(m: Mapping[str, Any]) -> Optional[int]:
        size = (m.get("mask") or {}).get("size")
        return None if size is None else int(size)

    def _kept(self, i: int) -> Tuple[Optional[int], bool]:
        """(positions, everything) that the cache rows of latent layer i's store are kept for: the widest window
        among the layer that writes them and the layers that read them; everything if one of them has none."""
        owner = self.layers[i]["mixer"].get("kv_from", i)
        if owner is None:
            owner = i
        windows = [self._window(layer["mixer"]) for j, layer in enumerate(self.layers)
                   if layer["type"] == "latent_attention" and (j == owner or layer["mixer"].get("kv_from") == owner)]
        if any(w is None for w in windows):
            return None, True
        return max(windows), False

    def _mixer(self, i: int, layer: Mapping[str, Any]):
        m, where, p = layer["mixer"], f"layers[{i}].mixer", f"l{i}.mix."
        rot = m.get("rot")
        heads = int(_need(m, "heads", where))
        if layer["type"] == "attention":
            head_dim = int(_need(m, "dim", where))
            position = NoPositionSpec()
            if rot is not None:
                position = RotarySpec(head_dim=head_dim, theta=float(_need(rot, "base", where + ".rot")),
                                      rotary_dim=int(_need(rot, "dims", where + ".rot")), interleaved=True)
            return CappedAttentionSpec(
                hidden_size=self.hidden_size, num_heads=heads, num_kv_heads=int(m.get("kv_heads", heads)),
                head_dim=head_dim, value_dim=head_dim, scale=float(_need(m, "scale", where)), position=position, prefix=p,
                names=names(q="q", k="k", o="o", q_bias="q.b", k_bias="k.b"), window=self._window(m), sink=True,
                values_are_keys=True)
        rot_dim = int(_need(m, "rot_dim", where))
        position = NoPositionSpec()
        if rot is not None and rot_dim > 0:
            ramp = rot.get("scaling")
            if ramp is not None:
                ramp = tuple(float(_need(ramp, key, where + ".rot.scaling")) for key in ("factor", "original", "fast", "slow"))
            position = RotarySpec(head_dim=rot_dim, theta=float(_need(rot, "base", where + ".rot")),
                                  rotary_dim=int(_need(rot, "dims", where + ".rot")), interleaved=False, index_ramp=ramp)
        q_rank = m.get("q_rank")
        own = m.get("kv_from") is None
        keep, everything = self._kept(i)
        roles = dict(uk="uk", uv="uv", o="o", g="g")
        roles.update(dict(q="q") if q_rank is None else dict(dq="dq", dq_norm="dq.norm", uq="uq"))
        if own:
            roles.update(dkv="dkv", dkv_norm="dkv.norm")
        return LatentAttentionSpec(
            hidden_size=self.hidden_size, num_heads=heads, qk_dim=int(_need(m, "dim", where)), rot_dim=rot_dim,
            v_dim=int(_need(m, "vdim", where)), kv_rank=int(_need(m, "kv_rank", where)),
            scale=float(_need(m, "scale", where)), norm_eps=self.norm_eps, position=position, prefix=p,
            names=names(**roles), q_rank=None if q_rank is None else int(q_rank), window=self._window(m), keep=keep,
            keeps_all=everything, gated=True, own_kv=own)

    def _mlp(self, i: int, layer: Mapping[str, Any]) -> Optional[PolyNormMLPSpec]:
        f = layer.get("mlp")
        if f is None:
            return None
        return PolyNormMLPSpec(self.hidden_size, int(_need(f, "ff", f"layers[{i}].mlp")), self.norm_eps, f"l{i}.mlp.",
                               names(up="up", up_bias="up.b", down="down", down_bias="down.b", act="act"))

    def to_plan(self) -> ModelPlan:
        layers: List[ParallelBlockSpec] = []
        order: List[OrderEntry] = []
        for i, layer in enumerate(self.layers):
            layers.append(ParallelBlockSpec(
                norm=self._norm(f"l{i}.norm1"), mixer=self._mixer(i, layer), ffn=self._mlp(i, layer),
                hidden_size=self.hidden_size, residual_mult=self.residual_mult,
                conv_taps=1 if self.conv_taps is None else self.conv_taps,
                conv_name=None if self.conv_taps is None else f"l{i}.canon1"))
            # layer i is order entry i: a layer that reads layer j's cache rows reads those of entry j
            order.append(OrderEntry(layer=i, cache_from=layer["mixer"].get("kv_from")))
        plan = ModelPlan(embedding=EmbeddingSpec(self.vocab_size, self.hidden_size, "embed", norm=self._norm("embed.norm")),
                         layers=tuple(layers), order=tuple(order), final_norm=self._norm("final.norm"),
                         head=HeadSpec(self.vocab_size, self.hidden_size, "head"))
        plan.validate()
        return plan

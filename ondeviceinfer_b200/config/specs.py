"""Architecture-neutral descriptions of a decoder: what each layer is made of and in which order layers run.

A model is data before it is code.  An architecture's configuration class turns its
``config.json`` into a :class:`ModelPlan`; the engine builds parts from the plan through
the part registries (``ondeviceinfer_b200.parts``).  Nothing in a spec names a model:
every size and constant is a field, and the checkpoint tensor names a part binds are
given to it by the plan (``names`` / ``prefix``), not known by the part.

Specs are frozen dataclasses.  A new kind of part brings its own spec class; the
registries key on the spec's *type*, so nothing here has to change for it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


def _frozen_names(names: Mapping[str, str]) -> Tuple[Tuple[str, str], ...]:
    return tuple(sorted(names.items()))


@dataclass(frozen=True)
class RMSNormSpec:
    """y = weight * cast(x * rsqrt(mean(x^2) + eps)); statistics in fp32.

    ``weight_offset``: the row is scaled by ``weight_offset + weight`` (1.0 for a weight that is stored as its
    deviation from one).  ``scale_in_fp32``: the scaling is done in fp32 before the one rounding to the compute
    dtype, y = cast(x * rsqrt(mean(x^2) + eps) * (weight_offset + weight)).  ``scalar_weight``: the stored weight
    is a single number (a tensor without dimensions) that scales every coordinate."""

    size: int
    eps: float
    weight_name: str  # full checkpoint name of the [size] weight
    weight_offset: float = 0.0
    scale_in_fp32: bool = False
    scalar_weight: bool = False


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding over the first ``rotary_dim`` lanes of a head: lane i turns with lane
    i + rotary_dim / 2 (half-split), or, with ``interleaved``, lane 2i with lane 2i + 1; the angle of pair i at
    position p is p * f_i, f_i = theta^(-2i / rotary_dim).  ``scaling`` = (factor, low, high, original) slows the
    long wavelengths: with l = 2 pi / f_i, f_i stays where l < original / high, becomes f_i / factor where
    l > original / low, and in between is (1 - s) f_i / factor + s f_i with s = (original / l - low) / (high - low).
    ``index_ramp`` = (factor, original, fast, slow) is another way to slow them, by a ramp over the pair index: with
    n(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta) the index of the pair that makes t turns over
    ``original`` positions, lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), rotary_dim - 1) and
    s_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is s_i f_i / factor + (1 - s_i) f_i, and cos and
    sin are both multiplied by 0.1 ln(factor) + 1."""

    head_dim: int
    theta: float
    rotary_dim: Optional[int] = None  # None: the whole head
    interleaved: bool = False
    scaling: Optional[Tuple[float, float, float, float]] = None
    index_ramp: Optional[Tuple[float, float, float, float]] = None

    @property
    def dim(self) -> int:
        return self.head_dim if self.rotary_dim is None else self.rotary_dim


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding inside the mixer."""


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query causal self-attention over cached keys and values.

    ``qk_norm_eps`` not None adds an RMSNorm over each query and key head (one [head_dim]
    weight shared by the heads) before the position encoding.  ``window`` not None keeps
    only the last ``window`` keys visible (the query's own position included).
    ``names`` maps the roles q, k, v, o, q_norm, k_norm to tensor names below ``prefix``; when it also
    names q_bias, k_bias, v_bias or o_bias, that projection adds the [out] bias of that name.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: object  # RotarySpec | NoPositionSpec | any registered position spec
    prefix: str
    names: Tuple[Tuple[str, str], ...]
    qk_norm_eps: Optional[float] = None
    window: Optional[int] = None
    scale: Optional[float] = None  # None: 1/sqrt(head_dim)

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]

    def has(self, role: str) -> bool:
        return role in dict(self.names)


@dataclass(frozen=True)
class CappedAttentionSpec:
    """Grouped-query causal attention whose queries and keys are rotated first and then scaled to unit root mean
    square, with a value width of its own, squashed scores and an optional window.

    q and k heads have ``head_dim`` lanes, v heads ``value_dim``.  ``position`` rotates q and k; afterwards, with
    ``unit_norm_eps`` not None, every q and k head is divided by sqrt(mean of its squares + eps) (no weight).
    score = q . k * ``scale``; with ``softcap`` c not None, score <- c tanh(score / c); ordinary softmax over the
    visible keys: all of 0..p, or with ``window`` w the last w of them (p itself included).  All of this in fp32.
    ``sink``: the softmax has one more term, of score 0 and without a value: p_j = exp(s_j) / (1 + sum_k exp(s_k)).
    ``values_are_keys``: there is no value projection; a head's value is its key as projected, before the rotation
    (``value_dim`` == ``head_dim``).
    ``keep_first`` k > 0 (with a window): keys 0..k-1 of a sequence stay visible beyond the window, at their true
    positions: position p sees j <= p with p - j < w or j < k.
    ``names`` maps the roles q, k, v, o to tensor names below ``prefix``; when it also names q_bias or k_bias, that
    projection adds the [out] bias of that name; when it names q_norm and k_norm (with ``unit_norm_eps``), every
    query resp. key head is multiplied, after the division, by that [head_dim] weight, which the heads share (an RMS
    norm per head with a plain weight)."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    position: object
    prefix: str
    names: Tuple[Tuple[str, str], ...]
    softcap: Optional[float] = None
    window: Optional[int] = None
    unit_norm_eps: Optional[float] = None
    sink: bool = False
    values_are_keys: bool = False
    keep_first: int = 0

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]

    def has(self, role: str) -> bool:
        return role in dict(self.names)


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are up-projections of one cached latent row per position.

    Per position the cache holds the latent c (``kv_rank`` lanes: the first rows of the down projection, RMS-normed
    with a plain weight and ``norm_eps``) and ``rot_dim`` rotated key lanes shared by all heads (the last rows of
    the down projection).  A head's query is ``qk_dim`` plain lanes followed by ``rot_dim`` rotated lanes; its key
    is ``W_uk c`` followed by the shared rotated lanes; its value ``W_uv c`` (``v_dim`` lanes); the score is the
    dot product times ``scale``; ordinary softmax over positions 0..p, or with ``window`` w over the last w of them
    (p itself included).  ``position`` rotates the ``rot_dim`` lanes.
    ``q_rank`` not None: the queries go through a latent of their own, q = W_uq RMSnorm(W_dq h) (plain weight,
    ``norm_eps``; roles dq, dq_norm, uq instead of q).  ``gated``: the concatenated heads are multiplied by
    sigmoid(W_g h) before the output projection (role g: one row of W_g per lane of the heads, or with
    ``gate_per_head`` one row per head, whose number multiplies all of the head's lanes).  ``own_kv`` False: the layer has no down projection and
    reads the cache rows that another layer execution wrote (the plan's order says which), with its own
    up-projections, queries and window; ``keep`` is then the window that the shared rows are kept for (None: all
    of them), at least the window of every layer that reads them.
    ``names`` maps the roles q, dkv, dkv_norm, uk, uv, o to tensor names below ``prefix``."""

    hidden_size: int
    num_heads: int
    qk_dim: int
    rot_dim: int
    v_dim: int
    kv_rank: int
    scale: float
    norm_eps: float
    position: object
    prefix: str
    names: Tuple[Tuple[str, str], ...]
    q_rank: Optional[int] = None
    window: Optional[int] = None
    keep: Optional[int] = None      # positions the cache keeps; None with a window: the window itself
    keeps_all: bool = False         # the cache keeps every position although this layer has a window (a reader has none)
    gated: bool = False
    own_kv: bool = True
    gate_per_head: bool = False

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]

    @property
    def cache_window(self) -> Optional[int]:
        """How many positions the cache rows are kept for (None: all)."""
        if self.keeps_all or self.window is None:
            return None
        return self.window if self.keep is None else max(self.keep, self.window)


@dataclass(frozen=True)
class ChannelDeltaSpec:
    """Gated delta rule with one decay per head and key channel (a recurrent mixer with a matrix state per head).

    q and k have ``num_kv_heads`` heads of ``qk_dim`` lanes, v has ``num_heads`` heads of ``v_dim``; head h reads
    q/k head h // (num_heads / num_kv_heads).  Each of q, k, v passes a causal convolution of ``conv_taps`` taps
    per channel and SiLU; q and k become unit vectors (``unit_eps`` inside the root), q times qk_dim^-1/2.
    Per token: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with beta = sigmoid(b x) and
    g = exp(-exp(A_log) softplus(a2 a1 x + dt_bias)).  o is RMS-normed per head (``norm_eps``, one plain weight of
    ``v_dim`` lanes), gated by sigmoid(g2 g1 x), and projected by o.  ``names`` maps the roles q, k, v, q_conv,
    k_conv, v_conv, b, A_log, dt_bias, a1, a2, g1, g2, norm, o to tensor names below ``prefix``."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    qk_dim: int
    v_dim: int
    conv_taps: int
    decay_rank: int
    gate_rank: int
    norm_eps: float
    prefix: str
    names: Tuple[Tuple[str, str], ...]
    unit_eps: float = 1e-6

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """Mixture of experts with a grouped top-k router, identity outputs and an optional shared expert.

    The router has ``num_experts + num_identity`` outputs; scores are the softmax over all of them (fp32); the
    choice adds ``correction`` (a stored vector, if ``has_correction``) to the scores; the outputs form
    ``num_groups`` equal groups of neighbours of which the ``keep_groups`` with the largest member may be chosen
    from; the ``top_k`` best are chosen and weighted by their scores (not renormalised).  The last
    ``num_identity`` outputs pass the input on; the others are experts
    down(g * sigmoid(``gate_alpha`` g) * (u + 1)), g = min(gate x, ``limit``), u = clamp(up x, +-``limit``).
    ``shared_size`` > 0 adds one expert of that form (its own ``shared_limit``) for every token.
    ``scoring`` "sigmoid": the score of an output is the logistic function of its logit instead of the softmax.
    ``expert_form`` "relu2": an expert (and the shared one) is down(max(up x, 0)^2), without gate, limit or bias.
    ``weight_on_input``: a chosen expert's weight multiplies its input, out = sum_k expert_k(w_k x), not its output.
    Tensor names below ``prefix``: ``router``, ``correction``, ``e<i>.gate|up|down``, ``shared.gate|up|down``
    (no ``gate`` tensors for ungated experts)."""

    hidden_size: int
    expert_size: int
    num_experts: int
    num_identity: int
    top_k: int
    num_groups: int
    keep_groups: int
    limit: float
    prefix: str
    has_correction: bool = True
    shared_size: int = 0
    shared_limit: float = 0.0
    gate_alpha: float = 1.702
    scoring: str = "softmax"
    expert_form: str = "gated_clamp"
    weight_on_input: bool = False


@dataclass(frozen=True)
class TableExpertsSpec:
    """Mixture of experts without a router: row ``token id`` of an integer table ([``vocab_size``, ``top_k``],
    distinct entries) names the experts of a token, each weighted 1 / top_k.  An expert is down(act(up x)) without
    biases, ``activation`` "gelu_erf" or "gelu_tanh".  ``shared_size`` > 0 adds one expert of that form for every
    token, multiplied (``shared_gated``) by sigmoid(sg . x), one number per token.
    Tensor names below ``prefix``: ``table``, ``e<i>.up|down``, ``shared.up|down|sg``."""

    hidden_size: int
    expert_size: int
    num_experts: int
    top_k: int
    vocab_size: int
    prefix: str
    activation: str = "gelu_erf"
    shared_size: int = 0
    shared_gated: bool = True


@dataclass(frozen=True)
class MLPSpec:
    """Dense feed-forward without a gate: down(act(up(x))), no biases; ``activation`` "gelu_erf" or "gelu_tanh"."""

    hidden_size: int
    intermediate_size: int
    activation: str
    prefix: str
    names: Tuple[Tuple[str, str], ...]

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]


@dataclass(frozen=True)
class PolyNormMLPSpec:
    """Dense feed-forward down(act(up x + b_up)) + b_down whose activation is a polynomial of row-normed powers:
    act(z) = a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N(v) = v / sqrt(mean(v^2) + ``eps``) over a
    token's ``intermediate_size`` values, (a, b, c, e) a stored tensor of four numbers.
    ``names`` maps the roles up, up_bias, down, down_bias, act to tensor names below ``prefix``."""

    hidden_size: int
    intermediate_size: int
    eps: float
    prefix: str
    names: Tuple[Tuple[str, str], ...]

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]


@dataclass(frozen=True)
class ClampedGatedMLPSpec:
    """Dense gated feed-forward with clamped halves: g = min(gate x, ``limit``), u = clamp(up x, -limit, limit),
    y = g * sigmoid(``alpha`` g) * (u + 1), output down y.  ``names`` maps the roles gate, up, down to tensor names
    below ``prefix``; when it also names gate_bias, up_bias or down_bias, that projection adds the bias."""

    hidden_size: int
    intermediate_size: int
    limit: float
    prefix: str
    names: Tuple[Tuple[str, str], ...]
    alpha: float = 1.702

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]

    def has(self, role: str) -> bool:
        return role in dict(self.names)


@dataclass(frozen=True)
class StateSpaceSpec:
    """A selective state-space mixer with one scalar decay per head (the recurrent form of the state-space duality).

    inner = ``num_heads`` * ``head_dim``.  One projection of the input gives [z: inner | x: inner | B: G N | C: G N |
    dt: heads] (G = ``groups``, N = ``state_dim``).  x, B and C together pass a causal convolution per channel
    (``conv_taps`` taps, the last one the current token's, zeros before the start, a bias) and SiLU.
    dt = softplus(dt + dt_bias).  Per head h (group h // (heads / G)), with S [N, head_dim] zero at the start:
    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T;  y_t = S_t^T C_t + D_h x_t.  y (heads side by side) is
    multiplied by silu(z), RMS-normed in ``norm_groups`` equal parts (``norm_eps`` inside each root), multiplied by a
    weight per lane, and projected by o.  The state and the convolution's last taps - 1 inputs are fp32 and are
    carried from token to token per sequence.  ``names`` maps the roles in, conv, conv_bias, dt_bias, A_log, D, norm,
    o to tensor names below ``prefix``."""

    hidden_size: int
    num_heads: int
    head_dim: int
    state_dim: int
    groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    prefix: str
    names: Tuple[Tuple[str, str], ...]

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]


@dataclass(frozen=True)
class SideBySideMixersSpec:
    """Two mixers that read the same input; the result is ``left_scale`` * left + ``right_scale`` * right.  Each
    keeps the cache or state that it would keep alone (at most one of them keys and values)."""

    left: object
    right: object
    left_scale: float = 1.0
    right_scale: float = 1.0


@dataclass(frozen=True)
class TokenSideInputSpec:
    """A per-layer input looked up by token id, added to the stream after a layer: e = lanes [``col``, ``col`` +
    ``dim``) of row ``token id`` of ``table_name`` [``vocab_size``, ``table_width``]; g = gelu_tanh(gate x) * e with
    gate [dim, hidden]; y = proj g with proj [hidden, dim]; x <- x + y / sqrt(mean(y^2) + ``eps``) * norm (a plain
    weight).  The norm and the add are fp32."""

    hidden_size: int
    vocab_size: int
    dim: int
    table_width: int
    col: int
    table_name: str
    gate_name: str
    proj_name: str
    norm_name: str
    eps: float


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x)), no biases."""

    hidden_size: int
    intermediate_size: int
    activation: str  # "silu"
    prefix: str
    names: Tuple[Tuple[str, str], ...]

    def name(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]


@dataclass(frozen=True)
class PreNormBlockSpec:
    """h += mixer(norm1(h)); h += feed_forward(norm2(h))."""

    mixer_norm: object
    mixer: object
    ffn_norm: object    # None together with ffn: the layer has no feed-forward
    ffn: object


@dataclass(frozen=True)
class SandwichBlockSpec:
    """h += mixer_post_norm(mixer(mixer_norm(h))); h += ffn_post_norm(feed_forward(ffn_norm(h))): a norm on both
    sides of every sublayer.  The post norms work on the fp32 output of the sublayer and add in fp32."""

    mixer_norm: object
    mixer: object
    mixer_post_norm: object
    ffn_norm: object    # the three of the feed-forward are None together: the layer has none
    ffn: object
    ffn_post_norm: object


@dataclass(frozen=True)
class ParallelBlockSpec:
    """h = norm(x); x <- x + ``residual_mult`` * (mixer(h + conv(h)) + feed_forward(h)): one norm, both sublayers read
    its output side by side.  conv is a causal convolution over time on each channel of h, ``conv_taps`` taps without
    a bias (``conv_name``: [hidden, taps]), conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j), zeros before a sequence's
    start; the last taps - 1 rows of h are part of a sequence's state.  ``conv_name`` None: the mixer reads h itself.
    ``ffn`` None: the layer has no feed-forward.  The norm, the convolution's sum and the residual sum are fp32."""

    norm: object
    mixer: object
    ffn: object
    hidden_size: int
    residual_mult: float = 1.0
    conv_taps: int = 1
    conv_name: Optional[str] = None


@dataclass(frozen=True)
class ScaledParallelBlockSpec:
    """x <- x + s1 * mixer(norm1(x)) + s2 * feed_forward(norm2(x)): both sublayers read the same x through a norm of
    their own, and each output is multiplied lane by lane by a stored vector (``mixer_scale_name``,
    ``ffn_scale_name``: [hidden]) before the sum.  ``ffn`` None (with its norm and scale): the layer has no
    feed-forward.  ``after`` (a spec of a part with ``forward(hidden, ctx, copy)``, or None) then adds to the new
    stream.  Norms, scales and sums are fp32."""

    mixer_norm: object
    mixer: object
    ffn_norm: object
    ffn: object
    hidden_size: int
    mixer_scale_name: str
    ffn_scale_name: Optional[str] = None
    after: object = None


@dataclass(frozen=True)
class ReinjectSpec:
    """A step between layers that keeps no cache: h <- W [h ; e] + steps[index], with e the output of the
    embedding, W [hidden, 2 hidden] (the columns of h first) and ``steps`` [``num_steps``, hidden].  It opens a
    pass of a looped stack; the passes share W and differ in ``index``."""

    hidden_size: int
    weight_name: str
    steps_name: str
    num_steps: int
    index: int


@dataclass(frozen=True)
class OrderEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelPlan.layers``; the same layer may appear in several
    entries (its weights are then shared, each execution has a cache of its own).
    ``cache_from`` not None makes this execution read the cache that the earlier order
    entry with that index wrote, instead of writing one itself.
    """

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    """Token embedding: hidden[t] = table[token[t]] * ``scale``; with ``sinusoid_base`` b an absolute position
    vector is added, entry 2i = sin(p b^(-2i / hidden_size)), entry 2i + 1 = the cosine of the same angle, p the
    token's position in its sequence (fp32); with ``norm`` (a norm spec) the rows then pass that norm, in fp32."""

    vocab_size: int
    hidden_size: int
    weight_name: str
    norm: object = None
    scale: float = 1.0
    sinusoid_base: Optional[float] = None


@dataclass(frozen=True)
class HeadSpec:
    """Output head: logits = rows W^T on the rows the final norm gives it.  ``weight_name`` None ties it to the
    embedding table (the model then fills in that tensor's name and sets ``tied``); with ``tied`` the head
    binds ``weight_name`` without declaring it, because another part already does.  ``softcap`` squashes the logits."""

    vocab_size: int
    hidden_size: int
    weight_name: Optional[str]
    tied: bool = False
    softcap: Optional[float] = None     # c: logits <- c tanh(logits / c)


@dataclass(frozen=True)
class ModelPlan:
    """``embedding`` and ``head`` are specs of registered parts like the layers' (any spec whose part has
    ``forward(ctx) -> hidden`` resp. ``forward(rows, ctx) -> logits`` and the sizes ``vocab_size`` /
    ``hidden_size``); :class:`EmbeddingSpec` and :class:`HeadSpec` are the plain ones."""

    embedding: object
    layers: Tuple[object, ...]
    order: Tuple[OrderEntry, ...]
    final_norm: object
    head: object
    # tensors that may be present in a checkpoint and are deliberately not used
    ignored_tensors: Tuple[str, ...] = field(default_factory=tuple)

    def validate(self) -> None:
        for i, entry in enumerate(self.order):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {entry.layer}, the plan has {len(self.layers)}")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < i:
                    raise ValueError(f"order[{i}] reads the cache of entry {entry.cache_from}, "
                                     "which must be an earlier entry")
                if self.order[entry.cache_from].cache_from is not None:
                    raise ValueError(f"order[{i}] reads the cache of entry {entry.cache_from}, "
                                     "which owns no cache itself")


def names(**roles: str) -> Tuple[Tuple[str, str], ...]:
    """Helper for plans: ``names(q="q_proj.weight", ...)``."""
    return _frozen_names(roles)

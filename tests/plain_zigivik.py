"""A plain, slow restatement of the Zigivik decoder for tests: one function per mechanism, whole sequences at
a time, float64 on the CPU, no cache, no batching.  It shares no code with the library.

A model is ``(config, tensors)``: the ``config.json`` dictionary and a dictionary name -> tensor.

Notation.  T tokens, D = width.  x0 = n_e(embed[ids]); layer: h = n(x), x <- x + m (mix(h + conv(h)) + ff(h));
logits = head n_f(x).  n(.) divides a row by sqrt(mean of squares + eps) and multiplies by ONE number.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------ small mechanisms


def rms(x, eps):
    """Rows of x divided by sqrt(mean of squares + eps)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is a single number for all coordinates."""
    return rms(x, eps) * g.reshape(())


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(h, w):
    """h [T, D], w [D, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    T, D = h.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, D, dtype=h.dtype), h], 0)
    out = torch.zeros_like(h)
    for j in range(taps):
        out += padded[j:j + T] * w[:, j][None, :]
    return out


def poly_norm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e with N = division of the row by its root mean square."""
    a, b, c, e = (coef[i] for i in range(4))
    return a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e


def dense_ff(h, w, p, eps):
    z = h @ w[p + "up"].T + w[p + "up.b"]
    return poly_norm(z, w[p + "act"], eps) @ w[p + "down"].T + w[p + "down.b"]


def plain_frequencies(dims, base):
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def yarn_frequencies(dims, base, s):
    """Frequencies blended between f_i and f_i / factor by a ramp over the pair index, and the number both cos
    and sin are multiplied by."""
    factor, original, fast, slow = (float(s[k]) for k in ("factor", "original", "fast", "slow"))

    def index_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(dims, base)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, magnitude, interleaved):
    """x [T, heads, lanes]: the first 2 len(freqs) lanes turn; pairs are (2i, 2i+1) or (i, i + len(freqs))."""
    n = len(freqs)
    angle = positions.to(F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]
    cos, sin = (torch.cos(angle) * magnitude)[:, None, :], (torch.sin(angle) * magnitude)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2] = u * cos - v * sin
        out[..., 1:2 * n:2] = v * cos + u * sin
    else:
        u, v = x[..., 0:n], x[..., n:2 * n]
        out[..., 0:n] = u * cos - v * sin
        out[..., n:2 * n] = v * cos + u * sin
    return out


def rotation_of(rot):
    """(frequencies, magnitude) of a layer's ``rot`` dictionary."""
    if rot.get("scaling"):
        return yarn_frequencies(int(rot["dims"]), float(rot["base"]), rot["scaling"])
    return plain_frequencies(int(rot["dims"]), float(rot["base"])), 1.0


def visible(T, window):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok &= (i - j) < window
    return ok


# ------------------------------------------------------------------------------ mixers


def sink_attention(h, w, p, m, positions):
    """Grouped-query attention whose values are the unrotated keys and whose softmax has one more term of
    score zero and no value."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = k
    freqs, magnitude = rotation_of(m["rot"])
    q, kr = rotate(q, positions, freqs, magnitude, True), rotate(k, positions, freqs, magnitude, True)
    window = (m.get("mask") or {}).get("size")
    see = visible(T, window)
    out = torch.zeros(T, H, d, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ kr[:, g].T) * float(m["scale"])
        s = s.masked_fill(~see, -math.inf)
        top = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - top)
        out[:, head] = (e / (torch.exp(-top) + e.sum(-1, keepdim=True))) @ v[:, g]
    return out.reshape(T, H * d) @ w[p + "o"].T


def latent_rows(h, w, p, m, eps, positions):
    """What a latent layer caches: the normed latent [T, kv_rank] and the rotated shared key lanes [T, rot_dim]."""
    R = int(m["kv_rank"])
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :R], eps) * w[p + "dkv.norm"]
    freqs, magnitude = rotation_of(m["rot"])
    k_rot = rotate(down[:, None, R:], positions, freqs, magnitude, False)[:, 0]
    return c, k_rot


def latent_attention(h, w, p, m, eps, positions, rows):
    """``rows`` = (c, k_rot), this layer's own or another layer's."""
    T = h.shape[0]
    H, d, r, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    c, k_rot = rows
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, d + r)
    freqs, magnitude = rotation_of(m["rot"])
    q_rot = rotate(q[..., d:], positions, freqs, magnitude, False)
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    see = visible(T, (m.get("mask") or {}).get("size"))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        s = (q[:, head, :d] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * float(m["scale"])
        out[:, head] = torch.softmax(s.masked_fill(~see, -math.inf), -1) @ v[:, head]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T


# ------------------------------------------------------------------------------ the model


def forward(cfg, w, ids, keep_layers=False):
    """Logits [T, vocab] of one sequence (float64); with ``keep_layers`` also the stream after every layer."""
    w = {k: v.to(F64) for k, v in w.items() if v.is_floating_point()}
    eps = float(cfg["norm"]["eps"])
    mult = float(cfg.get("residual_mult", 1.0))
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    x = scalar_norm(w["embed"][ids], w["embed.norm"], eps)
    cached = {}
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = scalar_norm(x, w[f"l{i}.norm1"], eps)
        hc = h + causal_conv(h, w[f"l{i}.canon1"]) if "canon" in cfg else h
        if layer["type"] == "attention":
            mixed = sink_attention(hc, w, p, m, positions)
        else:
            source = m.get("kv_from")
            if source is None:
                cached[i] = latent_rows(hc, w, p, m, eps, positions)
                source = i
            mixed = latent_attention(hc, w, p, m, eps, positions, cached[source])
        branch = mixed
        if layer.get("mlp") is not None:
            branch = branch + dense_ff(h, w, f"l{i}.mlp.", eps)
        x = x + mult * branch
        streams.append(x)
    logits = scalar_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(streams)) if keep_layers else logits


# ------------------------------------------------------------------------------ configurations and weights for tests


def attention_layer(*, heads, kv_heads, dim, scale, base=10000.0, dims=None, window=None, ff=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
             "rot": {"base": base, "dims": dim if dims is None else dims}}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def latent_layer(*, heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, dims=None, window=None,
                 scaling=None, kv_from=None, ff=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": scale, "rot": rot}
    if window is not None:
        mixer["mask"] = {"size": window}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def model_config(*, vocab, width, eps, mult, taps, layers):
    cfg = {"architecture": "Zigivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
           "layers": layers}
    if taps is not None:
        cfg["canon"] = {"taps": taps}
    return cfg


def tensor_shapes(cfg):
    D, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, D), "embed.norm": (), "final.norm": (), "head": (V, D)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        shapes[f"l{i}.norm1"] = ()
        if "canon" in cfg:
            shapes[f"l{i}.canon1"] = (D, cfg["canon"]["taps"])
        if layer["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            shapes.update({p + "q": (H * d, D), p + "q.b": (H * d,), p + "k": (G * d, D), p + "k.b": (G * d,),
                           p + "o": (D, H * d)})
        else:
            H, d, r, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            shapes.update({p + "dq": (Q, D), p + "dq.norm": (Q,), p + "uq": (H * (d + r), Q), p + "uk": (H * d, R),
                           p + "uv": (H * dv, R), p + "g": (H * dv, D), p + "o": (D, H * dv)})
            if m.get("kv_from") is None:
                shapes.update({p + "dkv": (R + r, D), p + "dkv.norm": (R,)})
        if layer.get("mlp") is not None:
            F, q = layer["mlp"]["ff"], f"l{i}.mlp."
            shapes.update({q + "up": (F, D), q + "up.b": (F,), q + "down": (D, F), q + "down.b": (D,), q + "act": (4,)})
    return shapes


def random_weights(cfg, seed, sharpen=1.0):
    """bfloat16 tensors: matrices normal(0, 1/sqrt(in)), norm weights near one, biases and taps of moderate size.
    ``sharpen`` multiplies what makes queries, so that scores spread and single keys stand out."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name.endswith("norm1") or name in ("embed.norm", "final.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last == "norm":
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last == "canon1":
            t = 0.4 * torch.randn(shape, generator=g)
        elif last == "act":
            t = torch.tensor([0.9, 0.4, -0.3, 0.05]) + 0.1 * torch.randn(shape, generator=g)
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
            if last in ("q", "uq"):
                t = t * sharpen
        out[name] = t.to(torch.bfloat16)
    return out


def random_prompts(cfg, lengths, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


YARN = (6.0, 96, 8.0, 0.5)

# latent layers with windows of their own on shared rows, grouped heads, a partly rotated attention, a window on an
# attention layer, a layer without a feed-forward, four taps
TINY_A = model_config(vocab=97, width=64, eps=1e-5, mult=0.7, taps=4, layers=[
    latent_layer(heads=2, dim=16, rot_dim=8, vdim=12, kv_rank=24, q_rank=20, scale=0.2, window=70, scaling=YARN, ff=96),
    attention_layer(heads=4, kv_heads=2, dim=16, scale=0.25, dims=8, ff=80),
    latent_layer(heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=24, q_rank=28, scale=0.22, window=40, scaling=YARN,
                 kv_from=0, ff=None),
    attention_layer(heads=2, kv_heads=2, dim=32, scale=0.18, window=50, ff=96),
    latent_layer(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=12, q_rank=8, scale=0.3, dims=2, ff=48),
])
# a width off the multiples of 16, heads of 20 lanes, a latent row of 14 lanes (stored as 16), two taps, multiplier one,
# a reader without a window on rows whose writer has one
TINY_B = model_config(vocab=131, width=40, eps=1e-6, mult=1.0, taps=2, layers=[
    attention_layer(heads=3, kv_heads=3, dim=20, scale=0.2, base=500.0, ff=56),
    latent_layer(heads=3, dim=8, rot_dim=4, vdim=8, kv_rank=10, q_rank=12, scale=0.3, window=33, ff=56),
    latent_layer(heads=2, dim=8, rot_dim=4, vdim=12, kv_rank=10, q_rank=16, scale=0.3, kv_from=1, ff=24),
])
# whole heads of 64 lanes (the kernels that keep scores in tensor memory), one tap, one key/value head for four
TINY_C = model_config(vocab=211, width=128, eps=1e-5, mult=0.4, taps=1, layers=[
    latent_layer(heads=2, dim=48, rot_dim=16, vdim=64, kv_rank=32, q_rank=48, scale=0.12, window=100, scaling=(4.0, 64, 16.0, 2.0), ff=160),
    attention_layer(heads=4, kv_heads=1, dim=64, scale=0.125, dims=32, ff=160),
    latent_layer(heads=2, dim=48, rot_dim=16, vdim=64, kv_rank=32, q_rank=40, scale=0.12, window=100, scaling=(4.0, 64, 16.0, 2.0),
                 kv_from=0, ff=160),
])
# no convolution at all
NO_CONV = model_config(vocab=61, width=32, eps=1e-5, mult=0.5, taps=None, layers=[
    attention_layer(heads=2, kv_heads=1, dim=16, scale=0.25, ff=48),
    latent_layer(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=16, scale=0.25, window=20, ff=48),
])
# one layer of each kind with long reach: sharpened queries pick single keys far back
SHARP = model_config(vocab=151, width=48, eps=1e-5, mult=0.8, taps=3, layers=[
    attention_layer(heads=2, kv_heads=1, dim=16, scale=0.25, base=100000.0, ff=None),
    latent_layer(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=16, q_rank=24, scale=0.2, base=100000.0, window=300, ff=64),
])


def random_config(seed):
    """A configuration drawn from odd sizes."""
    g = torch.Generator().manual_seed(seed)
    pick = lambda *values: values[int(torch.randint(0, len(values), (1,), generator=g))]
    width = pick(24, 36, 52, 72)
    layers = []
    writers = []
    for i in range(pick(2, 3, 4)):
        ff = pick(None, 20, 44, 72)
        if pick(0, 1) or (i == 1 and not writers):
            rot_dim, kv_rank = pick(2, 4, 6), pick(5, 8, 14, 27)
            source = pick(None, *writers) if writers else None
            if source is not None:
                rot_dim, kv_rank = layers[source]["mixer"]["rot_dim"], layers[source]["mixer"]["kv_rank"]
            layer = latent_layer(heads=pick(1, 2, 3), dim=pick(4, 6, 10), rot_dim=rot_dim, vdim=pick(3, 8, 10), kv_rank=kv_rank,
                                 q_rank=pick(6, 9, 16), scale=pick(0.2, 0.35), base=pick(100.0, 10000.0),
                                 window=pick(None, 1, 17, 64, 65), kv_from=source, ff=ff,
                                 scaling=pick(None, (3.0, 40, 6.0, 1.0)))
            if source is not None:
                layer["mixer"]["rot"] = dict(layers[source]["mixer"]["rot"])
            else:
                writers.append(i)
            layers.append(layer)
        else:
            kv = pick(1, 2)
            dim = pick(4, 6, 16, 18)
            layers.append(attention_layer(heads=kv * pick(1, 2, 3), kv_heads=kv, dim=dim, scale=pick(0.2, 0.4),
                                          base=pick(100.0, 10000.0), dims=pick(2, dim), window=pick(None, None, 30), ff=ff))
    return model_config(vocab=pick(50, 77, 130), width=width, eps=pick(1e-5, 1e-6), mult=pick(0.3, 1.0, 1.5),
                        taps=pick(None, 1, 2, 3, 5), layers=layers)

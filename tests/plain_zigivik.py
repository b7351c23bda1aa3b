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
    mult = float(cfg["residual_mult"])
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    x = scalar_norm(w["embed"][ids], w["embed.norm"], eps)
    cached = {}
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = scalar_norm(x, w[f"l{i}.norm1"], eps)
        hc = h + causal_conv(h, w[f"l{i}.canon1"])
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

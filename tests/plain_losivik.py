"""A plain, slow restatement of the Losivik design, written from its equations: one function per mechanism, whole
sequences, float64, no cache, no kernels, nothing shared with the package.  The GPU tests hold the engine to it.

Notation: T tokens, W the model's width, x the residual stream [T, W], positions p = 0..T-1.

  embedding      x_p = E[token_p] * s + pe(p), pe(p)[2i] = sin(p b^(-2i/W)), pe(p)[2i+1] = cos(p b^(-2i/W)), b = 10000
  norm           n(x; w) = x / sqrt(mean(x^2) + eps) * (1 + w)            (plain norms multiply by w itself)
  layer          x <- x + ls1 * mixer(n(x; norm1)) + ls2 * ff(n(x; norm2));  x <- x + side(x, token)
  side           e = S[token][i*d : (i+1)*d];  y = P (gelu_tanh(G x) * e);  side = y / sqrt(mean(y^2) + eps) * w
  latent         c = plainnorm(Wdkv h);  k_h = Wuk_h c;  v_h = Wuv_h c;  q = Wq h;  softmax over the window;
                 head h times sigmoid((Wg h)_h);  Wo
  side by side   a * left + b * right
  left           grouped heads, plain norm per query / key head, window that keeps the first positions
  right          z, x, B, C, dt = split(Win h);  (x, B, C) <- silu(conv(x, B, C));  dt <- softplus(dt + bias);
                 S <- exp(-exp(A) dt) S + dt B x^T;  y = S^T C + D x;  y <- groupnorm(y * silu(z)) * w;  Wo
  dense          g = min(Wg h + bg, L);  u = clamp(Wu h + bu, -L, L);  Wd (g sigmoid(1.702 g) (u + 1)) + bd
  experts        s = sigmoid(R h);  chosen = top_k(s);  sum_k E_k(s_k h) + shared(h);  E(v) = Wd relu(Wu v)^2
  head           logits = E n(x; final)
"""

import copy
import math

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- mechanisms


def rms_divide(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms_divide(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_divide(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def sinusoid(positions, width, base=10000.0):
    """The design takes positions and angles in 32 bits: the frequency base^(-2i/width) is rounded to a float, and so
    is its product with the position; sine and cosine of that angle are taken exactly."""
    out = torch.zeros(len(positions), width, dtype=F64)
    for row, p in enumerate(positions):
        for i in range((width + 1) // 2):
            frequency = torch.tensor(base ** (-2.0 * i / width), dtype=torch.float32)
            angle = float(torch.tensor(float(p), dtype=torch.float32) * frequency)
            out[row, 2 * i] = math.sin(angle)
            if 2 * i + 1 < width:
                out[row, 2 * i + 1] = math.cos(angle)
    return out


def visible(T, window=None, keep_first=0):
    """[T, T] booleans: row p sees column j."""
    p = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= p
    if window is not None:
        seen = seen & ((p - j < window) | (j < keep_first))
    return seen


def attend(q, k, v, scale, seen):
    """q [T, H, d], k [T, H, d], v [T, H, dv] -> [T, H, dv]; ordinary softmax over the visible keys."""
    scores = torch.einsum("phd,jhd->hpj", q, k) * scale
    scores = scores.masked_fill(~seen[None], float("-inf"))
    return torch.einsum("hpj,jhd->phd", torch.softmax(scores, -1), v)


def latent_attention(w, p, m, h, eps):
    T, H, d, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    c = norm_plain(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)
    k = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    out = attend(q, k, v, m["scale"], visible(T, (m.get("mask") or {}).get("size")))
    out = out * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def grouped_attention(w, p, m, h, eps):
    T, H, G, d, dv = h.shape[0], m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = norm_plain((h @ w[p + "q"].T).view(T, H, d), w[p + "q.norm"], eps)
    k = norm_plain((h @ w[p + "k"].T).view(T, G, d), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    k, v = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    mask = m.get("mask") or {}
    out = attend(q, k, v, m["scale"], visible(T, mask.get("size"), mask.get("keep_first") or 0))
    return out.reshape(T, H * dv) @ w[p + "o"].T


def causal_convolution(x, taps, bias):
    """x [T, C], taps [C, n] (the last column weighs the current token), zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=x.dtype), x], 0)
    return sum(padded[j:j + T] * taps[:, j] for j in range(n)) + bias


def state_space(w, p, m, h, eps, state=None):
    T, H, P, N, G = h.shape[0], m["heads"], m["vdim"], m["state"], m.get("groups", 1)
    inner, parts = H * P, m.get("norm_groups", 1)
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_convolution(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"])
    rate = torch.exp(w[p + "A_log"])
    S = torch.zeros(H, N, P, dtype=F64)
    y = torch.zeros(T, H, P, dtype=F64)
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            S[head] = torch.exp(-rate[head] * dt[t, head]) * S[head] + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S[head].T @ C[t, g] + w[p + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    y = rms_divide(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def dense_feed_forward(w, p, f, h):
    L = f["limit"]
    g = torch.clamp(h @ w[p + "gate"].T + w[p + "gate.b"], max=L)
    u = torch.clamp(h @ w[p + "up"].T + w[p + "up.b"], -L, L)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T + w[p + "down.b"]


def squared_relu_expert(w, p, v):
    return torch.relu(v @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def router_choice(w, p, f, h):
    """(indices [T, top], scores [T, top]) of the largest sigmoid scores, the lower index first among equals."""
    scores = torch.sigmoid(h @ w[p + "router"].T)
    order = torch.sort(scores, dim=-1, descending=True, stable=True)
    top = f["router"]["top"]
    return order.indices[:, :top], order.values[:, :top]


def routed_feed_forward(w, p, f, h):
    chosen, scores = router_choice(w, p, f, h)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), scores[t]):
            out[t] += squared_relu_expert(w, f"{p}e{e}.", (s * h[t])[None])[0]
    if f.get("shared"):
        out = out + squared_relu_expert(w, p + "shared.", h)
    return out


def token_side_input(w, cfg, layer, x, tokens):
    d = cfg["token_side"]["dim"]
    e = w["side.embed"][torch.tensor(tokens)][:, layer * d:(layer + 1) * d]
    y = (gelu_tanh(x @ w[f"l{layer}.side.gate"].T) * e) @ w[f"l{layer}.side.proj"].T
    return norm_plain(y, w[f"l{layer}.side.norm"], cfg["norm"]["eps"])


def forward(cfg, weights, tokens, keep_layers=False):
    """Logits [T, vocab] of the whole sequence (and, with ``keep_layers``, the stream after every layer)."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps, W = cfg["norm"]["eps"], cfg["width"]
    x = w["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0) + sinusoid(range(len(tokens)), W)
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = norm_one_plus(x, w[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            mixed = latent_attention(w, p + "mix.", m, h, eps)
        else:
            mixed = (m.get("left_scale", 1.0) * grouped_attention(w, p + "mix.left.", m["left"], h, eps)
                     + m.get("right_scale", 1.0) * state_space(w, p + "mix.right.", m["right"], h, eps))
        update = mixed * w[p + "ls1"]
        f = layer.get("mlp")
        if f is not None:
            h = norm_one_plus(x, w[p + "norm2"], eps)
            fed = dense_feed_forward(w, p + "mlp.", f, h) if f["kind"] == "dense" else routed_feed_forward(w, p + "mlp.", f, h)
            update = update + fed * w[p + "ls2"]
        x = x + update
        if cfg.get("token_side"):
            x = x + token_side_input(w, cfg, i, x, tokens)
        streams.append(x.clone())
    logits = norm_one_plus(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(streams)) if keep_layers else logits


# ----------------------------------------------------------------------------- configurations and weights


def _latent(heads, dim, vdim, rank, scale, window=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def _pair(heads, kv_heads, dim, vdim, scale, window, keep, r_heads, r_vdim, state, groups, conv, parts, a=0.7, b=1.2):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        left["mask"] = {"size": window, **({"keep_first": keep} if keep else {})}
    right = {"heads": r_heads, "vdim": r_vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": parts}
    return {"left": left, "right": right, "left_scale": a, "right_scale": b}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(experts, top, ff, shared=None):
    f = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def _config(vocab, width, layers, scale=1.0, side=None, eps=1e-5):
    cfg = {"architecture": "Losivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
           "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


# every size differs from its neighbours; two key/value heads for six, top 2, windows off the page size
TINY_A = _config(160, 96, [
    {"type": "parallel", "mixer": _pair(6, 2, 32, 48, 0.2, 40, 5, 6, 16, 24, 3, 4, 3), "mlp": _moe(6, 2, 40, 24)},
    {"type": "latent_attention", "mixer": _latent(3, 32, 16, 48, 0.15, 70), "mlp": _dense(72, 2.0)},
    {"type": "latent_attention", "mixer": _latent(2, 16, 32, 32, 0.3), "mlp": None},
    {"type": "parallel", "mixer": _pair(4, 4, 16, 16, 0.25, None, 0, 2, 40, 16, 1, 2, 1), "mlp": _dense(40, 0.7)},
], scale=1.7, side=8)
# sizes off the multiples of 8 and 16: the kernels' general forms
TINY_B = _config(97, 100, [
    {"type": "latent_attention", "mixer": _latent(3, 20, 12, 28, 0.22, 33), "mlp": _moe(5, 3, 28)},
    {"type": "parallel", "mixer": _pair(3, 1, 20, 12, 0.3, 50, 70, 3, 5, 10, 1, 1, 3), "mlp": _moe(3, 1, 36, 20)},
    {"type": "parallel", "mixer": _pair(2, 2, 24, 24, 0.2, 64, 64, 4, 9, 33, 2, 5, 2), "mlp": None},
], scale=0.6, side=5, eps=1e-6)
# windows and kept first tokens that need pinned pages and a ring; no token-side input, no embedding scale
TINY_C = _config(120, 64, [
    {"type": "parallel", "mixer": _pair(4, 2, 16, 32, 0.25, 30, 70, 4, 8, 16, 2, 3, 2), "mlp": _dense(48, 1.2)},
    {"type": "latent_attention", "mixer": _latent(4, 16, 16, 16, 0.25, 65), "mlp": _moe(4, 2, 32, 16)},
    {"type": "parallel", "mixer": _pair(2, 1, 32, 16, 0.18, 129, 1, 2, 32, 8, 1, 2, 1), "mlp": _dense(32, 3.0)},
])
# sizes in the middle: heads of 96 and 80 lanes, latent rows of 160, which take other kernel forms than the small ones
TINY_D = _config(200, 160, [
    {"type": "latent_attention", "mixer": _latent(5, 96, 80, 160, 0.1, 100), "mlp": _moe(4, 2, 64, 32)},
    {"type": "parallel", "mixer": _pair(6, 3, 96, 80, 0.1, 90, 10, 5, 24, 80, 5, 2, 1), "mlp": _dense(200, 1.0)},
], scale=0.8, side=24)
# heads of 128 lanes on both sides: the kernels that keep scores in tensor memory, with kept first positions
TINY_E = _config(150, 128, [
    {"type": "parallel", "mixer": _pair(4, 2, 128, 128, 0.09, 70, 3, 4, 32, 64, 2, 4, 2), "mlp": _dense(96, 1.5)},
    {"type": "latent_attention", "mixer": _latent(2, 128, 128, 64, 0.09, 100), "mlp": _moe(3, 2, 48)},
], scale=1.2, side=16)
# sharpened softmaxes: a layer of each attention kind with windows of hundreds of positions
SHARP = _config(90, 64, [
    {"type": "parallel", "mixer": _pair(4, 2, 16, 16, 0.25, 200, 40, 2, 16, 8, 1, 2, 1), "mlp": None},
    {"type": "latent_attention", "mixer": _latent(4, 16, 16, 32, 0.25, 300), "mlp": _dense(48, 1.5)},
])


def random_weights(cfg, seed, sharpen=1.0):
    """Every tensor of the design, rounded to bfloat16 values so that both compute dtypes hold the same numbers."""
    gen = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = torch.randn(rows, cols, generator=gen) * gain / math.sqrt(cols)

    def vector(name, n, mean=0.0, std=0.1):
        out[name] = mean + std * torch.randn(n, generator=gen)

    out["embed"] = torch.randn(V, W, generator=gen)
    side = (cfg.get("token_side") or {}).get("dim")
    if side:
        out["side.embed"] = torch.randn(V, side * len(cfg["layers"]), generator=gen)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        vector(p + "norm1", W)
        vector(p + "ls1", W, 0.6, 0.15)
        if layer["type"] == "latent_attention":
            H, d, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            matrix(p + "mix.q", H * d, W, sharpen)
            matrix(p + "mix.dkv", R, W)
            vector(p + "mix.dkv.norm", R, 1.0)
            matrix(p + "mix.uk", H * d, R, sharpen)
            matrix(p + "mix.uv", H * dv, R)
            matrix(p + "mix.g", H, W)
            matrix(p + "mix.o", W, H * dv)
        else:
            a, b = m["left"], m["right"]
            H, G, d, dv = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a.get("vdim", a["dim"])
            matrix(p + "mix.left.q", H * d, W)
            matrix(p + "mix.left.k", G * d, W)
            matrix(p + "mix.left.v", G * dv, W)
            vector(p + "mix.left.q.norm", d, sharpen * sharpen, 0.1)
            vector(p + "mix.left.k.norm", d, 1.0, 0.1)
            matrix(p + "mix.left.o", W, H * dv)
            Hs, P, N, Gs, taps = b["heads"], b["vdim"], b["state"], b.get("groups", 1), b.get("conv", 1)
            inner, C = Hs * P, Hs * P + 2 * Gs * N
            matrix(p + "mix.right.in", inner + C + Hs, W)
            out[p + "mix.right.conv"] = torch.randn(C, taps, generator=gen) * 0.5
            vector(p + "mix.right.conv.b", C)
            vector(p + "mix.right.dt_bias", Hs, -1.0, 0.5)
            out[p + "mix.right.A_log"] = torch.log(0.05 + 0.6 * torch.rand(Hs, generator=gen))     # memory over tens of tokens
            vector(p + "mix.right.D", Hs, 1.0, 0.3)
            vector(p + "mix.right.norm", inner, 1.0)
            matrix(p + "mix.right.o", W, inner)
        f = layer.get("mlp")
        if f is not None:
            vector(p + "norm2", W)
            vector(p + "ls2", W, 0.6, 0.15)
            if f["kind"] == "dense":
                matrix(p + "mlp.gate", f["ff"], W, 1.5)
                vector(p + "mlp.gate.b", f["ff"], 0.0, 0.3)
                matrix(p + "mlp.up", f["ff"], W, 1.5)
                vector(p + "mlp.up.b", f["ff"], 0.0, 0.3)
                matrix(p + "mlp.down", W, f["ff"])
                vector(p + "mlp.down.b", W)
            else:
                matrix(p + "mlp.router", f["router"]["experts"], W, 2.0)
                for e in range(f["router"]["experts"]):
                    matrix(f"{p}mlp.e{e}.up", f["expert"]["ff"], W, 1.5)
                    matrix(f"{p}mlp.e{e}.down", W, f["expert"]["ff"])
                if f.get("shared"):
                    matrix(p + "mlp.shared.up", f["shared"]["ff"], W, 1.5)
                    matrix(p + "mlp.shared.down", W, f["shared"]["ff"])
        if side:
            matrix(p + "side.gate", side, W)
            matrix(p + "side.proj", W, side)
            vector(p + "side.norm", W, 0.3, 0.1)
    vector("final.norm", W)
    return {k: v.to(torch.bfloat16) for k, v in out.items()}


def random_prompts(cfg, lengths, seed):
    gen = torch.Generator().manual_seed(1000 + seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=gen).tolist() for n in lengths]


def random_config(seed):
    """A configuration drawn from odd sizes: widths off the multiples of 8, head counts and group counts that do
    not divide alike, windows beside the page size, with and without each optional mechanism."""
    gen = torch.Generator().manual_seed(7000 + seed)
    pick = lambda *values: values[int(torch.randint(0, len(values), (1,), generator=gen))]
    layers = []
    for _ in range(pick(2, 3)):
        if pick(0, 1):
            heads = pick(1, 2, 3, 5)
            m = _latent(heads, pick(6, 16, 20, 33), pick(5, 8, 24), pick(7, 16, 36, 48), pick(0.1, 0.3), pick(None, 1, 31, 64, 100))
            kind = "latent_attention"
        else:
            kv = pick(1, 2, 3)
            rh = pick(1, 2, 6)
            window = pick(None, 17, 64, 90)
            m = _pair(kv * pick(1, 2, 4), kv, pick(6, 16, 20, 48), pick(5, 16, 40), pick(0.1, 0.3), window,
                      pick(0, 1, 9, 64, 65) if window else 0, rh, pick(3, 8, 33), pick(4, 7, 16, 40),
                      pick(*[g for g in (1, 2, 3) if rh % g == 0]), pick(1, 2, 4), 1, pick(0.5, 1.0), pick(1.0, 1.5))
            inner = m["right"]["heads"] * m["right"]["vdim"]
            m["right"]["norm_groups"] = pick(*[g for g in (1, 2, 3) if inner % g == 0])
            kind = "parallel"
        f = pick(None, "dense", "moe", "moe")
        if f == "dense":
            f = _dense(pick(10, 24, 52), pick(0.5, 2.0))
        elif f == "moe":
            experts = pick(2, 3, 7)
            f = _moe(experts, pick(*range(1, experts + 1)), pick(6, 16, 28), pick(None, 12))
        layers.append({"type": kind, "mixer": m, "mlp": f})
    return _config(pick(50, 131), pick(36, 50, 64, 72), layers, scale=pick(1.0, 0.5, 2.0), side=pick(None, 3, 8), eps=pick(1e-5, 1e-6))


def tensor_shapes(cfg):
    """Name -> shape of every tensor that a model of this configuration stores."""
    W, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,)}
    side = (cfg.get("token_side") or {}).get("dim")
    if side:
        shapes["side.embed"] = (V, side * len(cfg["layers"]))
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes.update({p + "norm1": (W,), p + "ls1": (W,)})
        if layer["type"] == "latent_attention":
            H, d, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.dkv": (R, W), p + "mix.dkv.norm": (R,), p + "mix.uk": (H * d, R),
                           p + "mix.uv": (H * dv, R), p + "mix.g": (H, W), p + "mix.o": (W, H * dv)})
        else:
            a, b = m["left"], m["right"]
            H, G, d, dv = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a.get("vdim", a["dim"])
            shapes.update({p + "mix.left.q": (H * d, W), p + "mix.left.k": (G * d, W), p + "mix.left.v": (G * dv, W),
                           p + "mix.left.q.norm": (d,), p + "mix.left.k.norm": (d,), p + "mix.left.o": (W, H * dv)})
            Hs, P, N, Gs, taps = b["heads"], b["vdim"], b["state"], b.get("groups", 1), b.get("conv", 1)
            inner, C = Hs * P, Hs * P + 2 * Gs * N
            shapes.update({p + "mix.right.in": (inner + C + Hs, W), p + "mix.right.conv": (C, taps), p + "mix.right.conv.b": (C,),
                           p + "mix.right.dt_bias": (Hs,), p + "mix.right.A_log": (Hs,), p + "mix.right.D": (Hs,),
                           p + "mix.right.norm": (inner,), p + "mix.right.o": (W, inner)})
        f = layer.get("mlp")
        if f is not None:
            shapes.update({p + "norm2": (W,), p + "ls2": (W,)})
            if f["kind"] == "dense":
                shapes.update({p + "mlp.gate": (f["ff"], W), p + "mlp.gate.b": (f["ff"],), p + "mlp.up": (f["ff"], W),
                               p + "mlp.up.b": (f["ff"],), p + "mlp.down": (W, f["ff"]), p + "mlp.down.b": (W,)})
            else:
                shapes[p + "mlp.router"] = (f["router"]["experts"], W)
                for e in range(f["router"]["experts"]):
                    shapes.update({f"{p}mlp.e{e}.up": (f["expert"]["ff"], W), f"{p}mlp.e{e}.down": (W, f["expert"]["ff"])})
                if f.get("shared"):
                    shapes.update({p + "mlp.shared.up": (f["shared"]["ff"], W), p + "mlp.shared.down": (W, f["shared"]["ff"])})
        if side:
            shapes.update({p + "side.gate": (side, W), p + "side.proj": (W, side), p + "side.norm": (W,)})
    return shapes

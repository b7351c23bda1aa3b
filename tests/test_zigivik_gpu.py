"""The Zigivik design in the engine against its plain restatement (``plain_zigivik``): each mechanism alone, whole
prompts, token-by-token decoding, portions, batches of unequal requests, slots and pages used again, far keys, page
borders and window edges, the first tokens, long decoding round the ring of a windowed cache, sizes of one, and
greedy generation through ``generate`` and the command line.

float32 is compared strictly.  bfloat16 is compared by the error of a row relative to the row's size (there is no
routing in this design, so no row can take another way than the plain implementation's, and every row is held)."""

import copy
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import ondeviceinfer_b200 as odi
import plain_zigivik as plain
from helpers import assert_logits_close, write_model_folder
from ondeviceinfer_b200.kernels import ops

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
CONFIGS = {"A": (plain.TINY_A, 41), "B": (plain.TINY_B, 42), "C": (plain.TINY_C, 43), "bare": (plain.NO_CONV, 44),
           "sharp": (plain.SHARP, 45)}
SHARPEN = {"sharp": 3.0}
_MODELS, _PLAIN = {}, {}


def weights_of(case):
    return plain.random_weights(*CONFIGS[case], sharpen=SHARPEN.get(case, 1.0))


def engine(case, dtype, tmp_path_factory):
    if (case, dtype) not in _MODELS:
        folder = write_model_folder(tmp_path_factory.mktemp(f"zigivik_{case}"), CONFIGS[case][0], weights_of(case))
        _MODELS[(case, dtype)] = odi.load_resident_model(folder, dtype=dtype)
    return _MODELS[(case, dtype)]


def expected(case, tokens):
    key = (case, tuple(tokens))
    if key not in _PLAIN:
        _PLAIN[key] = plain.forward(CONFIGS[case][0], weights_of(case), list(tokens)).float()
    return _PLAIN[key]


def close(actual, reference, dtype, what, atol=None):
    """float32: the helpers' strict comparison, or with ``atol`` |d| <= atol (for positions in the hundreds: the fp32
    angle of position p is off by up to p 2^-24 rad against the plain implementation's float64 one, which large
    scores and a softmax that picks single keys pass on to the logits).  bfloat16: row error relative to the row's
    size: median at most 1.5e-2, nine rows in ten within 5e-2, every row within 1.5e-1 (a row of small logits has a
    large relative error)."""
    if dtype == "float32" and atol is not None:
        gap = float((actual.float().cpu() - reference.float().cpu()).abs().max())
        assert actual.shape == reference.shape and gap <= atol, f"{what}: fp32 max |d| = {gap:.3e}"
        return
    if dtype == "float32":
        assert_logits_close(actual, reference, dtype, what)
        return
    actual, reference = actual.float().cpu(), reference.float().cpu()
    assert actual.shape == reference.shape and torch.isfinite(actual).all(), what
    error = (actual - reference).norm(dim=-1) / reference.norm(dim=-1).clamp_min(1e-6)
    ranked = error.sort().values
    high = ranked[int(0.9 * len(ranked))] if len(ranked) >= 10 else ranked[-1]
    assert float(ranked[-1]) <= 1.5e-1 and float(error.median()) <= 1.5e-2 and float(high) <= 5e-2, \
        f"{what}: bfloat16 row errors median {float(error.median()):.3e}, high {float(high):.3e}, max {float(ranked[-1]):.3e}"


def ints(*values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


# ----------------------------------------------------------------------------- kernels against plain functions


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,width,steps", [(1, 24, "short"), (2, 40, "short"), (3, 64, "short"), (5, 100, "short"),
                                              (8, 1032, "short"), (12, 40, "short"), (20, 28, "short"), (1, 24, "long"), (3, 40, "long"), (4, 136, "long"),
                                              (8, 72, "long")])
def test_norm_and_convolution_with_state_over_cut_sequences(dtype, taps, width, steps):
    """Three sequences cut into unequal runs (runs shorter than the taps among them): h and h + conv(h) of every run
    against the plain norm and convolution of the whole sequences.  The long steps carry hundreds and thousands of
    tokens (the kernel whose blocks take runs of four or eight tokens), single tokens of other sequences among them,
    and sequences that start in the middle of a block's run."""
    g = torch.Generator().manual_seed(taps)
    eps, scalar = 1e-5, torch.tensor([1.3])
    w = (0.5 * torch.randn(width, taps, generator=g))
    if steps == "short":
        lengths = [23, 9, 40]
        cuts = [[1, 1, 2, 7, 1, 11], [4, 1, 1, 3], [17, 1, 1, 1, 20]]
    else:
        lengths = [5000, 9, 903]
        cuts = [[4299, 1, 699, 1], [3, 1, 1, 4], [1, 298, 1, 603]]
    xs = [torch.randn(n, width, generator=g) * (1 + torch.arange(n)[:, None] % 3) for n in lengths]
    state = torch.full((5, max(taps - 1, 1), width), 9.0, device="cuda")[:, :taps - 1].contiguous() if taps > 1 else None
    slots = [3, 0, 2]
    if state is not None:
        state[slots] = 0.0              # what a sequence's start finds
    got_h = [[] for _ in lengths]
    got_hc = [[] for _ in lengths]
    at = [0, 0, 0]
    for step in range(max(len(c) for c in cuts)):
        live = [s for s in range(3) if step < len(cuts[s])]
        runs = [xs[s][at[s]:at[s] + cuts[s][step]] for s in live]
        x = torch.cat(runs).cuda()
        n = x.shape[0]
        cu = [0]
        for r in runs:
            cu.append(cu[-1] + r.shape[0])
        tok_seq = torch.cat([torch.full((r.shape[0],), i) for i, r in enumerate(runs)]).int().cuda()
        h, hc = torch.empty((n, width), dtype=dtype, device="cuda"), torch.empty((n, width), dtype=dtype, device="cuda")
        args = (x, scalar.cuda(), eps, w.cuda(), state, tok_seq, ints(*cu), ints(*[slots[s] for s in live]))
        ops.canon_norm(*args, h, hc)
        ops.canon_state(*args)
        for i, s in enumerate(live):
            got_h[s].append(h[cu[i]:cu[i + 1]].float().cpu())
            got_hc[s].append(hc[cu[i]:cu[i + 1]].float().cpu())
            at[s] += cuts[s][step]
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for s, x in enumerate(xs):
        want_h = plain.scalar_norm(x.double(), scalar.double(), eps)
        want_hc = want_h + plain.causal_conv(want_h, w.double())
        assert (torch.cat(got_h[s]) - want_h).abs().max() < tol, (taps, s)
        assert ((torch.cat(got_hc[s]) - want_hc).abs() <= tol * (1 + want_hc.abs())).all(), (taps, s)
        if taps > 1:        # the state holds h of the last positions (zeros before the start); other slots are untouched
            kept = torch.cat([torch.zeros(max(taps - 1 - x.shape[0], 0), width, dtype=torch.float64), want_h[-(taps - 1):]])
            assert (state[slots[s]].cpu() - kept).abs().max() < 2e-5
    if taps > 1:
        assert float(state[1].min()) == 9.0 and float(state[4].max()) == 9.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,F", [(1, 4), (7, 56), (33, 384), (5, 3000)])
def test_polynomial_activation(dtype, rows, F):
    g = torch.Generator().manual_seed(F)
    z = (1.5 * torch.randn(rows, F, generator=g)).to(dtype)
    coef = torch.tensor([0.8, -0.5, 0.3, 0.1])
    out = torch.empty_like(z, device="cuda")
    ops.poly_norm(z.cuda(), coef.cuda(), 1e-6, out)
    want = plain.poly_norm(z.double(), coef.double(), 1e-6)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert ((out.cpu().double() - want).abs() <= tol * (1 + want.abs())).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_slice_norm_head_gate_and_scaled_add(dtype):
    g = torch.Generator().manual_seed(5)
    n, ld, col, Q = 19, 90, 14, 37
    x = torch.randn(n, ld, generator=g).to(dtype)
    w = 1 + 0.3 * torch.randn(Q, generator=g)
    out = torch.empty((n, Q), dtype=dtype, device="cuda")
    ops.slice_norm(x.cuda(), w.cuda(), 1e-5, out, col=col)
    want = plain.rms(x[:, col:col + Q].double(), 1e-5) * w.double()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert ((out.cpu().double() - want).abs() <= tol * (1 + want.abs())).all()
    heads, dv, lanes = 3, 10, 16
    y = torch.randn(n, heads * lanes, generator=g).to(dtype)
    gated = y.clone().cuda()
    ops.gate_heads(gated, x.cuda(), heads=heads, dv=dv, lanes=lanes, col=col)
    want = y.double().view(n, heads, lanes).clone()
    want[..., :dv] *= torch.sigmoid(x[:, col:col + heads * dv].double().view(n, heads, dv))
    assert ((gated.cpu().double().view(n, heads, lanes) - want).abs() <= tol * (1 + want.abs())).all()
    assert torch.equal(gated.cpu().view(n, heads, lanes)[..., dv:], y.view(n, heads, lanes)[..., dv:])
    a, b = torch.randn(7, 33, generator=g), torch.randn(7, 33, generator=g)
    acc = a.clone().cuda()
    ops.scaled_add(acc, b.cuda(), 0.35)
    assert (acc.cpu() - (a + 0.35 * b)).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,rot,nq,nkv", [(16, 8, 4, 2), (6, 6, 3, 1), (48, 2, 2, 2), (20, 0, 1, 1), (160, 160, 2, 1)])
def test_head_preparation_keeps_unrotated_keys_as_values(dtype, d, rot, nq, nkv):
    g = torch.Generator().manual_seed(d)
    n, lanes = 70, -(-d // 4) * 4
    qk = torch.randn(n, (nq + nkv) * d, generator=g).to(dtype)
    pos = torch.randint(0, 500, (n,), generator=g).int()
    freqs = plain.plain_frequencies(rot, 50.0) if rot else None
    q_out = torch.full((n, nq * lanes), 7.0, dtype=dtype, device="cuda")
    k_pool = torch.zeros((n, nkv, 64, lanes), dtype=dtype, device="cuda")       # a ring of one page per token
    v_pool = torch.zeros((n, nkv, 64, d), dtype=dtype, device="cuda")
    cos = sin = None
    if rot:
        angle = pos.double()[:, None] * torch.tensor(freqs, dtype=torch.float64)[None, :]
        cos, sin = torch.cos(angle).float().cuda(), torch.sin(angle).float().cuda()
    seq = torch.arange(n, dtype=torch.int32, device="cuda")
    ops.rot_unit_prep(qk.cuda(), q_out, k_pool, v_pool, cos, sin, seq, pos.cuda(), seq, seq, nq=nq, nkv=nkv, d=d, dv=d,
                      rot_dim=rot, page_size=64, ring_pages=1, write_kv=True, unit_eps=None, d_store=lanes, v_from_k=True)
    wide = qk.double()
    q, k = wide[:, :nq * d].view(n, nq, d), wide[:, nq * d:].view(n, nkv, d)
    if rot:
        q, k = plain.rotate(q, pos, freqs, 1.0, True), plain.rotate(k, pos, freqs, 1.0, True)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    rows = torch.arange(n)
    got_k = k_pool[rows, :, (pos % 64).long()].cpu().double()
    assert (q_out.view(n, nq, lanes).cpu().double()[..., :d] - q).abs().max() < tol and (got_k[..., :d] - k).abs().max() < tol
    assert torch.equal(v_pool[rows, :, (pos % 64).long()].cpu().reshape(n, -1), qk[:, nq * d:])


def _paged(x, n_pages):
    """[T, heads, lanes] -> pool [pages, heads, 64, lanes] with position p in page p // 64."""
    T, heads, lanes = x.shape
    pool = torch.zeros((n_pages, heads, 64, lanes), dtype=x.dtype)
    for p in range(T):
        pool[p // 64, :, p % 64] = x[p]
    return pool


def _sink_reference(q, k, v, scale, window, past):
    T, nq, _ = q.shape
    total, nkv = k.shape[0], k.shape[1]
    i = past + torch.arange(T)[:, None]
    j = torch.arange(total)[None, :]
    see = (j <= i) & ((i - j) < window if window else True)
    out = torch.zeros(T, nq, v.shape[-1], dtype=torch.float64)
    for h in range(nq):
        s = (q[:, h].double() @ k[:, h // (nq // nkv)].double().T * scale).masked_fill(~see, -math.inf)
        e = torch.exp(s)
        out[:, h] = (e / (1.0 + e.sum(-1, keepdim=True))) @ v[:, h // (nq // nkv)].double()
    return out


def _sink_attention(kind, q, k, v, scale, window, past, splits=1):
    """Run one of the kernels that know the sink on ``T`` queries over ``past + T`` cached keys."""
    T, nq, d = q.shape
    total, nkv, dv = v.shape
    n_pages = -(-total // 64)
    out = torch.empty((T, nq * dv), dtype=q.dtype, device="cuda")
    common = dict(n_seqs=1, nq=nq, nkv=nkv, d=d, dv=dv, page_size=64, ring_pages=0, window=window or 0, scale=scale)
    tables = (ints(0, T), ints(past), ints(0, n_pages), torch.arange(n_pages, dtype=torch.int32, device="cuda"))
    partial = torch.empty(T * nq * splits * (dv + 2), device="cuda") if splits > 1 else None
    k_pool, v_pool = _paged(k, n_pages).cuda(), _paged(v, n_pages).cuda()
    if kind == "cores":
        ops.attention_simt(q.reshape(T, -1).cuda(), k_pool, v_pool, out, *tables, max_q_len=T, splits=splits, partial=partial,
                           sink=True, **common)
    elif kind == "mma":
        ops.attention_capped(q.reshape(T, -1).cuda(), k_pool, v_pool, out, *tables, max_q_len=T, sink=True, **common)
    elif kind == "mma single":
        ops.attention_capped_decode(q.reshape(T, -1).cuda(), k_pool, v_pool, out, *tables, splits=splits, partial=partial,
                                    sink=True, **common)
    else:
        del common["dv"], common["ring_pages"], common["window"]
        ops.attention_tcgen05(q.reshape(T, -1).cuda(), k_pool, v_pool, out, *tables, max_q_len=T, window=window or 0,
                              ring_pages=0, sink=True, **common)
    return out.view(T, nq, dv).cpu().double()


SINK_CASES = [(None, 200, 0, 1), (64, 200, 0, 1), (65, 131, 100, 1), (1, 40, 0, 1), (7, 1, 190, 3), (None, 1, 700, 5), (300, 1, 700, 4)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,T,past,splits", SINK_CASES)
def test_softmax_with_a_sink_on_the_cuda_cores(dtype, window, T, past, splits):
    g = torch.Generator().manual_seed(T + past)
    nq, nkv, d, scale, total = 4, 2, 12, 0.6, past + T
    q = torch.randn(T, nq, d, generator=g).to(dtype)
    k = torch.randn(total, nkv, d, generator=g).to(dtype)
    v = torch.randn(total, nkv, d, generator=g).to(dtype)
    got = _sink_attention("cores", q, k, v, scale, window, past, splits)
    want = _sink_reference(q, k, v, scale, window, past)
    assert (got - want).abs().max() < (2e-5 if dtype == torch.float32 else 2e-2)
    # without the sink's term the result would be another one
    plain_softmax = want / want.abs().sum(-1, keepdim=True).clamp_min(1e-9)
    assert (plain_softmax - want).abs().max() > 1e-3


@pytest.mark.parametrize("window,T,past,splits", SINK_CASES + [(None, 300, 0, 1), (100, 70, 300, 1)])
@pytest.mark.parametrize("d", [16, 48, 64])
def test_softmax_with_a_sink_on_the_tensor_cores(d, window, T, past, splits):
    """The bfloat16 kernels: the form for prompts and portions, the split-key form for single tokens, and for heads
    of 64 lanes and more than 16 queries the kernel that keeps scores in tensor memory.  Scores far below zero in
    some heads (the sink then takes nearly all the weight) and far above in others."""
    g = torch.Generator().manual_seed(T + past + d)
    nq, nkv, total = 4, 2, past + T
    scale = 1.0 / math.sqrt(d)
    q = torch.randn(T, nq, d, generator=g)
    q[:, 0] *= 4.0
    k = torch.randn(total, nkv, d, generator=g)
    q[:, 1] = -3.0 * k[past:past + T, 0] - 0.5 * k[:1, 0]                  # every visible score of head 1 is negative-ish
    q, k = q.bfloat16(), k.bfloat16()
    v = torch.randn(total, nkv, d, generator=g).bfloat16()
    want = _sink_reference(q, k, v, scale, window, past)
    kinds = ["mma single"] if T == 1 else ["mma"] + (["tcgen05"] if d == 64 and T > 16 else [])
    for kind in kinds:
        got = _sink_attention(kind, q, k, v, scale, window, past, splits)
        assert (got - want).abs().max() < 3e-2, kind


def _shared_row_reference(q, rows, dv, scale, window, past):
    """Ordinary softmax where a cached row is every head's key and its first ``dv`` lanes are the value."""
    T, nq, _ = q.shape
    i = past + torch.arange(T)[:, None]
    j = torch.arange(rows.shape[0])[None, :]
    see = (j <= i) & ((i - j) < window if window else True)
    out = torch.zeros(T, nq, dv, dtype=torch.float64)
    for h in range(nq):
        s = (q[:, h].double() @ rows.double().T * scale).masked_fill(~see, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ rows[:, :dv].double()
    return out


@pytest.mark.parametrize("window,T,past,splits", [(None, 150, 0, 1), (64, 150, 0, 1), (65, 70, 130, 1), (1, 20, 50, 1),
                                                   (None, 1, 0, 1), (7, 1, 190, 3), (None, 1, 700, 5), (300, 1, 700, 4),
                                                   (128, 1, 127, 2), (128, 1, 128, 2), (None, 3, 447, 1)])
@pytest.mark.parametrize("d,dv,nq", [(32, 16, 1), (48, 32, 3), (96, 80, 16), (576, 512, 20)])
def test_shared_row_attention_on_the_tensor_cores(d, dv, nq, window, T, past, splits):
    """The bfloat16 kernel over a latent cache: prompts' portions and single tokens with split keys, head counts
    below, at and above a block's sixteen rows.  One head asks sharply for the oldest key it may see and another for
    the one just outside its window, so a window that is one off, or a split that loses its range, shows."""
    g = torch.Generator().manual_seed(T + past + d + nq)
    total, scale = past + T, 1.0 / math.sqrt(d)
    rows = torch.randn(total, d, generator=g)
    q = torch.randn(T, nq, d, generator=g)
    for t in range(T):
        p = past + t
        oldest = max(0, p - window + 1) if window else 0
        q[t, 0] = 20.0 * rows[oldest] / scale / rows[oldest].square().sum()
        if nq > 1 and oldest > 0:
            q[t, 1] = 20.0 * rows[oldest - 1] / scale / rows[oldest - 1].square().sum()
    q, rows = q.bfloat16(), rows.bfloat16()
    want = _shared_row_reference(q, rows, dv, scale, window, past)
    n_pages = -(-total // 64)
    pool = _paged(rows[:, None], n_pages).reshape(n_pages, 64, d).cuda()
    out = torch.empty((T, nq * dv), dtype=torch.bfloat16, device="cuda")
    partial = torch.empty(T * nq * splits * (dv + 2), device="cuda") if splits > 1 else None
    ops.attention_latent(q.reshape(T, -1).cuda(), pool, out, ints(0, T), ints(past), ints(0, n_pages),
                         torch.arange(n_pages, dtype=torch.int32, device="cuda"), n_seqs=1, max_q_len=T, nq=nq, d=d, dv=dv,
                         page_size=64, ring_pages=0, window=window or 0, scale=scale, splits=splits, partial=partial)
    got = out.view(T, nq, dv).cpu().double()
    assert (got - want).abs().max() < 3e-2
    # the sharp head's output is (nearly) the row it asked for
    oldest = max(0, past + T - 1 - window + 1) if window else 0
    assert (got[-1, 0] - rows[oldest, :dv].double()).abs().max() < 6e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotary_tables_with_a_frequency_ramp(dtype, tmp_path_factory):
    model = engine("A", dtype, tmp_path_factory)
    position = model.decoder.layers[0].mixer.position
    want, magnitude = plain.yarn_frequencies(8, 10000.0, dict(zip(("factor", "original", "fast", "slow"), plain.YARN)))
    assert position.magnitude == pytest.approx(magnitude)
    assert position.inv_freq.cpu().double().tolist() == pytest.approx(want, rel=1e-6)
    pos = ints(0, 1, 77, 5000)
    cos, sin = torch.empty((4, 4), device="cuda"), torch.empty((4, 4), device="cuda")
    ops.rope_table(position.inv_freq, pos, cos, sin, position.magnitude)
    angle = pos.cpu().double()[:, None] * torch.tensor(want)[None, :]
    assert (cos.cpu() - magnitude * torch.cos(angle)).abs().max() < 2e-3     # fp32 angles at position 5000
    assert (cos[:3].cpu() - magnitude * torch.cos(angle[:3])).abs().max() < 2e-5
    assert (sin[:3].cpu() - magnitude * torch.sin(angle[:3])).abs().max() < 2e-5


# ----------------------------------------------------------------------------- whole models


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B", "C", "bare"])
def test_whole_prompts_and_their_first_tokens(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    cfg = CONFIGS[case][0]
    cache = model.make_cache(max_tokens=512, max_seqs=2)
    for n in (1, 2, 3, 150):
        tokens = plain.random_prompts(cfg, [n], n)[0]
        slot = cache.alloc()
        got = model.step(cache, [slot], [tokens], "all")
        cache.free(slot)
        if n >= 10 or dtype == "float32":
            close(got, expected(case, tokens), dtype, f"{case} whole prompt of {n}")
    cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "C"])
def test_residual_stream_after_every_layer(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    cfg = CONFIGS[case][0]
    tokens = plain.random_prompts(cfg, [40], 2)[0]
    want = plain.forward(cfg, weights_of(case), tokens, keep_layers=True)[1].float()
    seen, blocks = [], list(model.decoder.layers)
    originals = [block.forward for block in blocks]
    try:
        for block, original in zip(blocks, originals):
            def record(hidden, ctx, view, original=original):
                result = original(hidden, ctx, view)
                seen.append(hidden.clone())
                return result
            block.forward = record
        cache = model.make_cache(max_tokens=64, max_seqs=1)
        model.step(cache, [cache.alloc()], [tokens], "last")
    finally:
        for block, original in zip(blocks, originals):
            block.forward = original
    assert len(seen) == want.shape[0] == len(cfg["layers"])
    for run, (got, ref) in enumerate(zip(seen, want)):
        bound = 1e-4 if dtype == "float32" else 0.03 * float(ref.abs().max())
        assert float((got.cpu() - ref).abs().max()) < bound, run


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B", "C", "bare"])
def test_prompt_then_single_tokens_over_page_and_window_borders(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    cfg = CONFIGS[case][0]
    tokens = plain.random_prompts(cfg, [150], 4)[0]
    want = expected(case, tokens)
    cache = model.make_cache(max_tokens=192, max_seqs=1)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [tokens[:50]], "all")]
    rows += [model.step(cache, [slot], [[t]], "last") for t in tokens[50:]]         # past 64, 70, 100, 128
    close(torch.cat(rows), want, dtype, f"{case} decoded")
    cache.free(slot)
    slot = cache.alloc()                                                            # the same slot and pages again
    rows = [model.step(cache, [slot], [[t]], "last") for t in tokens[:80]]          # from the very first token
    close(torch.cat(rows), want[:80], dtype, f"{case} decoded from the first token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_portions_of_several_sizes_down_to_two_tokens(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    cfg = CONFIGS[case][0]
    tokens = plain.random_prompts(cfg, [200], 5)[0]
    want = expected(case, tokens)
    for sizes in ([2] * 40 + [120], [63, 2, 64, 1, 70], [7, 129, 64], [199, 1], [1, 2, 1, 196]):
        cache = model.make_cache(max_tokens=256, max_seqs=1)
        slot, at, rows = cache.alloc(), 0, []
        for size in sizes:
            rows.append(model.step(cache, [slot], [tokens[at:at + size]], "all"))
            at += size
        close(torch.cat(rows), want, dtype, f"{case} portions {sizes[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_unequal_batches_on_slots_and_pages_used_again(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    cfg = CONFIGS[case][0]
    requests = plain.random_prompts(cfg, [90, 1, 33, 70, 5, 129], 8)
    cache = model.make_cache(max_tokens=448, max_seqs=3)
    got = {r: [] for r in range(len(requests))}
    for batch in ([0, 1, 2], [3, 4, 5]):          # the second batch takes the slots and pages the first gave back
        slots = {r: cache.alloc() for r in batch}
        cut = {r: max(1, len(requests[r]) - 4 - 2 * (r % 3)) for r in batch}
        logits = model.step(cache, [slots[r] for r in batch], [requests[r][:cut[r]] for r in batch], "all")
        at = 0
        for r in batch:
            got[r].append(logits[at:at + cut[r]])
            at += cut[r]
        live = list(batch)
        while live:
            for r in [r for r in live if cut[r] == len(requests[r])]:
                cache.free(slots.pop(r))
                live.remove(r)
            if not live:
                break
            logits = model.step(cache, [slots[r] for r in live], [[requests[r][cut[r]]] for r in live], "last")
            for i, r in enumerate(live):
                got[r].append(logits[i:i + 1])
                cut[r] += 1
        cache.check()
    for r, tokens in enumerate(requests):
        if dtype == "float32":
            close(torch.cat(got[r]), expected(case, tokens), dtype, f"{case} batched request {r}")
    close(torch.cat([row for r in range(len(requests)) for row in got[r]]),
          torch.cat([expected(case, tokens) for tokens in requests]), dtype, f"{case} batched requests")


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_rows_do_not_depend_on_their_neighbours(dtype, tmp_path_factory):
    model = engine("A", dtype, tmp_path_factory)
    requests = plain.random_prompts(plain.TINY_A, [77, 12, 140], 6)
    cache = model.make_cache(max_tokens=512, max_seqs=4)
    alone = []
    for tokens in requests:
        slot = cache.alloc()
        alone.append(model.step(cache, [slot], [tokens], "all"))
        cache.free(slot)
    slots = [cache.alloc() for _ in requests]
    together = model.step(cache, slots, requests, "all")
    gap = (together - torch.cat(alone)).abs().max()
    assert float(gap) < (1e-5 if dtype == "float32" else 5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sharp_attention_finds_far_keys_in_prompts_and_in_decoding(dtype, tmp_path_factory):
    """Sharpened queries make both softmaxes pick single keys: anywhere among 700 positions in the attention layer,
    anywhere in a window of 300 in the latent layer, so a key that is lost, read from the wrong page or dropped one
    position early moves the logits.  float32 is held to the plain implementation; bfloat16 (whose rounded scores
    such a scale magnifies) to its own whole-prompt run, which the decoded run must repeat from the cache."""
    model = engine("sharp", dtype, tmp_path_factory)
    tokens = plain.random_prompts(plain.SHARP, [700], 9)[0]
    cache = model.make_cache(max_tokens=1536, max_seqs=2)
    whole = cache.alloc()
    whole_logits = model.step(cache, [whole], [tokens], "all")
    want = expected("sharp", tokens) if dtype == "float32" else whole_logits
    if dtype == "float32":
        close(whole_logits, want, dtype, "sharp whole", atol=3e-4)      # the effects looked for below are above 2e-2
    decoded = cache.alloc()
    rows = [model.step(cache, [decoded], [tokens[:500]], "all")]
    rows += [model.step(cache, [decoded], [[t]], "last") for t in tokens[500:]]
    close(torch.cat(rows), want, dtype, "sharp decoded", atol=3e-4)
    if dtype == "float32":
        weights = weights_of("sharp")
        # the plain logits really depend on keys hundreds of positions back ...
        near_only = plain.forward(plain.SHARP, weights, tokens[500:]).float()
        assert float((near_only[-20:] - want[-20:]).abs().max()) > 0.05
        # ... on the window's exact size ...
        narrower = copy.deepcopy(plain.SHARP)
        narrower["layers"][1]["mixer"]["mask"]["size"] = 299
        assert float((plain.forward(narrower, weights, tokens).float()[300:] - want[300:]).abs().max()) > 0.02
        # ... on the attention layer seeing every earlier key ...
        windowed = copy.deepcopy(plain.SHARP)
        windowed["layers"][0]["mixer"]["mask"] = {"size": 400}
        assert float((plain.forward(windowed, weights, tokens).float()[400:] - want[400:]).abs().max()) > 0.02
        # ... and on the first tokens of the sequence
        later = plain.forward(plain.SHARP, weights, tokens[1:]).float()
        assert float((later[-100:] - want[-100:]).abs().max()) > 0.02


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompts_are_cut_and_go_round_the_ring(dtype, tmp_path_factory):
    """A prompt of 700 tokens on a cache whose passes take 256 tokens of a sequence: three portions, the third one
    written over the ring's oldest pages, beside a short request in the same step."""
    model = engine("C", dtype, tmp_path_factory)
    long, short = plain.random_prompts(plain.TINY_C, [700, 40], 12)
    cache = model.make_cache(max_tokens=1024, max_seqs=2)
    assert cache.max_step_tokens == 256 and any(0 < group.ring_pages * 64 < 700 for group in cache.kv_groups)
    slots = [cache.alloc(), cache.alloc()]
    got = model.step(cache, slots, [long, short], "all")
    close(got[:700], expected("C", long), dtype, "long prompt in portions")
    close(got[700:], expected("C", short), dtype, "short prompt beside it")
    more = plain.random_prompts(plain.TINY_C, [30], 13)[0]
    rows = [model.step(cache, slots[:1], [[t]], "last") for t in more]
    close(torch.cat(rows), expected("C", long + more)[700:], dtype, "single tokens after the long prompt")


def test_long_decoding_wraps_the_ring_of_a_windowed_cache(tmp_path_factory):
    """Windows of 70 and 40 on shared rows keep a ring of a few pages per sequence; 700 single-token steps go round it."""
    model = engine("A", "float32", tmp_path_factory)
    tokens = plain.random_prompts(plain.TINY_A, [720], 11)[0]
    want = expected("A", tokens)
    cache = model.make_cache(max_tokens=768, max_seqs=1, max_step_tokens=16)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [tokens[:20]], "all")]
    rows += [model.step(cache, [slot], [[t]], "last") for t in tokens[20:]]
    close(torch.cat(rows), want, "float32", "long decoding", atol=1e-4)
    assert any(group.ring_pages and 720 > group.ring_pages * 64 for group in cache.kv_groups)


def test_decode_steps_are_captured_as_graphs(tmp_path_factory):
    assert engine("A", "bfloat16", tmp_path_factory).decoder.graph_safe


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype, tmp_path_factory):
    for case in ("A", "B"):
        model = engine(case, dtype, tmp_path_factory)
        cfg = CONFIGS[case][0]
        prompts = plain.random_prompts(cfg, [9, 30, 3], 10)
        weights = weights_of(case)
        for use_graphs in (False, True):              # the step function, then the captured decode steps
            result = model.generate(prompts, max_new_tokens=6, use_graphs=use_graphs)
            for prompt, produced in zip(prompts, result.generated_ids):
                assert len(produced) == 6
                ids = list(prompt)
                for token in produced:
                    logits = plain.forward(cfg, weights, ids)[-1]
                    slack = 1e-4 if dtype == "float32" else 0.05 * float(logits.abs().max())
                    assert float(logits.max() - logits[token]) < slack, "the generated token is not the plain argmax"
                    ids.append(token)


def test_command_line_writes_a_random_model_and_generates_from_it(tmp_path):
    cfg = plain.TINY_B
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    root = Path(__file__).resolve().parent.parent
    run = lambda *a: subprocess.run([sys.executable, "-m", "ondeviceinfer_b200", *a], cwd=root, text=True,
                                    capture_output=True, timeout=600)
    made = run("random-model", "--config", str(tmp_path / "config.json"), "--seed", "3", "--out", str(tmp_path / "model"))
    assert made.returncode == 0, made.stderr
    done = run("generate", "--model", str(tmp_path / "model"), "--prompt-ids", "5,9,2,40,7", "--dtype", "float32",
               "--max-new-tokens", "4", "--warmup-runs", "0", "--repeats", "1", "--output", str(tmp_path / "report.json"))
    assert done.returncode == 0, done.stderr
    report = json.loads((tmp_path / "report.json").read_text())
    from ondeviceinfer_b200.weights import SafetensorsSource
    source = SafetensorsSource(tmp_path / "model")
    weights = {n: source.fetch(n) for n in source.stored()}
    ids = [5, 9, 2, 40, 7]
    for token in report["measurements"][0]["output_token_ids"]:
        logits = plain.forward(cfg, weights, ids)[-1]
        assert float(logits.max() - logits[token]) < 1e-4
        ids.append(token)
    assert len(ids) == 9


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(12))
def test_models_of_random_odd_sizes(seed, dtype, tmp_path):
    """Configurations drawn from odd sizes: a prompt, then single tokens, then a portion, on a cache that a shorter
    request used before."""
    cfg = plain.random_config(seed)
    weights = plain.random_weights(cfg, 300 + seed)
    model = odi.load_resident_model(write_model_folder(tmp_path / "model", cfg, weights), dtype=dtype)
    tokens = plain.random_prompts(cfg, [150], seed)[0]
    want = plain.forward(cfg, weights, tokens).float()
    cache = model.make_cache(max_tokens=192, max_seqs=1)
    slot = cache.alloc()
    model.step(cache, [slot], [tokens[:37]], "none")
    cache.free(slot)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [tokens[:100]], "all")]
    rows += [model.step(cache, [slot], [[t]], "last") for t in tokens[100:130]]
    rows.append(model.step(cache, [slot], [tokens[130:]], "all"))
    close(torch.cat(rows), want, dtype, f"random sizes {seed}: {json.dumps(cfg)[:300]}")

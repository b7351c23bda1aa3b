"""The Lemesun design in the engine against its plain restatement (``plain_lemesun``): each mechanism alone, whole
prompts, token-by-token decoding, portions, batches of unequal requests, slots and pages used again, far keys and
page borders, the first tokens, long decoding, sizes of one, and greedy generation through ``generate``.

float32 is compared strictly.  In bfloat16 a router whose two best choices lie closer than the rounding may send a
token to another expert than the plain implementation does, which changes that row by more than rounding; so the
bfloat16 comparisons of models with routed experts hold nine rows in ten to the bfloat16 bound, and every row of
models without (``close``)."""

import copy
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import ondeviceinfer_b200 as odi
import plain_lemesun as plain
from helpers import assert_logits_close, write_model_folder
from ondeviceinfer_b200.kernels import ops

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
CONFIGS = {"A": (plain.TINY_A, 21), "B": (plain.TINY_B, 22), "latent": (plain.ONLY_LATENT, 23),
           "delta": (plain.ONLY_DELTA, 24), "sharp": (plain.ONLY_LATENT, 25), "lanes64": (plain.LATENT_64, 26)}
_MODELS, _PLAIN = {}, {}


def weights_of(case):
    cfg, seed = CONFIGS[case]
    return plain.random_weights(cfg, seed, sharpen=6.0 if case == "sharp" else 1.0)


def engine(case, dtype, tmp_path_factory):
    if (case, dtype) not in _MODELS:
        folder = write_model_folder(tmp_path_factory.mktemp(f"lemesun_{case}"), CONFIGS[case][0], weights_of(case))
        _MODELS[(case, dtype)] = odi.load_resident_model(folder, dtype=dtype)
    return _MODELS[(case, dtype)]


def expected(case, tokens):
    key = (case, tuple(tokens))
    if key not in _PLAIN:
        _PLAIN[key] = plain.forward(CONFIGS[case][0], plain.widened(weights_of(case)), list(tokens)).float()
    return _PLAIN[key]


def close(actual, reference, dtype, what, routed):
    """float32: the helpers' strict comparison.  bfloat16: the error of a row relative to the row's size.  Without
    routed experts its median over the rows is at most 1.5e-2, nine rows in ten are within 5e-2 and every row within
    1.5e-1 (a row of small logits has a large relative error).  With them a row may have
    gone to another expert, and the test weights are large so that every mechanism shows: median at most 4e-2,
    four rows in five at most 1e-1 (comparisons of fewer than ten rows are made together with others)."""
    if dtype == "float32":
        # the recurrent state sums over every earlier token of the sequence: sums of about a thousand terms
        assert_logits_close(actual, reference, dtype, what, longest_sum=1024)
        return
    actual, reference = actual.float().cpu(), reference.float().cpu()
    assert actual.shape == reference.shape and torch.isfinite(actual).all(), what
    error = (actual - reference).norm(dim=-1) / reference.norm(dim=-1).clamp_min(1e-6)
    ranked = error.sort().values
    if routed:
        assert len(ranked) >= 10, "too few rows for a comparison by rank"
        median_bound, high_bound, high, worst_bound = 4e-2, 1e-1, ranked[int(0.8 * len(ranked))], float("inf")
    else:
        high = ranked[int(0.9 * len(ranked))] if len(ranked) >= 10 else ranked[-1]
        median_bound, high_bound, worst_bound = 1.5e-2, 5e-2, 1.5e-1
    assert float(ranked[-1]) <= worst_bound, f"{what}: bfloat16 row error {float(ranked[-1]):.3e}"
    assert float(error.median()) <= median_bound and float(high) <= high_bound, \
        f"{what}: bfloat16 row errors median {float(error.median()):.3e}, high {float(high):.3e}, max {float(ranked[-1]):.3e}"


def routed(case):
    return any(layer.get("mlp") for layer in CONFIGS[case][0]["layers"])


# ----------------------------------------------------------------------------- kernels against plain functions


def test_offset_norm_scales_in_fp32():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(7, 50, generator=g) * 3
    w = torch.randn(50, generator=g) * 0.2
    for dtype in (torch.float32, torch.bfloat16):
        out = torch.empty((7, 50), dtype=dtype, device="cuda")
        ops.rmsnorm_scaled(x.cuda(), (1.0 + w).cuda(), 1e-5, out)
        want = plain.offset_norm(x.double(), w.double(), 1e-5).float()
        if dtype == torch.bfloat16:
            assert torch.equal(out.cpu(), want.to(torch.bfloat16)) or (out.float().cpu() - want).abs().max() < 2e-2
        else:
            assert (out.cpu() - want).abs().max() < 1e-5
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
    out = torch.empty((3, 50), dtype=torch.float32, device="cuda")
    ops.rmsnorm_scaled(x.cuda(), (1.0 + w).cuda(), 1e-5, out, rows)
    assert torch.equal(out[0], out[2]) and (out[1].cpu() - plain.offset_norm(x[0], w, 1e-5)).abs().max() < 1e-5


@pytest.mark.parametrize("experts,identity,top,groups,keep", [(6, 2, 3, 4, 2), (3, 0, 1, 1, 1), (40, 8, 6, 8, 3),
                                                             (5, 1, 2, 2, 2), (30, 0, 4, 3, 1)])
def test_router_chooses_like_the_plain_router(experts, identity, top, groups, keep):
    g = torch.Generator().manual_seed(experts)
    n_all, T = experts + identity, 300
    logits = torch.randn(T, n_all, generator=g) * 2
    correction = torch.randn(n_all, generator=g) * 0.1          # may push a choice score below zero
    f = {"router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}}
    # the plain router takes h and a router matrix: an identity matrix makes the logits themselves the input
    want_ids, want_w = plain.route(logits, {"r.router": torch.eye(n_all), "r.correction": correction}, "r.", f)
    ids = torch.empty((T, top), dtype=torch.int32, device="cuda")
    weights = torch.empty((T, top), dtype=torch.float32, device="cuda")
    ops.moe_route(logits.cuda(), correction.cuda(), ids, weights, n_groups=groups, keep=keep)
    assert torch.equal(ids.cpu().long(), want_ids)
    assert (weights.cpu() - want_w).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [1, 5, 700])
@pytest.mark.parametrize("K,F", [(44, 36), (96, 40)])         # element by element; eight elements at a time
def test_routed_products_against_a_loop_over_pairs(dtype, tokens, K, F):
    g = torch.Generator().manual_seed(tokens)
    E, ident, top = 5, 2, 3
    x = torch.randn(tokens, K, generator=g).to(dtype)
    w_gu = (torch.randn(E, 2 * F, K, generator=g) / K ** 0.5).to(dtype)
    w_d = (torch.randn(E, K, F, generator=g) / F ** 0.5).to(dtype)
    ids = torch.stack([torch.randperm(E + ident, generator=g)[:top] for _ in range(tokens)]).int()
    weights = torch.rand(tokens, top, generator=g)
    # aligned sizes and few rows per expert: the form that streams the weights through registers
    table = ops.RoutingTable(tokens, top, E, "cuda", few_rows_ok=ops.grouped_few_rows_ok((K, F), dtype))
    assert table.tm == (4 if K % 8 == 0 and tokens <= 5 else 16 if tokens <= 5 else 64)
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    ops.moe_group(ids.cuda(), counts, table)
    assert int(counts.abs().sum()) == 0                    # left clean for the next step
    act = torch.empty((tokens * top, F), dtype=dtype, device="cuda")
    ops.grouped_gemm_routed(x.cuda(), w_gu.cuda(), act, table, gather=True, epi=ops.GROUPED_GATED_CLAMP, limit=0.8, alpha=1.702)
    out = torch.zeros((tokens * top, K), dtype=torch.float32, device="cuda")
    ops.grouped_gemm_routed(act, w_d.cuda(), out, table, gather=False, epi=ops.GROUPED_STORE_F32)
    residual = torch.zeros((tokens, K), dtype=torch.float32, device="cuda")
    ops.moe_combine(residual, out, x.cuda(), ids.cuda(), weights.cuda(), table)
    want = torch.zeros(tokens, K, dtype=torch.float64)
    for t in range(tokens):
        for k in range(top):
            e = int(ids[t, k])
            h = x[t:t + 1].double()
            y = h if e >= E else plain.clamped_expert(h, w_gu[e, :F].double(), w_gu[e, F:].double(), w_d[e].double(), 0.8)
            want[t] += float(weights[t, k]) * y[0]
    tol = 1e-4 if dtype == torch.float32 else 4e-2
    assert (residual.cpu().double() - want).abs().max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,K,N,M,a_gap,c_gap", [(3, 10, 7, 37, 2, 4), (4, 16, 12, 3, 8, 4), (4, 16, 12, 7, 8, 4),
                                                     (2, 24, 70, 130, 8, 2),
                                                     (3, 264, 20, 7, 8, 4), (4, 512, 40, 8, 0, 8), (2, 256, 9, 5, 8, 3),   # five to eight rows, long inner size: two row tiles of the form for few rows
                                                     (2400, 16, 320, 3, 8, 4)])     # bf16: more than 32 items a warp
def test_products_per_head(dtype, heads, K, N, M, a_gap, c_gap):
    g = torch.Generator().manual_seed(3)
    a = torch.randn(M, heads * (K + a_gap) + 8, generator=g).to(dtype)     # a head's K lanes lie K + a_gap apart
    w = torch.randn(heads, N, K, generator=g).to(dtype)
    c = torch.zeros((M, heads * (N + c_gap)), dtype=dtype, device="cuda")
    ops.grouped_gemm_heads(a.cuda(), w.cuda(), c, a_col=0, a_stride=K + a_gap, c_col=0, c_stride=N + c_gap, K=K)
    for h in range(heads):
        want = a[:, h * (K + a_gap):h * (K + a_gap) + K].double() @ w[h].double().T
        got = c[:, h * (N + c_gap):h * (N + c_gap) + N].cpu().double()
        bound = 1e-4 if dtype == torch.float32 else 2e-2 + 1e-2 * want.abs()      # one rounding of the result
        assert ((got - want).abs() <= bound).all()
        assert float(c[:, h * (N + c_gap) + N:(h + 1) * (N + c_gap)].abs().max()) == 0.0       # lanes between heads untouched


# ----------------------------------------------------------------------------- each mixer alone, whole models


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["latent", "delta", "A", "B", "lanes64"])
def test_whole_prompts_and_first_tokens(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    cache = model.make_cache(max_tokens=512, max_seqs=2)
    got, want = [], []
    for r, tokens in enumerate(plain.random_prompts(CONFIGS[case][0], [1, 2, 3, 70, 130], 5)):
        slot = cache.alloc()
        got.append(model.step(cache, [slot], [tokens], "all"))
        want.append(expected(case, tokens))
        if dtype == "float32":
            close(got[-1], want[-1], dtype, f"{case} whole prompt {r}", routed(case))
        cache.free(slot)
    close(torch.cat(got), torch.cat(want), dtype, f"{case} whole prompts", routed(case))
    cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["latent", "delta", "A", "B", "lanes64"])
def test_prefill_then_long_decoding_over_page_borders(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    tokens = plain.random_prompts(CONFIGS[case][0], [200], 6)[0]
    cache = model.make_cache(max_tokens=256, max_seqs=1)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [tokens[:60]], "all")]                 # then positions 60..199 one by one:
    rows += [model.step(cache, [slot], [[t]], "last") for t in tokens[60:]]  # over the borders at 64, 128 and 192
    close(torch.cat(rows), expected(case, tokens), dtype, f"{case} long decoding", routed(case))
    cache.free(slot)
    # from the very first token, one by one
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [[t]], "last") for t in tokens[:12]]
    close(torch.cat(rows), expected(case, tokens)[:12], dtype, f"{case} from the first token", routed(case))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B"])
def test_portions_of_several_sizes(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    tokens = plain.random_prompts(CONFIGS[case][0], [150], 7)[0]
    cache = model.make_cache(max_tokens=256, max_seqs=1)
    for cuts in ([2, 2, 3, 57, 1, 64, 21], [63, 2, 64, 2, 19], [1, 1, 2, 146]):
        slot = cache.alloc()
        rows, at = [], 0
        for n in cuts:
            rows.append(model.step(cache, [slot], [tokens[at:at + n]], "all"))
            at += n
        assert at == len(tokens)
        close(torch.cat(rows), expected(case, tokens), dtype, f"{case} portions {cuts}", routed(case))
        cache.free(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B"])
def test_unequal_batches_and_slots_used_again(case, dtype, tmp_path_factory):
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
            close(torch.cat(got[r]), expected(case, tokens), dtype, f"{case} batched request {r}", routed(case))
    close(torch.cat([row for r in range(len(requests)) for row in got[r]]),
          torch.cat([expected(case, tokens) for tokens in requests]), dtype, f"{case} batched requests", routed(case))


@pytest.mark.parametrize("dtype", DTYPES)
def test_sharp_attention_finds_far_keys_in_prompts_and_in_decoding(dtype, tmp_path_factory):
    """Queries six times larger make the softmax pick single keys, hundreds of positions back as often as near:
    a key that is lost, read from the wrong page or seen one position too early moves the logits.  float32 is held
    to the plain implementation; bfloat16 (whose rounded scores such queries magnify) to its own whole-prompt run,
    which the decoded run must repeat from the cache."""
    model = engine("sharp", dtype, tmp_path_factory)
    tokens = plain.random_prompts(plain.ONLY_LATENT, [330], 9)[0]
    cache = model.make_cache(max_tokens=832, max_seqs=2)
    whole = cache.alloc()
    whole_logits = model.step(cache, [whole], [tokens], "all")
    want = expected("sharp", tokens) if dtype == "float32" else whole_logits
    if dtype == "float32":
        close(whole_logits, want, dtype, "sharp whole", False)
    decoded = cache.alloc()
    rows = [model.step(cache, [decoded], [tokens[:250]], "all")]
    rows += [model.step(cache, [decoded], [[t]], "last") for t in tokens[250:]]      # past the border at 256
    close(torch.cat(rows), want, dtype, "sharp decoded", False)
    # the plain logits really depend on far keys: without the first 200 positions the last rows differ
    if dtype == "float32":
        near_only = plain.forward(plain.ONLY_LATENT, plain.widened(weights_of("sharp")), tokens[200:]).float()
        assert float((near_only[-20:] - want[-20:]).abs().max()) > 0.05


def test_decode_steps_are_captured_as_graphs(tmp_path_factory):
    assert engine("A", "bfloat16", tmp_path_factory).decoder.graph_safe


def test_greedy_generation_through_the_entry_point(tmp_path_factory):
    model = engine("A", "float32", tmp_path_factory)
    cfg = CONFIGS["A"][0]
    prompts = plain.random_prompts(cfg, [9, 30, 3], 10)
    weights = plain.widened(weights_of("A"))
    for use_graphs in (False, True):              # the step function, then the captured decode steps
        result = model.generate(prompts, max_new_tokens=6, use_graphs=use_graphs)
        for prompt, produced in zip(prompts, result.generated_ids):
            assert len(produced) == 6
            ids = list(prompt)
            for token in produced:
                logits = plain.forward(cfg, weights, ids)[-1]
                assert float(logits.max() - logits[token]) < 1e-4, "the generated token is not the plain argmax"
                ids.append(token)


def test_command_line_writes_a_random_model_and_generates_from_it(tmp_path):
    """``random-model`` needs the two bottleneck widths in the configuration (no tensors give them yet); the folder it
    writes loads like any other, and ``generate`` produces the plain implementation's greedy tokens."""
    cfg = copy.deepcopy(plain.TINY_B)
    for layer in cfg["layers"]:
        if layer["type"] == "channel_delta":
            layer["mixer"].update(decay_rank=5, gate_rank=7)
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
    weights = {n: source.fetch(n).double() for n in source.stored()}
    ids = [5, 9, 2, 40, 7]
    for token in report["measurements"][0]["output_token_ids"]:
        logits = plain.forward(cfg, weights, ids)[-1]
        assert float(logits.max() - logits[token]) < 1e-4
        ids.append(token)
    assert len(ids) == 9


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(8))
def test_models_of_random_odd_sizes(seed, dtype, tmp_path):
    """Configurations drawn from odd sizes: a prompt, then single tokens, then a portion, on a cache that a shorter
    request used before."""
    cfg = plain.random_config(seed)
    weights = plain.random_weights(cfg, 300 + seed)
    model = odi.load_resident_model(write_model_folder(tmp_path / "model", cfg, weights), dtype=dtype)
    tokens = plain.random_prompts(cfg, [150], seed)[0]
    want = plain.forward(cfg, plain.widened(weights), tokens).float()
    cache = model.make_cache(max_tokens=192, max_seqs=1)
    slot = cache.alloc()
    model.step(cache, [slot], [tokens[:37]], "none")
    cache.free(slot)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [tokens[:100]], "all")]
    rows += [model.step(cache, [slot], [[t]], "last") for t in tokens[100:130]]
    rows.append(model.step(cache, [slot], [tokens[130:]], "all"))
    has_experts = any(layer.get("mlp") for layer in cfg["layers"])
    close(torch.cat(rows), want, dtype, f"random sizes {seed}: {json.dumps(cfg)[:300]}", has_experts)

"""The Zigivik configuration without a GPU: reading and writing back, declared tensors, the order of executions and
whose cache rows each reads, what the cache keeps for shared rows, the frequency ramp, refused configurations."""

import copy
import math

import pytest
import torch

import plain_zigivik as plain
from ondeviceinfer_b200.cache import KVNeed, SequenceCache, StateNeed
from ondeviceinfer_b200.config.specs import (CappedAttentionSpec, LatentAttentionSpec, ParallelBlockSpec,
                                             PolyNormMLPSpec)
from ondeviceinfer_b200.config.zigivik import ZigivikConfig
from ondeviceinfer_b200.engine.model import DecoderModel
from ondeviceinfer_b200.parts.position import ramped_frequencies
from ondeviceinfer_b200.registry import config_from_dict

CONFIGS = {"A": plain.TINY_A, "B": plain.TINY_B, "C": plain.TINY_C, "bare": plain.NO_CONV, "sharp": plain.SHARP}


@pytest.mark.parametrize("case", sorted(CONFIGS))
def test_reads_and_writes_back(case):
    cfg = CONFIGS[case]
    config = config_from_dict(cfg)
    assert isinstance(config, ZigivikConfig) and config.to_dict() == cfg
    assert config_from_dict(config.to_dict()) == config


@pytest.mark.parametrize("case", sorted(CONFIGS))
def test_declares_the_designs_tensors(case):
    cfg = CONFIGS[case]
    model = DecoderModel(config_from_dict(cfg).to_plan())
    declared = {d.name: tuple(d.shape) for d in model.tensor_decls()}
    assert declared == plain.tensor_shapes(cfg)


@pytest.mark.parametrize("seed", range(12))
def test_random_configurations_declare_their_tensors(seed):
    cfg = plain.random_config(seed)
    model = DecoderModel(config_from_dict(cfg).to_plan())
    assert {d.name: tuple(d.shape) for d in model.tensor_decls()} == plain.tensor_shapes(cfg)


def test_plan_follows_the_layer_list():
    plan = config_from_dict(plain.TINY_A).to_plan()
    assert [(e.layer, e.cache_from) for e in plan.order] == [(0, None), (1, None), (2, 0), (3, None), (4, None)]
    kinds = [type(block.mixer) for block in plan.layers]
    assert kinds == [LatentAttentionSpec, CappedAttentionSpec, LatentAttentionSpec, CappedAttentionSpec, LatentAttentionSpec]
    assert all(isinstance(block, ParallelBlockSpec) and block.residual_mult == 0.7 and block.conv_taps == 4 for block in plan.layers)
    assert plan.layers[2].ffn is None and isinstance(plan.layers[0].ffn, PolyNormMLPSpec)
    reader, writer, attention = plan.layers[2].mixer, plan.layers[0].mixer, plan.layers[1].mixer
    assert not reader.own_kv and writer.own_kv and reader.gated and writer.q_rank == 20
    # the rows are kept for the wider of the two windows; each layer masks with its own
    assert (writer.window, reader.window, writer.cache_window, reader.cache_window) == (70, 40, 70, 70)
    assert attention.sink and attention.values_are_keys and attention.window is None and attention.position.interleaved
    assert attention.position.rotary_dim == 8 and plan.layers[3].mixer.window == 50
    assert plan.layers[4].mixer.window is None and plan.layers[4].mixer.position.index_ramp is None
    assert plan.layers[0].mixer.position.index_ramp == plain.YARN and not plan.layers[0].mixer.position.interleaved
    assert plan.embedding.norm is not None and plan.embedding.norm.scalar_weight and plan.final_norm.scalar_weight


def test_a_reader_without_a_window_keeps_every_row():
    plan = config_from_dict(plain.TINY_B).to_plan()
    writer, reader = plan.layers[1].mixer, plan.layers[2].mixer
    assert writer.window == 33 and reader.window is None
    assert writer.cache_window is None and reader.cache_window is None


def test_cache_shares_rows_but_not_state():
    model = DecoderModel(config_from_dict(plain.TINY_A).to_plan())
    needs = [tuple(n for n in model.layers[e.layer].cache_needs() if e.cache_from is None or not isinstance(n, KVNeed))
             for e in model.plan.order]
    assert [sum(isinstance(n, StateNeed) for n in entry) for entry in needs] == [1] * 5
    assert [sum(isinstance(n, KVNeed) for n in entry) for entry in needs] == [1, 1, 0, 1, 1]
    cache = SequenceCache(needs, [e.cache_from for e in model.plan.order], dtype=torch.float32, device="cpu",
                          max_tokens=256, max_seqs=3, max_step_tokens=64)
    reader, writer = cache.view(2), cache.view(0)
    assert reader.keys.data_ptr() == writer.keys.data_ptr() and not reader.writes_kv and writer.writes_kv
    assert reader.states[-1].data_ptr() != writer.states[-1].data_ptr()
    assert reader.states[-1].shape == (3 + 1, 3, 64)
    states = {cache.view(e).states[-1].data_ptr() for e in range(5)}
    assert len(states) == 5


def test_an_entry_that_reads_anothers_rows_may_not_ask_for_its_own():
    with pytest.raises(ValueError):
        SequenceCache([(KVNeed(1, 8),), (KVNeed(1, 8),)], [None, 0], dtype=torch.float32, device="cpu", max_tokens=64,
                      max_seqs=1)


@pytest.mark.parametrize("dims,base,ramp", [(8, 10000.0, plain.YARN), (16, 64, (4.0, 64, 16.0, 2.0)), (6, 100.0, (3.0, 40, 6.0, 1.0)),
                                            (32, 1e6, (16.0, 4096, 32.0, 1.0)), (4, 50.0, (2.0, 10, 1000.0, 900.0))])
def test_frequency_ramp_against_the_plain_formula(dims, base, ramp):
    exact = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    got, magnitude = ramped_frequencies(exact, float(base), dims, ramp)
    want, want_magnitude = plain.yarn_frequencies(dims, float(base), dict(zip(("factor", "original", "fast", "slow"), ramp)))
    assert got == pytest.approx(want, rel=1e-12) and magnitude == pytest.approx(want_magnitude)
    assert magnitude == pytest.approx(0.1 * math.log(ramp[0]) + 1.0)
    # the fastest pairs keep their frequency, the slowest are divided by the factor (where the ramp reaches them)
    assert got[0] <= exact[0] and all(g <= e * (1 + 1e-12) and g >= e / ramp[0] * (1 - 1e-12) for g, e in zip(got, exact))


def _broken(change):
    cfg = copy.deepcopy(plain.TINY_A)
    change(cfg)
    return cfg


@pytest.mark.parametrize("change", [
    lambda c: c["layers"][2]["mixer"].update(kv_from=2),                    # itself
    lambda c: c["layers"][2]["mixer"].update(kv_from=1),                    # an attention layer
    lambda c: c["layers"][2]["mixer"].update(kv_from=4),                    # a later layer
    lambda c: c["layers"][2]["mixer"].update(kv_rank=16),                   # rows of another width
    lambda c: c["layers"][2]["mixer"]["rot"].update(base=5.0),              # another rotation
    lambda c: c["layers"][1].update(type="convolution"),
    lambda c: c["layers"][1]["mixer"].update(vdim=24),                      # values are keys: one width
    lambda c: c["layers"][0]["mlp"].update(kind="moe"),
    lambda c: c["canon"].update(taps=0),
    lambda c: c.pop("vocab"),
])
def test_refused_configurations(change):
    with pytest.raises((ValueError, KeyError)):
        config_from_dict(_broken(change))


def test_a_reader_of_a_reader_is_refused():
    cfg = copy.deepcopy(plain.TINY_A)
    cfg["layers"][4] = copy.deepcopy(cfg["layers"][2])
    cfg["layers"][4]["mixer"]["kv_from"] = 2
    with pytest.raises(ValueError):
        config_from_dict(cfg)

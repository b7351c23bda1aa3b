"""The Losivik configuration without a GPU: reading and writing back, declared tensors, the plan, what the cache keeps
for a window with kept first positions (pinned pages in front of a ring), refused configurations."""

import copy

import pytest
import torch

import plain_losivik as plain
from ondeviceinfer_b200.cache import KVNeed, SequenceCache, StateNeed, pages_for
from ondeviceinfer_b200.config.losivik import LosivikConfig
from ondeviceinfer_b200.config.specs import (CappedAttentionSpec, ClampedGatedMLPSpec, LatentAttentionSpec, RoutedExpertsSpec,
                                             ScaledParallelBlockSpec, SideBySideMixersSpec, StateSpaceSpec, TokenSideInputSpec)
from ondeviceinfer_b200.engine.model import DecoderModel
from ondeviceinfer_b200.registry import config_from_dict

CONFIGS = {"A": plain.TINY_A, "B": plain.TINY_B, "C": plain.TINY_C, "D": plain.TINY_D, "E": plain.TINY_E, "sharp": plain.SHARP}


@pytest.mark.parametrize("case", sorted(CONFIGS))
def test_reads_and_writes_back(case):
    cfg = CONFIGS[case]
    config = config_from_dict(cfg)
    assert isinstance(config, LosivikConfig) and config.to_dict() == cfg
    assert config_from_dict(config.to_dict()) == config


@pytest.mark.parametrize("case", sorted(CONFIGS))
def test_declares_the_designs_tensors(case):
    cfg = CONFIGS[case]
    model = DecoderModel(config_from_dict(cfg).to_plan())
    assert {d.name: tuple(d.shape) for d in model.tensor_decls()} == plain.tensor_shapes(cfg)
    assert set(plain.random_weights(cfg, 1)) == set(plain.tensor_shapes(cfg))


@pytest.mark.parametrize("seed", range(12))
def test_random_configurations_declare_their_tensors(seed):
    cfg = plain.random_config(seed)
    model = DecoderModel(config_from_dict(cfg).to_plan())
    assert {d.name: tuple(d.shape) for d in model.tensor_decls()} == plain.tensor_shapes(cfg)


def test_plan_follows_the_layer_list():
    plan = config_from_dict(plain.TINY_A).to_plan()
    assert [(e.layer, e.cache_from) for e in plan.order] == [(0, None), (1, None), (2, None), (3, None)]
    assert all(isinstance(block, ScaledParallelBlockSpec) for block in plan.layers)
    kinds = [type(block.mixer) for block in plan.layers]
    assert kinds == [SideBySideMixersSpec, LatentAttentionSpec, LatentAttentionSpec, SideBySideMixersSpec]
    pair = plan.layers[0].mixer
    assert isinstance(pair.left, CappedAttentionSpec) and isinstance(pair.right, StateSpaceSpec)
    assert (pair.left_scale, pair.right_scale) == (0.7, 1.2)
    assert (pair.left.num_heads, pair.left.num_kv_heads, pair.left.head_dim, pair.left.value_dim) == (6, 2, 32, 48)
    assert (pair.left.window, pair.left.keep_first, pair.left.scale) == (40, 5, 0.2) and pair.left.unit_norm_eps == 1e-5
    assert pair.left.has("q_norm") and pair.left.has("k_norm") and not pair.left.sink and pair.left.softcap is None
    assert (pair.right.num_heads, pair.right.head_dim, pair.right.state_dim, pair.right.groups, pair.right.conv_taps,
            pair.right.norm_groups) == (6, 16, 24, 3, 4, 3)
    assert plan.layers[3].mixer.left.window is None and plan.layers[3].mixer.left.keep_first == 0
    latent = plan.layers[1].mixer
    assert latent.rot_dim == 0 and latent.gated and latent.gate_per_head and latent.window == 70 and latent.q_rank is None
    assert plan.layers[2].mixer.window is None and plan.layers[2].ffn is None and plan.layers[2].ffn_norm is None
    experts, dense = plan.layers[0].ffn, plan.layers[1].ffn
    assert isinstance(experts, RoutedExpertsSpec) and isinstance(dense, ClampedGatedMLPSpec)
    assert (experts.scoring, experts.expert_form, experts.weight_on_input, experts.top_k, experts.num_experts,
            experts.shared_size, experts.has_correction) == ("sigmoid", "relu2", True, 2, 6, 24, False)
    assert (dense.limit, dense.alpha, dense.intermediate_size) == (2.0, 1.702, 72) and dense.has("down_bias")
    side = plan.layers[3].after
    assert isinstance(side, TokenSideInputSpec) and (side.dim, side.col, side.table_width) == (8, 24, 32)
    assert plan.embedding.scale == 1.7 and plan.embedding.sinusoid_base == 10000.0 and plan.head.weight_name is None
    assert plan.final_norm.weight_offset == 1.0 and plan.final_norm.scale_in_fp32
    bare = config_from_dict(plain.TINY_C).to_plan()
    assert bare.layers[0].after is None and bare.embedding.scale == 1.0


def test_a_layer_without_a_feed_forward_may_still_store_its_norm():
    plan = config_from_dict(plain.TINY_A).to_plan()
    assert set(plan.ignored_tensors) == {"l2.norm2", "l2.ls2"}


def test_cache_needs_of_both_mixers_side_by_side():
    model = DecoderModel(config_from_dict(plain.TINY_C).to_plan())
    needs = model.layers[0].cache_needs()
    assert needs[0] == KVNeed(2, 16, 30, value_dim=32, keep_first=70)
    assert [type(n) for n in needs[1:]] == [StateNeed, StateNeed] and needs[1].shape == (4, 16, 8)
    assert needs[2].shape == (2, 4 * 8 + 2 * 2 * 16)
    assert model.layers[1].cache_needs() == (KVNeed(1, 16, 65, value_plane=False),)
    one_tap = copy.deepcopy(plain.TINY_C)
    one_tap["layers"][0]["mixer"]["right"]["conv"] = 1
    assert len(DecoderModel(config_from_dict(one_tap).to_plan()).layers[0].cache_needs()) == 2


def slot_of_page(page, pinned, ring):
    """The place of a sequence's page in its page list, as the kernels compute it."""
    return page if ring == 0 or page < pinned else pinned + (page - pinned) % ring


def test_kept_first_positions_pin_pages_in_front_of_the_ring():
    need = KVNeed(2, 16, window=30, keep_first=70)
    cache = SequenceCache([(need,), (KVNeed(2, 16, window=30),)], [None, None], dtype=torch.float32, device="cpu",
                          max_tokens=2048, max_seqs=2, max_step_tokens=16)
    group = next(g for g in cache.kv_groups if g.need.keep_first == 70)
    plain_ring = next(g for g in cache.kv_groups if g.need.keep_first == 0)
    assert (group.pinned_pages, group.ring_len) == (2, pages_for(30 + 16 - 1) + 1)
    assert group.ring_pages == 2 * 65536 + group.ring_len and plain_ring.ring_pages == plain_ring.ring_len
    slot = cache.alloc()
    held = []
    for step in range(80):          # 1,280 positions, 16 at a time
        cache.reserve([slot], [16])
        cache.advance([slot], [16])
        held.append(len(group.slot_pages[slot]))
    assert held[0] == 1 and max(held) == group.pinned_pages + group.ring_len == len(group.slot_pages[slot])
    assert len(plain_ring.slot_pages[slot]) == plain_ring.ring_len
    # every position that a query may still ask for has a page of its own: the kept ones and the window of any query
    # of a step (the step's own later tokens included)
    pinned, ring = group.pinned_pages, group.ring_len
    for p in (100, 500, 1279):
        wanted = set(range(70)) | set(range(p - 29 - 15, p + 1))
        pages = {q // 64 for q in wanted if q >= 0}
        assert len({slot_of_page(page, pinned, ring) for page in pages}) == len(pages)
    cache.free(slot)
    cache.check()
    with pytest.raises(ValueError):
        SequenceCache([(KVNeed(1, 8, keep_first=3),)], [None], dtype=torch.float32, device="cpu", max_tokens=64, max_seqs=1)


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="attention"), ValueError),
    (lambda c: c["layers"][1]["mlp"].update(kind="gated"), ValueError),
    (lambda c: c["layers"][0]["mixer"].pop("right"), KeyError),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].pop("size"), ValueError),
    (lambda c: c.pop("width"), KeyError),
    (lambda c: c["norm"].update(eps=0.0), ValueError),
    (lambda c: c["token_side"].update(dim=0), ValueError),
    (lambda c: c.update(layers=[]), ValueError),
])
def test_refused_configurations(change, error):
    cfg = copy.deepcopy(plain.TINY_A)
    change(cfg)
    with pytest.raises(error):
        config_from_dict(cfg).to_plan()


def test_sizes_that_the_kernels_do_not_take_are_refused_when_the_model_is_built():
    cfg = copy.deepcopy(plain.TINY_A)
    cfg["layers"][0]["mixer"]["right"]["state"] = 300
    with pytest.raises(ValueError):
        DecoderModel(config_from_dict(cfg).to_plan())
    cfg = copy.deepcopy(plain.TINY_A)
    cfg["layers"][0]["mixer"]["right"]["groups"] = 4      # six heads do not form four groups
    with pytest.raises(ValueError):
        DecoderModel(config_from_dict(cfg).to_plan())

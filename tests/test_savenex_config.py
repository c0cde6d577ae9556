"""Savenex without a GPU: config.json parsing, the spec that is built from it, the tensor list, and the cache's
bookkeeping of kept first positions."""
from __future__ import annotations

import copy

import pytest
import torch

import savenex_tiny as V
from cpi_b200.cache.manager import CacheManager, KVRequirement
from cpi_b200.config.common import ConfigError
from cpi_b200.config.registry import architecture_of
from cpi_b200.config.savenex import SavenexConfig
from cpi_b200.engine.model import tensor_requirements
from cpi_b200.models.savenex import build_spec, refine_spec


def test_the_family_is_registered_and_parses_every_key():
    assert architecture_of(V.MIXED_A).name == "Savenex"
    cfg = SavenexConfig.from_json_dict(V.MIXED_A)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.residual_mult, cfg.loop) == (97, 52, 1e-5, 0.7, (1, 3, 2))
    l0 = cfg.layers[0]
    assert l0.left["mask"] == {"size": 12, "keep_first": 5} and l0.left["rot"] == {"base": 5000.0, "dims": 16, "factor": 4.0}
    assert l0.right == {"heads": 6, "kv_heads": 3, "dim": 12, "vdim": 20, "conv": 3}
    assert l0.mlp == {"kind": "dense", "ff": 50, "limit": 1.5}
    assert cfg.layers[1].mlp == {"kind": "moe", "ff": 28, "experts": 7, "top": 3, "shared_ff": 36}
    assert cfg.layers[2].mlp is None and cfg.layers[3].mlp["shared_ff"] is None
    assert cfg.run_order() == [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    b = SavenexConfig.from_json_dict(V.MIXED_B)
    assert b.loop is None and b.residual_mult == 1.0 and b.layers[2].left["mask"] is None
    assert b.layers[0].left["rot"]["factor"] == 1.0 and b.layers[0].left["mask"]["keep_first"] == 0


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "left"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=26), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c.update(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused_by_name(change, word):
    c = copy.deepcopy(V.MIXED_A)
    change(c)
    with pytest.raises(ConfigError) as e:
        SavenexConfig.from_json_dict(c)
    assert word in str(e.value)


def test_the_spec_names_parts_and_the_run_order_enters_each_pass_through_the_junction():
    cfg = SavenexConfig.from_json_dict(V.MIXED_A)
    spec = build_spec(cfg)
    spec.validate()
    assert [(e.layer, e.before) for e in spec.run_order] == [(0, None), (1, "loop_in"), (2, None), (1, "loop_in"),
                                                             (2, None), (3, None)]
    assert all(e.cache_of is None for e in spec.run_order)            # every pass owns its cache and state
    L = spec.layers[1]
    assert L.block.kind == "scaled_pre_norm" and L.block["residual_scale"] == 0.7 and L.mixer.kind == "parallel"
    left, right = (b["mixer"] for b in L.mixer["branches"])
    assert left.kind == "attention" and left["window"] == {"kind": "sliding", "size": 9, "keep_first": 3}
    assert right.kind == "gated_delta" and right["conv"] == 4
    assert L.feed_forward.kind == "moe_swiglu" and L.feed_forward["router_gate"] == "softmax_chosen"
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward["activation"] == "swish_clamped"
    assert dict(spec.junctions)["loop_in"].kind == "concat_linear" and spec.embedding["norm"].kind == "rmsnorm"
    b = build_spec(SavenexConfig.from_json_dict(V.MIXED_B))
    assert b.junctions == () and b.layers[0].block.kind == "pre_norm"


def test_tensor_list_and_ranks_from_shapes():
    cfg = SavenexConfig.from_json_dict(V.MIXED_A)
    W = V.draw_weights(V.MIXED_A, 1, ranks=(6, 5))

    class Shapes:
        def has(self, n): return n in W
        def shape(self, n): return tuple(W[n].shape)

    spec = refine_spec(cfg, build_spec(cfg), Shapes())
    reqs = {r.name: tuple(r.shape) for r in tensor_requirements(spec)}
    assert reqs == {n: tuple(t.shape) for n, t in W.items()}
    assert reqs["l0.mix.right.a1"] == (6, 52) and reqs["l0.mix.right.g2"] == (120, 5) and reqs["loop.in"] == (52, 104)


def test_pages_of_kept_first_positions_are_never_given_back():
    req = KVRequirement(1, 8, "sliding", 10, keep_first=70)          # kept positions reach into the second page
    plain = KVRequirement(1, 8, "sliding", 10)
    cm = CacheManager({0: req, 1: plain}, {}, max_tokens=1024, max_seqs=2, page_size=64, dtype=torch.float32,
                      device="cpu", max_step_tokens=128)
    kept, slid = cm.group_of_entry[0], cm.group_of_entry[1]
    assert kept is not slid and kept.pool.n_pages > slid.pool.n_pages
    s = cm.acquire()
    for n in (100, 100, 1, 1, 128, 60):
        cm.prepare_step([s], [n])
        cm.commit_step([s], [n])
    # 390 positions: the window needs blocks 5 and 6; the kept range holds blocks 0 and 1 besides
    assert sorted(kept.blocks[s]) == [0, 1, 5, 6] and sorted(slid.blocks[s]) == [5, 6]
    cm.check_consistency()
    cm.release(s)
    assert kept.pages_held() == 0 and kept.pool.free_count == kept.pool.n_pages
    s2 = cm.acquire()
    cm.prepare_step([s2], [5])
    assert sorted(kept.blocks[s2]) == [0]
    assert not req.droppable(1, 10_000, 64) and req.droppable(2, 10_000, 64) and not req.droppable(2, 130, 64)

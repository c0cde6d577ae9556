"""Veredra without a GPU: config.json parsing, run order, the spec's parts and the tensors they ask for."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_veredra as P
import veredra_tiny as V
from cpi_b200.config.common import ConfigError
from cpi_b200.config.registry import architecture_of
from cpi_b200.config.veredra import VeredraConfig
from cpi_b200.engine.model import tensor_requirements
from cpi_b200.models.veredra import build_spec, refine_spec
from cpi_b200.weights.store import DictSource, check_source


def test_the_architecture_is_found_by_either_key():
    assert architecture_of({"architecture": "Veredra"}).name == "Veredra"
    assert architecture_of({"architectures": ["Veredra"]}).name == "Veredra"
    with pytest.raises(ConfigError):
        architecture_of({"architecture": 3})


@pytest.mark.parametrize("cfg", [V.MIXED_A, V.MIXED_B, V.MIXED_C, V.GLA_ONLY])
def test_run_order_and_parts_follow_the_configuration(cfg):
    c = VeredraConfig.from_json_dict(cfg)
    assert c.run_order() == P.run_order(cfg)
    spec = build_spec(c)
    spec.validate()
    assert [e.layer for e in spec.run_order] == P.run_order(cfg) and all(e.cache_of is None for e in spec.run_order)
    assert spec.residual_streams == (cfg.get("streams") or 1)
    for ls, L in zip(spec.layers, cfg["layers"]):
        assert ls.mixer.kind == L["type"]
        assert (ls.feed_forward is None) == (L["mlp"] is None)
        assert ls.block.kind == ("hyper_connections" if "streams" in cfg else "pre_norm")
    assert spec.head.get("logit_softcap") == (cfg.get("logit_softcap") or 0.0)


@pytest.mark.parametrize("cfg,rank", [(V.MIXED_A, 8), (V.MIXED_B, 5), (V.GLA_ONLY, 3)])
def test_the_tensors_asked_for_are_the_tensors_of_the_folder(cfg, rank):
    """Names and shapes of every tensor, the rank of the decay projection read from the weights."""
    W = V.draw_weights(cfg, 1, decay_rank=rank)
    src = DictSource(W)
    c = VeredraConfig.from_json_dict(cfg)
    spec = refine_spec(c, build_spec(c), src)
    check_source(tensor_requirements(spec), src)
    gone = dict(W)
    name = next(n for n in W if n.endswith("mix.o"))
    del gone[name]
    with pytest.raises(Exception) as e:
        check_source(tensor_requirements(spec), DictSource(gone))
    assert name in str(e.value)


def test_bad_configurations_are_refused_by_name():
    def broken(change):
        c = copy.deepcopy(V.MIXED_A)
        change(c)
        return c
    for change, word in [(lambda c: c["layers"][0].update(type="conv"), "type"),
                         (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
                         (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=15), "dims"),
                         (lambda c: c["layers"][2]["mixer"].update(groups=4), "groups"),
                         (lambda c: c.update(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
                         (lambda c: c.pop("norm"), "norm"),
                         (lambda c: c["layers"][0]["mixer"].pop("tau"), "tau"),
                         (lambda c: c.update(width=0), "width")]:
        with pytest.raises(ConfigError) as e:
            VeredraConfig.from_json_dict(broken(change))
        assert word in str(e.value)


def test_the_plain_implementation_decodes_like_it_prefills():
    """The oracle itself: logits of a prefix are the first rows of the logits of the whole (causality)."""
    cfg = V.MIXED_B
    W = V.draw_weights(cfg, 2, decay_rank=5)
    toks = V.tokens(30, cfg["vocab"], 1)
    full = P.forward(cfg, W, toks)
    part = P.forward(cfg, W, toks[:11])
    assert (full[:11] - part).abs().max() < 1e-9
    lo = []
    P.forward(cfg, W, toks[:4], layer_outputs=lo)
    assert len(lo) == len(P.run_order(cfg)) and lo[0].shape == (4, cfg["width"])


def test_random_weights_mode_draws_a_veredra_folder(tmp_path):
    from cpi_b200.weights import write_random_model
    from cpi_b200.weights.safetensors_io import SafetensorsDir
    d = str(tmp_path / "m")
    write_random_model(d, V.MIXED_A, seed=3)
    sd = SafetensorsDir(d)
    names = set(sd.names())
    assert {"embed", "head", "final.norm", "l0.hc1.in", "l1.mix.sink", "l2.mix.A_log", "l0.mix.a2.b"} <= names
    assert "l2.norm2" not in names and "l2.hc2.mix" not in names          # layer 2 has no feed-forward
    mix = sd.tensor("l0.hc2.mix").float()
    assert mix.shape == (3, 3) and (mix - torch.eye(3)).abs().max() < 0.2

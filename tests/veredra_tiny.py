"""Small Veredra configurations and weights for the tests.

The weights are drawn here, not by the library's random mode, with spreads chosen so that faults show: attention
scores a few units wide (a single key can carry a row), sinks that weigh as much as a key, decays that keep some
state for hundreds of tokens and lose other state within a few, stream coefficients away from 0 and 1.
"""
from __future__ import annotations

import copy
import json
import os
import tempfile

import torch


def attention(heads, kv_heads, dim, vdim, window=None, rot_dims=None, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": (3.0 / dim ** 0.5) if scale is None else scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention", "mixer": m}


def mamba2(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def gla(heads, dim, vdim, tau):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def with_mlp(layer, ff):
    out = copy.deepcopy(layer)
    out["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return out


def model(layers, width, vocab, streams=None, loop=None, eps=1e-5, logit_scale=None, softcap=None):
    cfg = {"architecture": "Veredra", "layers": [l if "mlp" in l else with_mlp(l, None) for l in layers],
           "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if streams is not None:
        cfg["streams"] = streams
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    if softcap is not None:
        cfg["logit_softcap"] = softcap
    return cfg


# A: every mixer, three streams, a loop over an attention and a recurrent layer, grouped keys, values wider than
# keys, a rotation of part of the head, a short window.
MIXED_A = model([
    with_mlp(gla(3, 24, 40, 4.0), 96),
    with_mlp(attention(4, 2, 24, 40, window=12, rot_dims=16), 80),
    with_mlp(mamba2(6, 20, 24, 3, 4, 3), None),
    with_mlp(attention(2, 2, 32, 32, window=None, rot_dims=32, base=500.0), 64),
    with_mlp(mamba2(4, 16, 40, 1, 2, 1), 72),
], width=88, vocab=211, streams=3, loop=(1, 3, 2), logit_scale=0.7, softcap=12.0)

# B: no streams key (the plain residual), no loop, no softcap, one stream of attention without rotation, a window of
# one page and a bit, sizes that are no multiples of 8 (the float32-pipe products run in both precisions).
MIXED_B = model([
    with_mlp(attention(3, 1, 20, 12, window=70), 50),
    with_mlp(gla(2, 36, 28, 16.0), None),
    with_mlp(mamba2(5, 12, 20, 5, 3, 5), 44),
    with_mlp(attention(6, 3, 16, 16, window=5, rot_dims=8, base=1e6), 30),
], width=52, vocab=97, eps=1e-6)

# C: widths that are multiples of 8 so that the bfloat16 path runs on the tensor-core products; one stream with
# coefficients; a loop that runs once.
MIXED_C = model([
    with_mlp(mamba2(4, 32, 64, 2, 4, 2), 192),
    with_mlp(attention(4, 1, 64, 64, window=40, rot_dims=64), 192),
    with_mlp(gla(2, 64, 64, 8.0), 128),
], width=128, vocab=384, streams=1, loop=(0, 2, 1), logit_scale=1.5, softcap=30.0)

# D: four streams, a loop over everything, layers of one kind only.
GLA_ONLY = model([with_mlp(gla(2, 16, 24, 2.0), 48), with_mlp(gla(4, 8, 8, 32.0), None)], width=40, vocab=64,
                 streams=4, loop=(0, 2, 3))


def draw_weights(cfg: dict, seed: int, decay_rank: int = 8) -> dict:
    """{name: bfloat16 tensor} for a configuration."""
    g = torch.Generator().manual_seed(seed)
    W = {}

    def rn(shape, std, mean=0.0):
        if isinstance(shape, int):
            shape = (shape,)
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    width, vocab = cfg["width"], cfg["vocab"]
    W["embed"] = rn((vocab, width), 1.0)
    W["head"] = rn((vocab, width), 2.0 * width ** -0.5)
    W["final.norm"] = rn(width, 0.15)
    S = cfg.get("streams")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = rn(width, 0.15)
        if L["type"] == "attention":
            H, D = m["heads"], m["dim"]
            G, Dv = m.get("kv_heads", H), m.get("vdim", D)
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                W[p + f"mix.{n}"] = rn((rows, width), width ** -0.5)
                W[p + f"mix.{n}.b"] = rn(rows, 0.3)
            W[p + "mix.q.norm"] = rn(H * D, 0.25, 1.0)
            W[p + "mix.k.norm"] = rn(G * D, 0.25, 1.0)
            W[p + "mix.sink"] = rn(H, 2.0)
            W[p + "mix.o"] = rn((width, H * Dv), (H * Dv) ** -0.5)
        elif L["type"] == "mamba2":
            H, Dv, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, C = H * Dv, H * Dv + 2 * G * N
            W[p + "mix.in"] = rn((2 * inner + 2 * G * N + H, width), width ** -0.5)
            W[p + "mix.conv"] = rn((C, taps), 0.5)
            W[p + "mix.conv.b"] = rn(C, 0.2)
            W[p + "mix.dt_bias"] = rn(H, 1.0)
            W[p + "mix.A_log"] = rn(H, 1.5, -2.5)                 # decays from a few tokens to hundreds
            W[p + "mix.D"] = rn(H, 0.3, 1.0)
            W[p + "mix.norm"] = rn(inner, 0.2, 1.0)
            W[p + "mix.o"] = rn((width, inner), inner ** -0.5)
        else:
            H, D, Dv = m["heads"], m["dim"], m["vdim"]
            W[p + "mix.q"] = rn((H * D, width), width ** -0.5)
            W[p + "mix.k"] = rn((H * D, width), width ** -0.5)
            W[p + "mix.v"] = rn((H * Dv, width), width ** -0.5)
            W[p + "mix.g"] = rn((H * Dv, width), width ** -0.5)
            W[p + "mix.o"] = rn((width, H * Dv), (H * Dv) ** -0.5)
            W[p + "mix.norm"] = rn(Dv, 0.2, 1.0)
            W[p + "mix.a1"] = rn((decay_rank, width), width ** -0.5)
            W[p + "mix.a2"] = rn((H * D, decay_rank), 1.5 * decay_rank ** -0.5)
            W[p + "mix.a2.b"] = rn(H * D, 1.5, 2.0)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            W[p + "norm2"] = rn(width, 0.15)
            W[p + "mlp.gate"] = rn((ff, width), 1.5 * width ** -0.5)
            W[p + "mlp.up"] = rn((ff, width), width ** -0.5)
            W[p + "mlp.down"] = rn((width, ff), ff ** -0.5)
        if S is not None:
            for q in ((1, 2) if L.get("mlp") else (1,)):
                W[p + f"hc{q}.in"] = rn(S, 0.2, 1.0 / S)
                W[p + f"hc{q}.out"] = rn(S, 0.25, 1.0)
                W[p + f"hc{q}.mix"] = (torch.eye(S) + torch.randn(S, S, generator=g) * 0.15).to(torch.bfloat16)
    return W


def write_model(cfg: dict, W: dict, root=None) -> str:
    from cpi_b200.weights.safetensors_io import write_safetensors
    d = tempfile.mkdtemp(prefix="veredra_tiny_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), {k: v.contiguous() for k, v in W.items()})
    return d


def tokens(n: int, vocab: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()

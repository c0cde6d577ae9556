"""Small Savenex configurations and weights for the tests.

The weights are drawn here, not by the library's random mode, with spreads chosen so that faults show: attention
scores a few units wide (a single key can carry a row), decays that keep some state for hundreds of tokens and lose
other state within a few, write strengths on both sides of one half, router logits a unit apart, gates and clamps
that bite.
"""
from __future__ import annotations

import json
import os
import tempfile

import torch


def left(heads, kv_heads, dim, vdim, window=None, keep_first=None, rot_dims=None, base=10000.0, factor=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": (3.0 / dim ** 0.5) if scale is None else scale}
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    return m


def right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top, shared_ff=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff is not None:
        m["shared"] = {"ff": shared_ff}
    return m


def layer(l, r, mlp):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}


def model(layers, width, vocab, loop=None, eps=1e-5, mult=None):
    cfg = {"architecture": "Savenex", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if mult is not None:
        cfg["residual_mult"] = mult
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# A: sizes that are no multiples of 8 (the float32-pipe products in both precisions); grouped keys on both sides, values
# of another size than keys, a rotation of part of the head with scaling, a short window with kept first tokens, a loop
# in the middle, every kind of feed-forward, a shared expert.
MIXED_A = model([
    layer(left(4, 2, 24, 20, window=12, keep_first=5, rot_dims=16, base=5000.0, factor=4.0), right(6, 3, 12, 20, 3), dense(50, 1.5)),
    layer(left(3, 1, 20, 12, window=9, keep_first=3, rot_dims=20), right(2, 2, 36, 28, 4), moe(28, 7, 3, shared_ff=36)),
    layer(left(2, 2, 16, 24, window=70, keep_first=1), right(4, 1, 20, 12, 2), None),
    layer(left(6, 3, 12, 12, window=5, keep_first=9, rot_dims=8, base=1e6), right(3, 3, 8, 16, 3), moe(20, 5, 1)),
], width=52, vocab=97, loop=(1, 3, 2), mult=0.7)

# B: multiples of 8 and 16, so that the bfloat16 path runs the tensor-core products; a head whose keys, values and
# rotation have one size (the per-head preparation kernel), one layer with a plain sliding window (the tensor-core
# attention kernels), one with kept first tokens, one that sees everything; no loop; the plain residual sum; one
# expert per token without a shared expert; all experts at once.
MIXED_B = model([
    layer(left(4, 1, 64, 64, window=40, rot_dims=64), right(4, 2, 64, 64, 4), dense(192, 3.0)),
    layer(left(4, 2, 64, 64, window=24, keep_first=16, rot_dims=64, factor=2.0), right(2, 2, 48, 64, 3), moe(64, 4, 1)),
    layer(left(2, 2, 32, 64, rot_dims=16), right(8, 4, 16, 32, 2), moe(32, 3, 3, shared_ff=64)),
], width=128, vocab=384, eps=1e-6)

# C: what the other two make equal or absent: a loop from the first layer that runs three times, a window of one,
# no rotation, a convolution of one tap, more kept tokens than the window is wide, eight taps, a factor below one, a
# key size of four, one head, a single expert choice that takes every expert.
MIXED_C = model([
    layer(left(2, 1, 16, 8, window=1, keep_first=2), right(2, 1, 16, 8, 1), dense(40, 0.5)),
    layer(left(1, 1, 40, 40, window=3, keep_first=7, rot_dims=40, factor=0.5), right(5, 5, 4, 20, 8), moe(24, 2, 2, shared_ff=8)),
], width=40, vocab=64, loop=(0, 2, 3), mult=0.4)


def draw_config(seed: int) -> dict:
    """A configuration whose every size, option and constant is drawn from the seed: head counts and groups, head
    sizes from 4 to 128 (keys, values and rotated parts of different sizes or equal), windows from 1 position to none,
    kept first tokens from none to more than the window, taps 1 to 8, every kind of feed-forward, a loop anywhere."""
    import random
    rng = random.Random(seed)
    n_layers = rng.randint(1, 4)
    layers = []
    for _ in range(n_layers):
        G = rng.choice([1, 2, 3])
        H = G * rng.choice([1, 2, 4])
        D = rng.choice([8, 16, 20, 32, 64, 128])
        Dv = rng.choice([D, D, 8, 24, 64])
        l = left(H, G, D, Dv, window=rng.choice([None, 1, 7, 30, 64, 100]), keep_first=rng.choice([None, 0, 1, 20, 64, 70]),
                 rot_dims=rng.choice([None, D, max(2, D // 4 * 2)]), base=rng.choice([100.0, 1e4, 5e5]),
                 factor=rng.choice([None, 1.0, 2.0, 8.0]), scale=rng.choice([None, 2.0 / D ** 0.5]))
        Gr = rng.choice([1, 2, 4])
        Hr = Gr * rng.choice([1, 2, 3])
        r = right(Hr, Gr, rng.choice([4, 10, 16, 32, 64, 128]), rng.choice([8, 13, 64, 128]), rng.choice([1, 2, 3, 4, 8]))
        mlp = rng.choice([None, dense(rng.choice([24, 64, 256]), rng.choice([0.5, 2.0, 7.0])),
                          moe(rng.choice([16, 96]), rng.choice([2, 12, 33]), 1, shared_ff=rng.choice([None, 32])),
                          moe(rng.choice([16, 40]), 8, rng.choice([2, 4, 8]), shared_ff=rng.choice([None, 128]))])
        layers.append(layer(l, r, mlp))
    loop = None
    if rng.random() < 0.6:
        a = rng.randint(0, n_layers - 1)
        loop = (a, rng.randint(a + 1, n_layers), rng.randint(1, 3))
    return model(layers, width=rng.choice([24, 40, 64, 128, 264]), vocab=rng.choice([50, 131, 449]), loop=loop,
                 eps=rng.choice([1e-5, 1e-6]), mult=rng.choice([None, 1.0, 0.5, 0.25]))


def draw_weights(cfg: dict, seed: int, ranks=(6, 5)) -> dict:
    """{name: bfloat16 tensor} for a configuration; `ranks`: of the decay and the gate projection."""
    g = torch.Generator().manual_seed(seed)
    W = {}

    def rn(shape, std, mean=0.0):
        if isinstance(shape, int):
            shape = (shape,)
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    width, vocab = cfg["width"], cfg["vocab"]
    W["embed"] = rn((vocab, width), 1.0)
    W["embed.norm"] = rn(width, 0.2, 1.0)
    W["head"] = rn((vocab, width), 2.0 * width ** -0.5)
    W["final.norm"] = rn(width, 0.15, 1.0)
    if cfg.get("loop"):
        W["loop.in"] = torch.cat([torch.eye(width) * 0.8, torch.eye(width) * 0.3], dim=1).add_(
            torch.randn(width, 2 * width, generator=g) * 0.5 * width ** -0.5).to(torch.bfloat16)
    ra, rg = ranks
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        W[p + "norm1"] = rn(width, 0.15, 1.0)
        l, r = L["mixer"]["left"], L["mixer"]["right"]
        H, D = l["heads"], l["dim"]
        G, Dv = l.get("kv_heads", H), l.get("vdim", D)
        q = p + "mix.left."
        W[q + "q"] = rn((H * D, width), width ** -0.5)
        W[q + "k"] = rn((G * D, width), width ** -0.5)
        W[q + "v"] = rn((G * Dv, width), width ** -0.5)
        W[q + "o"] = rn((width, H * Dv), (H * Dv) ** -0.5)
        W[q + "out"] = rn(width, 0.2, 1.0)
        H, D = r["heads"], r["dim"]
        G, Dv, taps = r.get("kv_heads", H), r.get("vdim", D), r.get("conv", 1)
        q = p + "mix.right."
        W[q + "q"] = rn((G * D, width), 2.0 * width ** -0.5)
        W[q + "k"] = rn((G * D, width), 2.0 * width ** -0.5)
        W[q + "v"] = rn((H * Dv, width), 2.0 * width ** -0.5)
        for n, rows in (("q", G * D), ("k", G * D), ("v", H * Dv)):
            W[q + n + ".conv"] = rn((rows, taps), 0.5, 0.3)
        W[q + "b"] = rn((H, width), 2.0 * width ** -0.5)
        W[q + "A_log"] = rn(H, 1.5, -2.0)                        # decays from a few tokens to hundreds
        W[q + "dt_bias"] = rn(H * D, 1.0)
        W[q + "a1"] = rn((ra, width), width ** -0.5)
        W[q + "a2"] = rn((H * D, ra), 1.5 * ra ** -0.5)
        W[q + "g1"] = rn((rg, width), width ** -0.5)
        W[q + "g2"] = rn((H * Dv, rg), 2.0 * rg ** -0.5)
        W[q + "norm"] = rn(Dv, 0.2, 1.0)
        W[q + "o"] = rn((width, H * Dv), (H * Dv) ** -0.5)
        W[q + "out"] = rn(width, 0.2, 1.0)
        mlp = L.get("mlp")
        if not mlp:
            continue
        W[p + "norm2"] = rn(width, 0.15, 1.0)
        m = p + "mlp."

        def ffn(pre, ff, gate_std):
            W[pre + "gate"] = rn((ff, width), gate_std * width ** -0.5)
            W[pre + "up"] = rn((ff, width), gate_std * width ** -0.5)
            W[pre + "down"] = rn((width, ff), ff ** -0.5)

        if mlp["kind"] == "dense":
            ffn(m, mlp["ff"], 2.0)                                # pre-activations a few units wide: the clamps bite
        else:
            E = mlp["router"]["experts"]
            for e in range(E):
                ffn(f"{m}e{e}.", mlp["expert"]["ff"], 1.5)
            W[m + "router"] = rn((E, width), 2.0 * width ** -0.5)
            W[m + "router.b"] = rn(E, 1.0)
            if mlp.get("shared"):
                ffn(m + "shared.", mlp["shared"]["ff"], 1.5)
                W[m + "shared.sg"] = rn((1, width), 2.0 * width ** -0.5)
    return W


def write_model(cfg: dict, W: dict, root=None) -> str:
    from cpi_b200.weights.safetensors_io import write_safetensors
    d = tempfile.mkdtemp(prefix="savenex_tiny_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), {k: v.contiguous() for k, v in W.items()})
    return d


def tokens(n: int, vocab: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()

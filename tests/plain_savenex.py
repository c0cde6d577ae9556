"""A plain, slow Savenex: one function per mechanism, float64 on the CPU, whole sequences, nothing shared with
the library.  `weights` is {tensor name: torch tensor}; `cfg` the config.json dictionary.

Notation: T tokens, W model width; a linear map is y = x @ M.T for a stored M [out, in].
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(x, positions, dims, base, factor):
    """x [T, heads, D]: the first `dims` elements of every head turn, element i with element i + dims/2, by the
    angle position * base^(-2i/dims) / factor; the rest pass."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) / factor for i in range(half)], dtype=F64)
    a = positions.to(F64)[:, None] * f[None, :]                      # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(i, j, size, keep_first):
    """Does the query at position i see the key at position j?"""
    if j > i:
        return False
    if size is None:
        return True
    return i - j < size or j < keep_first


def softmax_attention(q, k, v, scale, size, keep_first):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]; query head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, size, keep_first)]
            s = torch.stack([(q[i, h] * k[j, g]).sum() * scale for j in js])
            p = torch.softmax(s, dim=0)
            out[i, h] = (p[:, None] * v[js, g]).sum(0)
    return out


def softmax_attention_fast(q, k, v, scale, size, keep_first):
    """The same as `softmax_attention` with the mask as a matrix (for long sequences)."""
    T, H, _ = q.shape
    G = k.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size is not None:
        ok = ok & ((i - j < size) | (j < keep_first))
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~ok, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def left_mixer(h, w, p, m, eps, positions):
    """`p` the tensor-name prefix ('l0.mix.left.'), `m` the config of this side."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, Dv)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate(q, positions, rot["dims"], rot["base"], factor)
        k = rotate(k, positions, rot["dims"], rot["base"], factor)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    mask = m.get("mask")
    size = mask["size"] if mask else None
    keep = (mask.get("keep_first") or 0) if mask else 0
    o = softmax_attention_fast(q, k, v, m["scale"], size, keep)
    return o.reshape(T, H * Dv) @ w[p + "o"].T


def short_conv(x, taps_w):
    """x [T, C], taps_w [C, taps]; the last column multiplies the current token, zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += taps_w[:, j] * x[src]
    return out


def silu(z):
    return z * torch.sigmoid(z)


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def gated_delta(q, k, v, beta, g):
    """q, k [T, H, D]; v [T, H, Dv]; beta [T, H]; g [T, H, D] -> o [T, H, Dv].  The state S [D, Dv] starts at
    zero: S <- g S (rows), u = beta (v - S^T k), S <- S + k u^T, o = S^T q."""
    T, H, D = q.shape
    Dv = v.shape[2]
    out = torch.zeros(T, H, Dv, dtype=F64)
    for h in range(H):
        S = torch.zeros(D, Dv, dtype=F64)
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, h])
            S = S + torch.outer(k[t, h], u)
            out[t, h] = S.T @ q[t, h]
    return out


def right_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, Dv)
    q = unit(q) * D ** -0.5
    k = unit(k)
    rep = H // G
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ w[p + "b"].T)                            # [T, H]
    z = ((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, D)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * torch.nn.functional.softplus(z))
    o = gated_delta(q, k, v, beta, g)
    o = rms_norm(o, w[p + "norm"], eps)
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, Dv)
    return (o * gate).reshape(T, H * Dv) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps, positions):
    a = left_mixer(h, w, p + "left.", m["left"], eps, positions)
    b = right_mixer(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(a, w[p + "left.out"], eps) + rms_norm(b, w[p + "right.out"], eps))


def dense_ff(h, w, p, m):
    limit = m["limit"]
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def moe_ff(h, w, p, m, chosen=None):
    E, top = m["router"]["experts"], m["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(z[t, e]), e))[:top]
        if chosen is not None:
            chosen.append(order)
        wts = torch.softmax(z[t, order], dim=0)
        for e, a in zip(order, wts):
            out[t] += a * expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if m.get("shared"):
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * expert(h, w, p + "shared.")
    return out


def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg, weights, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; `layers_out` (a list) receives the residual after every layer run."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    T = len(tokens)
    positions = torch.arange(T)
    x = rms_norm(w["embed"][torch.tensor(tokens)], w["embed.norm"], eps)
    x0 = x
    for i, pass_start in run_order(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if pass_start:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        assert L["type"] == "parallel"
        x = x + mult * parallel_mixer(rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", L["mixer"], eps, positions)
        mlp = L.get("mlp")
        if mlp:
            h = rms_norm(x, w[p + "norm2"], eps)
            y = dense_ff(h, w, p + "mlp.", mlp) if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
            x = x + mult * y
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T

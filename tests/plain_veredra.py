"""A plain, slow implementation of the Veredra decoder, one function per mechanism, in torch on the CPU.

It shares no code with the library: it reads the raw config.json dictionary and a {name: tensor} dictionary of
the stored weights and works on whole sequences from position 0 (no cache, no state between calls), so that the
library's prefill, decoding, batching and state keeping can all be compared with it.  Everything is computed in
`dtype` (float64 by default), which stands for "exact" beside the library's float32 and bfloat16 paths.

Notation: T tokens, W model width, H heads, G key/value heads or groups, D query/key size per head, Dv value
size per head, N state size.
"""
from __future__ import annotations

import math

import torch


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms_unit(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_half_split(x, positions, base, dims):
    """x [T, heads, D]: the first `dims` elements of each head turn, pair (i, i + dims/2) by the angle
    position * base^(-2i/dims); the rest stay."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]                # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def attention_mixer(h, m, w, eps):
    """Grouped-query softmax attention with biases, a norm over the whole q and k projections, partial rotation,
    a sliding window and a sink in the denominator.  h [T, W]; m: the mixer's config; w(name) -> tensor."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    G, Dv = m.get("kv_heads", H), m.get("vdim", D)
    q = h @ w("q").T + w("q.b")
    k = h @ w("k").T + w("k.b")
    v = h @ w("v").T + w("v.b")
    q = rms_unit(q, eps) * w("q.norm")
    k = rms_unit(k, eps) * w("k.norm")
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, Dv)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        q = rotate_half_split(q, pos, float(rot["base"]), int(rot["dims"]))
        k = rotate_half_split(k, pos, float(rot["base"]), int(rot["dims"]))
    window = (m.get("mask") or {}).get("size")
    sink = w("sink")
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    per = H // G
    for hd in range(H):
        g = hd // per
        s = (q[:, hd] @ k[:, g].T) * m["scale"]                         # [T query, T key]
        dist = pos[:, None] - pos[None, :]
        allowed = dist >= 0
        if window:
            allowed &= dist < window
        s = s.masked_fill(~allowed, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, sink[hd])
        e = torch.exp(s - top)
        denom = e.sum(-1, keepdim=True) + torch.exp(sink[hd] - top)
        out[:, hd] = (e / denom) @ v[:, g]
    return out.reshape(T, H * Dv) @ w("o").T


def causal_conv(x, weight, bias):
    """x [T, C]; weight [C, taps] whose last column multiplies the current token; zeros before the start."""
    T, C = x.shape
    taps = weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    out = bias[None, :].expand(T, C).clone()
    for j in range(taps):
        out = out + padded[j:j + T] * weight[:, j][None, :]
    return out


def mamba2_mixer(h, m, w, eps):
    """State-space mixer: S <- exp(-exp(A) dt) S + dt B x^T per head, y = S^T C + D x, gated, group-normed."""
    T = h.shape[0]
    H, Dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * Dv
    p = h @ w("in").T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w("conv"), w("conv.b")))
    x = xbc[:, :inner].view(T, H, Dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w("dt_bias"))                                     # [T, H]
    decay = torch.exp(-torch.exp(w("A_log"))[None, :] * dt)              # [T, H]
    per = H // G
    y = torch.zeros(T, H, Dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // per
        S = torch.zeros(N, Dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + w("D")[hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w("norm")
    return y @ w("o").T


def gla_mixer(h, m, w, eps):
    """Gated linear attention: S <- diag(alpha) S + k v^T per head, o = S^T q, head norm, output gate."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w("q").T * D ** -0.5).view(T, H, D)
    k = (h @ w("k").T).view(T, H, D)
    v = (h @ w("v").T).view(T, H, Dv)
    z = (h @ w("a1").T) @ w("a2").T + w("a2.b")
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).view(T, H, D)
    o = torch.zeros(T, H, Dv, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(D, Dv, dtype=h.dtype)
        for t in range(T):
            S = alpha[t, hd][:, None] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms_unit(o, eps) * w("norm")
    o = o.reshape(T, H * Dv) * silu(h @ w("g").T)
    return o @ w("o").T


def dense_mlp(h, w):
    return (gelu_tanh(h @ w("gate").T) * (h @ w("up").T)) @ w("down").T


MIXERS = {"attention": attention_mixer, "mamba2": mamba2_mixer, "gla": gla_mixer}


def run_order(cfg) -> list:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, weights, tokens, dtype=torch.float64, layer_outputs=None):
    """Logits [T, vocab] of one sequence from its first token.  `layer_outputs`: a list that receives the
    residual stream (the sum of the streams) after every layer run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    hyper = "streams" in cfg
    S = int(cfg.get("streams", 1))
    xs = [x.clone() for _ in range(S)]
    for li in run_order(cfg):
        layer = cfg["layers"][li]
        pre = f"l{li}."

        def sub(q, fn):
            nonlocal xs
            if hyper and (pre + f"hc{q}.in") in W:
                hin, hout, hmix = W[pre + f"hc{q}.in"], W[pre + f"hc{q}.out"], W[pre + f"hc{q}.mix"]
            else:
                hin, hout, hmix = torch.ones(S, dtype=dtype), torch.ones(S, dtype=dtype), torch.eye(S, dtype=dtype)
            u = sum(hin[s] * xs[s] for s in range(S))
            y = fn(norm_one_plus(u, W[pre + f"norm{q}"], eps))
            xs = [sum(hmix[s, t] * xs[s] for s in range(S)) + hout[t] * y for t in range(S)]

        mixer = MIXERS[layer["type"]]
        sub(1, lambda hh: mixer(hh, layer["mixer"], lambda n: W[pre + "mix." + n], eps))
        if layer.get("mlp"):
            sub(2, lambda hh: dense_mlp(hh, lambda n: W[pre + "mlp." + n]))
        if layer_outputs is not None:
            layer_outputs.append(sum(xs))
    x = norm_one_plus(sum(xs), W["final.norm"], eps)
    logits = x @ W["head"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits

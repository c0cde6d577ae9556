"""Typed configuration of the Veredra decoder, read from config.json keys.

A Veredra model is a list of layers, each with one of three mixers (softmax attention with a sliding window and
a sink, a selective state-space mixer, gated linear attention) and an optional gated feed-forward; a range of
layers may be run several times in a row with the same weights; the residual may be kept as several streams.
Every size and every constant that can differ between models is a key of config.json:

    architecture  "Veredra"                       vocab, width
    layers        [{type, mixer {...}, mlp {kind, ff} | null}, ...]
    loop          {start, stop, times} | absent   streams (absent: one plain residual)
    norm          {eps}                           logit_scale, logit_softcap (absent: none)

mixer keys -- attention: heads, kv_heads, dim, vdim, scale, rot {base, dims} | absent, mask {size} | absent;
mamba2: heads, vdim, state, groups, conv, norm_groups; gla: heads, dim, vdim, tau.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from .common import ConfigError

MIXER_TYPES = ("attention", "mamba2", "gla")


def _need(d: dict, key: str, where: str, kind=(int, float)):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"config.json: {where}.{key} has the wrong type ({v!r})")
    return v


def _pos_int(d: dict, key: str, where: str, default=None) -> int:
    if default is not None and d.get(key) is None:
        return default
    v = _need(d, key, where, int)
    if v < 1:
        raise ConfigError(f"config.json: {where}.{key} must be positive, not {v}")
    return int(v)


@dataclass(frozen=True)
class VeredraLayer:
    type: str
    mixer: dict                    # the validated mixer keys, with defaults filled in
    ff: Optional[int]              # hidden size of the feed-forward, None: the layer has none


@dataclass(frozen=True)
class VeredraConfig:
    architecture: str
    vocab: int
    width: int
    layers: tuple
    loop: Optional[tuple]          # (start, stop, times)
    streams: Optional[int]         # None: the key is absent and the residual is the plain sum
    eps: float
    logit_scale: float
    logit_softcap: float           # 0: none
    initializer_range: float

    def run_order(self) -> list:
        """Layer index of every layer run: layers start .. stop-1 `times` times in a row, the rest once."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    @staticmethod
    def from_json_dict(raw: dict) -> "VeredraConfig":
        vocab, width = _pos_int(raw, "vocab", "the model"), _pos_int(raw, "width", "the model")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {', '.join(MIXER_TYPES)}")
            m = L.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where} lacks its 'mixer' sizes")
            layers.append(VeredraLayer(L["type"], _mixer(L["type"], m, where + ".mixer"), _mlp(L.get("mlp"), where)))
        loop = None
        if raw.get("loop"):
            lp = raw["loop"]
            a, b = int(_need(lp, "start", "loop", int)), int(_need(lp, "stop", "loop", int))
            times = _pos_int(lp, "times", "loop")
            if not 0 <= a <= b <= len(layers):
                raise ConfigError(f"config.json: loop {a}..{b} is outside the {len(layers)} layers")
            loop = (a, b, times)
        streams = None
        if raw.get("streams") is not None:
            streams = _pos_int(raw, "streams", "the model")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        cap = raw.get("logit_softcap") or 0.0
        if isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap < 0:
            raise ConfigError(f"config.json: logit_softcap must be a positive number, not {cap!r}")
        scale = raw.get("logit_scale")
        return VeredraConfig(
            architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Veredra"])[0]),
            vocab=vocab, width=width, layers=tuple(layers), loop=loop, streams=streams,
            eps=float(_need(norm, "eps", "norm")), logit_scale=1.0 if scale is None else float(scale),
            logit_softcap=float(cap), initializer_range=float(raw.get("initializer_range", 0.02)))


def _mlp(m: Any, where: str) -> Optional[int]:
    if m is None:
        return None
    if not isinstance(m, dict) or m.get("kind", "dense") != "dense":
        raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense' (or mlp null)")
    return _pos_int(m, "ff", where + ".mlp")


def _mixer(kind: str, m: dict, where: str) -> dict:
    out = {"heads": _pos_int(m, "heads", where)}
    if kind == "attention":
        out["dim"] = _pos_int(m, "dim", where)
        out["kv_heads"] = _pos_int(m, "kv_heads", where, default=out["heads"])
        out["vdim"] = _pos_int(m, "vdim", where, default=out["dim"])
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"config.json: {where}: {out['heads']} heads over {out['kv_heads']} kv_heads")
        out["scale"] = float(_need(m, "scale", where))
        out["rot"] = None
        if m.get("rot"):
            dims = _pos_int(m["rot"], "dims", where + ".rot")
            if dims % 2 or dims > out["dim"]:
                raise ConfigError(f"config.json: {where}.rot.dims = {dims} must be even and at most dim")
            out["rot"] = {"base": float(_need(m["rot"], "base", where + ".rot")), "dims": dims}
        out["mask"] = None
        if m.get("mask"):
            out["mask"] = {"size": _pos_int(m["mask"], "size", where + ".mask")}
    elif kind == "mamba2":
        for k in ("vdim", "state", "groups", "conv"):
            out[k] = _pos_int(m, k, where)
        out["norm_groups"] = _pos_int(m, "norm_groups", where, default=1)
        if out["heads"] % out["groups"]:
            raise ConfigError(f"config.json: {where}: {out['heads']} heads over {out['groups']} groups")
        if (out["heads"] * out["vdim"]) % out["norm_groups"]:
            raise ConfigError(f"config.json: {where}: norm_groups does not divide heads * vdim")
    else:
        out["dim"], out["vdim"] = _pos_int(m, "dim", where), _pos_int(m, "vdim", where)
        out["tau"] = float(_need(m, "tau", where))
        if out["tau"] <= 0:
            raise ConfigError(f"config.json: {where}.tau must be positive")
    return out

"""Typed configuration of the Savenex decoder, read from config.json keys.

A Savenex layer runs two mixers side by side on the same normed input -- softmax attention with a sliding window that
keeps a sequence's first tokens, and a gated delta rule -- averages their normed outputs, and follows with a
feed-forward that is dense (a clamped gate), a mixture of experts (with an optional shared expert), or absent.  A range
of layers may run several times with the same weights; before each pass the residual and the embedding output go
through one matrix together.  Every size and every constant that can differ between models is a key of config.json:

    architecture  "Savenex"                        vocab, width, residual_mult
    layers        [{type: "parallel", mixer {left {...}, right {...}}, mlp {...} | null}, ...]
    loop          {start, stop, times} | absent    norm {eps}

left:  heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor} | absent} | absent,
       mask {size, keep_first} | absent
right: heads, kv_heads, dim, vdim, conv
mlp:   {kind: "dense", ff, limit} | {kind: "moe", expert {ff}, router {experts, top}, shared {ff} | absent}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .common import ConfigError
from .veredra import _need, _pos_int

MIXER_TYPES = ("parallel",)


@dataclass(frozen=True)
class SavenexLayer:
    type: str
    left: dict                     # validated keys of the attention side, defaults filled in
    right: dict                    # validated keys of the recurrent side
    mlp: Optional[dict]            # {"kind": "dense", "ff", "limit"} | {"kind": "moe", "ff", "experts", "top", "shared_ff"} | None


@dataclass(frozen=True)
class SavenexConfig:
    architecture: str
    vocab: int
    width: int
    layers: tuple
    loop: Optional[tuple]          # (start, stop, times)
    eps: float
    residual_mult: float
    initializer_range: float

    def run_order(self) -> list:
        """(layer index, first of a pass) of every layer run: layers start .. stop-1 `times` times in a row, the
        rest once."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        a, b, times = self.loop
        out = [(i, False) for i in range(a)]
        for _ in range(times):
            out += [(i, i == a) for i in range(a, b)]
        return out + [(i, False) for i in range(b, n)]

    @staticmethod
    def from_json_dict(raw: dict) -> "SavenexConfig":
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
            if not isinstance(m, dict) or not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                raise ConfigError(f"config.json: {where}.mixer needs the sizes of its 'left' and 'right' sides")
            layers.append(SavenexLayer(L["type"], _left(m["left"], where + ".mixer.left"),
                                       _right(m["right"], where + ".mixer.right"), _mlp(L.get("mlp"), where + ".mlp")))
        loop = None
        if raw.get("loop"):
            lp = raw["loop"]
            a, b = int(_need(lp, "start", "loop", int)), int(_need(lp, "stop", "loop", int))
            times = _pos_int(lp, "times", "loop")
            if not 0 <= a < b <= len(layers):
                raise ConfigError(f"config.json: loop {a}..{b} is not a range of the {len(layers)} layers")
            loop = (a, b, times)
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        mult = raw.get("residual_mult")
        return SavenexConfig(
            architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Savenex"])[0]),
            vocab=vocab, width=width, layers=tuple(layers), loop=loop, eps=float(_need(norm, "eps", "norm")),
            residual_mult=1.0 if mult is None else float(_need(raw, "residual_mult", "the model")),
            initializer_range=float(raw.get("initializer_range", 0.02)))


def _heads(m: dict, where: str) -> dict:
    out = {"heads": _pos_int(m, "heads", where)}
    out["kv_heads"] = _pos_int(m, "kv_heads", where, default=out["heads"])
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}: {out['heads']} heads over {out['kv_heads']} kv_heads")
    out["dim"] = _pos_int(m, "dim", where)
    out["vdim"] = _pos_int(m, "vdim", where, default=out["dim"])
    return out


def _left(m: dict, where: str) -> dict:
    out = _heads(m, where)
    out["scale"] = float(_need(m, "scale", where))
    out["rot"] = None
    if m.get("rot"):
        r = m["rot"]
        dims = _pos_int(r, "dims", where + ".rot")
        if dims % 2 or dims > out["dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims = {dims} must be even and at most dim")
        factor = 1.0
        if r.get("scaling"):
            factor = float(_need(r["scaling"], "factor", where + ".rot.scaling"))
            if not factor > 0:
                raise ConfigError(f"config.json: {where}.rot.scaling.factor must be positive")
        out["rot"] = {"base": float(_need(r, "base", where + ".rot")), "dims": dims, "factor": factor}
    out["mask"] = None
    if m.get("mask"):
        k = m["mask"]
        keep = k.get("keep_first") or 0
        if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
            raise ConfigError(f"config.json: {where}.mask.keep_first must be a count, not {keep!r}")
        out["mask"] = {"size": _pos_int(k, "size", where + ".mask"), "keep_first": int(keep)}
    return out


def _right(m: dict, where: str) -> dict:
    out = _heads(m, where)
    out["conv"] = _pos_int(m, "conv", where, default=1)
    return out


def _mlp(m, where: str) -> Optional[dict]:
    if m is None:
        return None
    if not isinstance(m, dict) or m.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where}.kind must be 'dense' or 'moe' (or mlp null)")
    if m["kind"] == "dense":
        limit = float(_need(m, "limit", where))
        if not limit > 0:
            raise ConfigError(f"config.json: {where}.limit must be positive")
        return {"kind": "dense", "ff": _pos_int(m, "ff", where), "limit": limit}
    if not isinstance(m.get("expert"), dict) or not isinstance(m.get("router"), dict):
        raise ConfigError(f"config.json: {where} needs 'expert' and 'router'")
    experts, top = _pos_int(m["router"], "experts", where + ".router"), _pos_int(m["router"], "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router: top {top} of {experts} experts")
    shared = m.get("shared")
    return {"kind": "moe", "ff": _pos_int(m["expert"], "ff", where + ".expert"), "experts": experts, "top": top,
            "shared_ff": None if not shared else _pos_int(shared, "ff", where + ".shared")}

"""Veredra as a `ModelSpec`: per layer one of three mixers and an optional gated feed-forward, a range of layers
that runs several times with the same weights (each pass with a cache or state of its own), and a residual kept
as several streams (hyper-connections).

Tensor names: `embed`, `head`, `final.norm`; layer i under `l<i>.`: `norm1`, `norm2`, `mix.*`, `mlp.{gate,up,down}`,
`hc<q>.{in,out,mix}` for sublayer q.  Norm weights of the layers and the final norm are stored as distances from
one; the norms inside the mixers have plain weights.  The decay projection of a gated-linear-attention layer has
a low rank that is read from the shape of its first matrix.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..config.veredra import VeredraConfig


def _mixer_spec(cfg: VeredraConfig, layer, decay_rank) -> PartSpec:
    m, W = layer.mixer, cfg.width
    if layer.type == "attention":
        rot = m["rot"]
        position = PartSpec("none", {}) if rot is None else PartSpec("rope", {
            "head_dim": m["dim"], "theta": rot["base"], "pairing": "half_split", "scaling": None,
            "rotary_dims": rot["dims"]})
        window = {"kind": "full", "size": 0} if m["mask"] is None else {"kind": "sliding", "size": m["mask"]["size"]}
        return PartSpec("attention", {
            "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "softmax_scale": m["scale"], "position": position, "bias": True,
            "qk_norm": True, "qk_norm_scope": "projection", "qk_norm_eps": cfg.eps, "qk_norm_order": "before_rope",
            "window": window, "sink": True, "query_temperature": None,
            "tensor_names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_bias": "mix.q.b",
                             "k_bias": "mix.k.b", "v_bias": "mix.v.b", "q_norm": "mix.q.norm", "k_norm": "mix.k.norm",
                             "sink": "mix.sink"}})
    if layer.type == "mamba2":
        return PartSpec("mamba2", {
            "hidden_size": W, "heads": m["heads"], "head_dim": m["vdim"], "state": m["state"], "groups": m["groups"],
            "conv": m["conv"], "norm_groups": m["norm_groups"], "norm_eps": cfg.eps,
            "tensor_names": {"in": "mix.in", "conv": "mix.conv", "conv_bias": "mix.conv.b", "dt_bias": "mix.dt_bias",
                             "A_log": "mix.A_log", "D": "mix.D", "norm": "mix.norm", "o": "mix.o"}})
    return PartSpec("gla", {
        "hidden_size": W, "heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"], "tau": m["tau"],
        "decay_rank": decay_rank, "norm_eps": cfg.eps,
        "tensor_names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "g": "mix.g", "o": "mix.o", "norm": "mix.norm",
                         "a1": "mix.a1", "a2": "mix.a2", "a2_bias": "mix.a2.b"}})


def build_spec(cfg: VeredraConfig, decay_ranks: dict | None = None) -> ModelSpec:
    """`decay_ranks`: {layer index: rank of the gla decay projection}, read from the weights' shapes by
    `spec_for_source`; a layer that is not named gets 16."""
    W = cfg.width
    norm = {"size": W, "eps": cfg.eps, "weight_offset": 1.0}
    layers = []
    for i, L in enumerate(cfg.layers):
        has_ff = L.ff is not None
        if cfg.streams is None:
            block = PartSpec("pre_norm", {})
        else:
            block = PartSpec("hyper_connections", {
                "streams": cfg.streams,
                "names": [{"read": f"hc{q}.in", "write": f"hc{q}.out", "mix": f"hc{q}.mix"}
                          for q in ((1, 2) if has_ff else (1,))]})
        layers.append(LayerSpec(
            prefix=f"l{i}.",
            block=block,
            mixer=_mixer_spec(cfg, L, (decay_ranks or {}).get(i, 16)),
            feed_forward=None if not has_ff else PartSpec("dense_swiglu", {
                "hidden_size": W, "intermediate_size": L.ff, "activation": "gelu_tanh",
                "tensor_names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}}),
            mixer_norm=PartSpec("rmsnorm", {**norm, "weight": "norm1"}),
            feed_forward_norm=None if not has_ff else PartSpec("rmsnorm", {**norm, "weight": "norm2"}),
        ))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"weight": "embed", "vocab_size": cfg.vocab, "hidden_size": W}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in cfg.run_order()),      # every pass of a repeated layer owns its cache
        final_norm=PartSpec("rmsnorm", {**norm, "weight": "final.norm"}),
        head=PartSpec("linear_head", {"weight": "head", "vocab_size": cfg.vocab, "hidden_size": W,
                                      "logit_scale": cfg.logit_scale, "logit_softcap": cfg.logit_softcap}),
        initializer_range=cfg.initializer_range,
        residual_streams=cfg.streams or 1,
    )


def refine_spec(cfg: VeredraConfig, spec: ModelSpec, source) -> ModelSpec:
    """Sizes that only the weights give: the rank of each gla layer's decay projection is the row count of its
    first matrix."""
    ranks = {}
    for i, L in enumerate(cfg.layers):
        name = f"l{i}.mix.a1"
        if L.type == "gla" and source.has(name):
            ranks[i] = int(source.shape(name)[0])
    return build_spec(cfg, ranks) if ranks else spec


register_architecture(Architecture("Veredra", VeredraConfig.from_json_dict, build_spec, refine_spec=refine_spec))

"""Savenex as a `ModelSpec`: every layer a `parallel` mixer of windowed softmax attention (left) and a gated delta rule
(right) whose normed outputs are averaged, then a dense feed-forward with a clamped gate, routed experts with an
optional gated shared expert, or none; the residual takes each sublayer's output times a constant; a range of layers
may run several times with the same weights, each pass with a cache and state of its own and entered through a
matrix over [residual ; embedding output]; the embedding output is normed.

Tensor names: `embed`, `embed.norm`, `loop.in`, `final.norm`, `head`; layer i under `l<i>.`: `norm1`, `norm2`,
`mix.left.{q,k,v,o,out}`, `mix.right.{q,k,v,q.conv,k.conv,v.conv,b,A_log,dt_bias,a1,a2,g1,g2,norm,o,out}`,
`mlp.{gate,up,down}` or `mlp.{router,router.b,e<n>.{gate,up,down},shared.{gate,up,down,sg}}`.  The ranks of the two
low-rank projections of the right side are read from the shapes of their first matrices.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.savenex import SavenexConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

DEFAULT_RANK = 16


def _mixer_spec(cfg: SavenexConfig, layer, ranks) -> PartSpec:
    W, l, r = cfg.width, layer.left, layer.right
    rot = l["rot"]
    position = PartSpec("none", {}) if rot is None else PartSpec("rope", {
        "head_dim": l["dim"], "theta": rot["base"], "pairing": "half_split", "rotary_dims": rot["dims"],
        "scaling": None if rot["factor"] == 1.0 else {"rope_type": "linear", "factor": rot["factor"]},
        "frequency_math": "float64"})
    window = {"kind": "full", "size": 0} if l["mask"] is None else \
        {"kind": "sliding", "size": l["mask"]["size"], "keep_first": l["mask"]["keep_first"]}
    left = PartSpec("attention", {
        "hidden_size": W, "num_heads": l["heads"], "num_kv_heads": l["kv_heads"], "head_dim": l["dim"],
        "value_dim": l["vdim"], "softmax_scale": l["scale"], "position": position, "qk_norm": True,
        "qk_norm_scope": "head", "qk_norm_eps": cfg.eps, "qk_norm_order": "after_rope", "window": window,
        "query_temperature": None,
        "tensor_names": {"q": "mix.left.q", "k": "mix.left.k", "v": "mix.left.v", "o": "mix.left.o"}})
    n = "mix.right."
    right = PartSpec("gated_delta", {
        "hidden_size": W, "heads": r["heads"], "kv_heads": r["kv_heads"], "key_dim": r["dim"], "value_dim": r["vdim"],
        "conv": r["conv"], "decay_rank": ranks[0], "gate_rank": ranks[1], "norm_eps": cfg.eps, "unit_eps": 1e-6,
        "tensor_names": {"q": n + "q", "k": n + "k", "v": n + "v", "q_conv": n + "q.conv", "k_conv": n + "k.conv",
                         "v_conv": n + "v.conv", "b": n + "b", "A_log": n + "A_log", "dt_bias": n + "dt_bias",
                         "a1": n + "a1", "a2": n + "a2", "g1": n + "g1", "g2": n + "g2", "norm": n + "norm", "o": n + "o"}})
    return PartSpec("parallel", {
        "hidden_size": W, "branches": [{"name": "left", "mixer": left}, {"name": "right", "mixer": right}],
        "combine": {"kind": "normed_mean", "eps": cfg.eps, "weights": ["mix.left.out", "mix.right.out"]}})


def _ff_spec(cfg: SavenexConfig, mlp) -> PartSpec:
    W = cfg.width
    if mlp["kind"] == "dense":
        return PartSpec("dense_swiglu", {
            "hidden_size": W, "intermediate_size": mlp["ff"], "activation": "swish_clamped", "limit": mlp["limit"],
            "tensor_names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
    shared = None
    if mlp["shared_ff"] is not None:
        shared = {"intermediate_size": mlp["shared_ff"], "token_gate": "mlp.shared.sg",
                  "tensor_names": {"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"}}
    return PartSpec("moe_swiglu", {
        "hidden_size": W, "num_experts": mlp["experts"], "top_k": mlp["top"], "expert_size": mlp["ff"],
        "router_gate": "softmax_chosen", "router_name": "mlp.router", "router_bias": "mlp.router.b",
        "expert_layout": "per_expert",
        "expert_names": {"gate": "mlp.e{e}.gate", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down"}, "shared": shared})


def build_spec(cfg: SavenexConfig, ranks: dict | None = None) -> ModelSpec:
    """`ranks`: {layer index: (rank of the decay projection, rank of the gate projection)}, read from the weights'
    shapes by `refine_spec`; a layer that is not named gets DEFAULT_RANK for both."""
    W = cfg.width
    norm = {"size": W, "eps": cfg.eps}
    block = PartSpec("pre_norm", {}) if cfg.residual_mult == 1.0 else \
        PartSpec("scaled_pre_norm", {"residual_scale": cfg.residual_mult})
    layers = []
    for i, L in enumerate(cfg.layers):
        has_ff = L.mlp is not None
        layers.append(LayerSpec(
            prefix=f"l{i}.", block=block,
            mixer=_mixer_spec(cfg, L, (ranks or {}).get(i, (DEFAULT_RANK, DEFAULT_RANK))),
            feed_forward=_ff_spec(cfg, L.mlp) if has_ff else None,
            mixer_norm=PartSpec("rmsnorm", {**norm, "weight": "norm1"}),
            feed_forward_norm=PartSpec("rmsnorm", {**norm, "weight": "norm2"}) if has_ff else None))
    looped = cfg.loop is not None
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"weight": "embed", "vocab_size": cfg.vocab, "hidden_size": W,
                                               "norm": PartSpec("rmsnorm", {**norm, "weight": "embed.norm"})}),
        layers=tuple(layers),
        # every pass of a repeated layer owns its cache and state; a pass is entered through the junction
        run_order=tuple(RunEntry(i, before="loop_in" if first else None) for i, first in cfg.run_order()),
        final_norm=PartSpec("rmsnorm", {**norm, "weight": "final.norm"}),
        head=PartSpec("linear_head", {"weight": "head", "vocab_size": cfg.vocab, "hidden_size": W}),
        initializer_range=cfg.initializer_range,
        junctions=(("loop_in", PartSpec("concat_linear", {"hidden_size": W, "weight": "loop.in"})),) if looped else (),
    )


def refine_spec(cfg: SavenexConfig, spec: ModelSpec, source) -> ModelSpec:
    """Sizes that only the weights give: the ranks of each layer's decay and gate projections are the row counts of
    their first matrices."""
    ranks = {}
    for i in range(len(cfg.layers)):
        a, g = f"l{i}.mix.right.a1", f"l{i}.mix.right.g1"
        if source.has(a) and source.has(g):
            ranks[i] = (int(source.shape(a)[0]), int(source.shape(g)[0]))
    return build_spec(cfg, ranks) if ranks else spec


register_architecture(Architecture("Savenex", SavenexConfig.from_json_dict, build_spec, refine_spec=refine_spec))

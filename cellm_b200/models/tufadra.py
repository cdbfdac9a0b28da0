"""Tufadra as a plan: a decoder of parallel layers (one norm; attention and a mixture of experts both read its
output and both results join the stream), with learned position vectors added to the embedding and no rotation.

The attention norms queries and keys over the whole projection, has values of a width of their own and a query
temperature that grows with the position; the feed-forward routes every token to a few of many small experts
(sigmoid scores, a correction that only the choice sees, groups of which the best are kept) beside one shared expert
behind a sigmoid gate. Norm weights are stored around zero (the factor is 1 + w). A layer may use an earlier
layer's tensors and keeps a cache of its own: it is that layer once more in the run order. The output product
reads the embedding table.

Tensor names: `embed`, `pos`, `final.norm`, and for layer i `l<i>.norm1`, `l<i>.mix.q|k|v|o`, `l<i>.mix.q.norm`,
`l<i>.mix.k.norm`, `l<i>.mlp.router|correction`, `l<i>.mlp.e<n>.up|down`, `l<i>.mlp.shared.up|down|sg`."""
from __future__ import annotations

from ..config.plan import LayerSpec, ModelPlan, OrderEntry, PartSpec
from ..config.registry import register_architecture
from ..config.tufadra import TufadraConfig


def _norm(cfg: TufadraConfig, tensor: str) -> PartSpec:
    return PartSpec("rms_norm", {"dim": cfg.width, "eps": cfg.norm_eps, "offset": 1.0}, {"weight": tensor})


def build_plan(cfg: TufadraConfig) -> ModelPlan:
    H = cfg.width
    layers, plan_index, order = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        m = layer.mixer
        mixer = PartSpec(
            "attention",
            {"hidden_size": H, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
             "scale": m.scale, "window": 0, "position": None, "pad_heads": True,
             "qk_norm": PartSpec("rms_norm", {"dim": m.dim, "eps": cfg.norm_eps}), "qk_norm_span": "projection",
             "query_temperature": {"coef": m.q_temp.coef, "every": m.q_temp.every} if m.q_temp is not None else None},
            {"q_proj": p + "mix.q", "k_proj": p + "mix.k", "v_proj": p + "mix.v", "out_proj": p + "mix.o",
             "q_norm": p + "mix.q.norm", "k_norm": p + "mix.k.norm"})
        ffn = None
        if layer.mlp is not None:
            f = layer.mlp
            names = {"router": p + "mlp.router", "correction": p + "mlp.correction"}
            for e in range(f.experts):
                names[f"up_{e}"] = f"{p}mlp.e{e}.up"
                names[f"down_{e}"] = f"{p}mlp.e{e}.down"
            if f.shared_ff:
                names.update(shared_up=p + "mlp.shared.up", shared_down=p + "mlp.shared.down", shared_gate=p + "mlp.shared.sg")
            ffn = PartSpec("routed_experts",
                           {"hidden_size": H, "experts": f.experts, "top": f.top, "ff_dim": f.ff, "activation": "gelu",
                            "route_scale": f.scale, "groups": f.groups, "keep_groups": f.keep, "correction": True,
                            "shared_ff": f.shared_ff, "shared_gate": True}, names)
        plan_index[i] = len(layers)
        layers.append(LayerSpec("parallel", mixer, ffn, _norm(cfg, p + "norm1"), None))
    for i, layer in enumerate(cfg.layers):
        order.append(OrderEntry(plan_index[i if layer.weights_of is None else layer.weights_of]))
    return ModelPlan(
        hidden_size=H, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("lookup", {"vocab_size": cfg.vocab, "dim": H, "max_positions": cfg.max_positions},
                           {"weight": "embed", "positions": "pos"}),
        final_norm=_norm(cfg, "final.norm"),
        head=None,          # the embedding table itself
        layers=tuple(layers), order=tuple(order), eos_token_id=cfg.eos_token_id)


register_architecture("Tufadra", TufadraConfig, build_plan, model_types=("tufadra",))

"""Vezalorn as a plan: a decoder whose layers mix by latent attention or by a minGRU recurrence, in the order the
configuration lists them. Every sublayer reads the residual stream itself; its result is gated by a sigmoid of a
product over the same input, RMS-normed in groups and added into the stream (`gated_post_norm`). Feed-forwards are
gated, with the tanh form of gelu and biases, and a layer may have none. The embedding row is multiplied by a constant;
the output product reads the embedding table itself after the model's norm.

Tensor names: `embed`, `final.norm`, and for layer i `l<i>.norm1|norm2`, `l<i>.rg1|rg2` with `.b`, `l<i>.mix.*`,
`l<i>.mlp.*`. The parts themselves do not know they are in this design."""
from __future__ import annotations

from ..config.plan import LayerSpec, ModelPlan, OrderEntry, PartSpec
from ..config.registry import register_architecture
from ..config.vezalorn import LatentAttentionConfig, VezalornConfig

# The design sets no limit on positions; the scheduler wants a number.
NO_POSITION_LIMIT = 1 << 30


def _norm(cfg: VezalornConfig, tensor: str) -> PartSpec:
    return PartSpec("rms_norm", {"dim": cfg.width, "eps": cfg.norm_eps, "groups": cfg.norm_groups}, {"weight": tensor})


def build_plan(cfg: VezalornConfig) -> ModelPlan:
    H = cfg.width
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, LatentAttentionConfig):
            mixer = PartSpec(
                "latent_attention",
                {"hidden_size": H, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                 "scale": m.scale, "eps": cfg.norm_eps,
                 "position": PartSpec("rope", {"head_dim": m.rot_dim, "rotary_dim": m.rot.dims, "theta": m.rot.base,
                                               "layout": "interleaved"})},
                {"q": p + "mix.q", "dkv": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk",
                 "uv": p + "mix.uv", "o": p + "mix.o"})
        else:
            mixer = PartSpec("mingru", {"hidden_size": H, "width": m.width, "bias": True},
                             {"z": p + "mix.z", "z_bias": p + "mix.z.b", "x": p + "mix.x", "x_bias": p + "mix.x.b",
                              "g": p + "mix.g", "o": p + "mix.o"})
        ffn = ffn_norm = None
        gates = {"mixer_gate": p + "rg1", "mixer_gate_bias": p + "rg1.b"}
        if layer.mlp is not None:
            ffn = PartSpec("gated_mlp", {"hidden_size": H, "ff_dim": layer.mlp.ff, "activation": "gelu_tanh", "bias": True},
                           {"gate": p + "mlp.gate", "gate_bias": p + "mlp.gate.b", "up": p + "mlp.up", "up_bias": p + "mlp.up.b",
                            "down": p + "mlp.down", "down_bias": p + "mlp.down.b"})
            ffn_norm = _norm(cfg, p + "norm2")
            gates.update(feed_forward_gate=p + "rg2", feed_forward_gate_bias=p + "rg2.b")
        block = PartSpec("gated_post_norm", {"hidden_size": H, "gate": True, "feed_forward": ffn is not None}, gates)
        layers.append(LayerSpec(block, mixer, ffn, _norm(cfg, p + "norm1"), ffn_norm))
    return ModelPlan(
        hidden_size=H, vocab_size=cfg.vocab, max_positions=NO_POSITION_LIMIT,
        embedding=PartSpec("lookup", {"vocab_size": cfg.vocab, "dim": H, "scale": cfg.embedding_scale}, {"weight": "embed"}),
        final_norm=_norm(cfg, "final.norm"),
        head=None,          # the embedding table itself, without its scale
        layers=tuple(layers), order=tuple(OrderEntry(i) for i in range(len(layers))),
        eos_token_id=cfg.eos_token_id)


register_architecture("Vezalorn", VezalornConfig, build_plan, model_types=("vezalorn",))

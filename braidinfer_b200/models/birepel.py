"""The Birepel decoder as a description of parts.

token embedding + a learned vector a position -> layers -> RMS norm -> the embedding table as the output head.
A layer norms what its sublayers return, not what they read: h += rmsnorm(mixer(h)); h += rmsnorm(feed_forward(h))
(the feed-forward may be absent); every norm keeps a zero-centred weight w and multiplies by 1 + w.
Mixers: "attention" is causal grouped-query attention without rotation, its query and key heads brought to unit
root mean square, the query times a temperature that grows with the logarithm of its position, a learned sink a
head in the softmax, a sigmoid gate a head on the result; "mlstm" is a matrix memory with exponential gates.
Feed-forwards: a clamped gated unit, or a mixture of small experts without gates whose activation is the square
of relu, the chosen experts weighted by the softmax over their logits alone.
A layer may read another layer's tensors (`weights_of`) and still keeps a cache or state of its own: the schedule
then names that layer again.  Tensor names: `embed`, `pos`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`,
`l<i>.mlp.{gate,up,down}` or `l<i>.mlp.router`, `l<i>.mlp.e<k>.{up,down}`, `final.norm`.
"""
from __future__ import annotations

from ..config.birepel import BirepelConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import Architecture, register_architecture


def build_birepel_spec(cfg: BirepelConfig) -> ModelSpec:
    def rms(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.norm_eps, "name": name, "offset": 1.0})

    layers, index_of = [], {}
    for i, L in enumerate(cfg.layers):
        if L.weights_of != i:
            continue
        m = L.mixer
        if L.type == "attention":
            mixer = PartSpec("gqa_attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "value_dim": m.vdim, "window": None, "position_encoding": PartSpec("none", {"head_dim": m.dim}),
                "q_proj": "mix.q", "k_proj": "mix.k", "v_proj": "mix.v", "o_proj": "mix.o", "head_gate": "mix.g",
                "sink_name": "mix.sink", "scale": m.scale, "unit_qk_eps": cfg.norm_eps,
                "q_temp": None if m.temp_coef is None else {"coef": m.temp_coef, "every": m.temp_every}})
        else:
            mixer = PartSpec("mlstm", {"hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                       "gate_cap": m.gate_cap, "eps": cfg.norm_eps})
        ffn = ffn_norm = None
        f = L.mlp
        if f is not None:
            if hasattr(f, "limit"):
                ffn = PartSpec("clamped_glu", {"hidden_size": cfg.width, "intermediate_size": f.ff, "limit": f.limit,
                                               "alpha": 1.702, "gate_proj": "mlp.gate", "up_proj": "mlp.up",
                                               "down_proj": "mlp.down"})
            else:
                ffn = PartSpec("moe", {"hidden_size": cfg.width, "intermediate_size": f.ff, "experts": f.experts,
                                       "top": f.top, "gated": False, "activation": "relu2", "router": "mlp.router",
                                       "expert_up": "mlp.e{e}.up", "expert_down": "mlp.e{e}.down"})
            ffn_norm = rms("norm2")
        index_of[i] = len(layers)
        layers.append(LayerSpec(block="sublayer_norm_residual", prefix=f"l{i}.", mixer=mixer, mixer_norm=rms("norm1"),
                                feed_forward=ffn, feed_forward_norm=ffn_norm))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed",
                                               "positions": {"name": "pos", "max": cfg.max_positions}}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(index_of[L.weights_of]) for L in cfg.layers),
        final_norm=rms("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "head", "tied": True}),
        max_position=cfg.max_positions, eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id)


BIREPEL = register_architecture(Architecture(
    name="Birepel", config_from_dict=BirepelConfig.from_dict, build_spec=build_birepel_spec))

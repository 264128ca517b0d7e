"""The Ludazen decoder as a description of parts.

token embedding -> layers -> RMS norm -> output head (a matrix of its own).
A layer: h += mixer(rmsnorm(h)); h += feed_forward(rmsnorm(h)) (the feed-forward may be absent).
Mixers: "attention" is grouped-query attention whose heads are rotated in halves over their first numbers with
YaRN-stretched frequencies, with a stored factor a head on the scores, a window that also keeps the sequence's first
tokens in sight, and a stored matrix that mixes the heads' probabilities after the softmax; "latent_attention" keeps
one low-rank latent and one rotated key part a token (rotated in neighbouring pairs) behind a plain window, and a layer
may read the latent that an earlier layer cached (`kv_from`) with queries and up-projections of its own.
Feed-forwards: one hidden layer with biases and the xIELU activation, or a mixture of gated experts chosen by sigmoid
scores that multiply the expert's input, beside an expert that every token uses.
Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.{q,k,v,o,temp,talk}` or `l<i>.mix.{q,dkv,dkv.norm,uk,uv,o}`,
`l<i>.mlp.{up,up.b,down,down.b,act}` or `l<i>.mlp.router`, `l<i>.mlp.e<k>.{gate,up,down}`, `l<i>.mlp.shared.{gate,up,down}`,
`final.norm`, `head`.
"""
from __future__ import annotations

from ..config.ludazen import LudazenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import Architecture, register_architecture


def build_ludazen_spec(cfg: LudazenConfig) -> ModelSpec:
    def rms(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.norm_eps, "name": name})

    # a latent that later layers read is kept for the longest window among its readers
    keep = {}
    for i, L in enumerate(cfg.layers):
        if L.type == "latent_attention":
            owner = i if L.mixer.kv_from is None else L.mixer.kv_from
            keep[owner] = max(keep.get(owner, 0), L.mixer.window)
    layers, schedule = [], []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "attention":
            sc = m.rot_scaling
            rope = PartSpec("rope", {
                "head_dim": m.dim, "theta": m.rot_base, "rope_dim": m.rot_dims, "pairing": "half",
                "scaling": None if sc is None else {"factor": sc.factor, "original": sc.original, "fast": sc.fast,
                                                     "slow": sc.slow}})
            mixer = PartSpec("gqa_attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "value_dim": m.vdim, "window": m.window, "keep_first": m.keep_first, "position_encoding": rope,
                "q_proj": "mix.q", "k_proj": "mix.k", "v_proj": "mix.v", "o_proj": "mix.o", "scale": m.scale,
                "head_scale": "mix.temp", "talk": "mix.talk"})
            schedule.append(ScheduleEntry(i))
        else:
            rope = PartSpec("rope", {"head_dim": m.rot_dim, "theta": m.rot_base, "rope_dim": m.rot_dims,
                                     "pairing": "adjacent"})
            mixer = PartSpec("latent_attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "window": m.window, "gated": False,
                "shared_kv": m.kv_from is not None,
                "cache_window": keep[i if m.kv_from is None else m.kv_from], "position_encoding": rope})
            schedule.append(ScheduleEntry(i, cache_of=m.kv_from))
        ffn = ffn_norm = None
        f = L.mlp
        if f is not None:
            if hasattr(f, "experts"):
                shared = None
                if f.shared_ff is not None:
                    shared = PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": f.shared_ff,
                                                 "gate_proj": "mlp.shared.gate", "up_proj": "mlp.shared.up",
                                                 "down_proj": "mlp.shared.down"})
                ffn = PartSpec("moe", {"hidden_size": cfg.width, "intermediate_size": f.ff, "experts": f.experts,
                                       "top": f.top, "scoring": "sigmoid", "weight_on": "input", "shared": shared})
            else:
                ffn = PartSpec("biased_mlp", {"hidden_size": cfg.width, "intermediate_size": f.ff, "activation": "xielu"})
            ffn_norm = rms("norm2")
        layers.append(LayerSpec(block="prenorm_residual", prefix=f"l{i}.", mixer=mixer, mixer_norm=rms("norm1"),
                                feed_forward=ffn, feed_forward_norm=ffn_norm))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed"}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=rms("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "head", "tied": False}),
        eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id)


LUDAZEN = register_architecture(Architecture(
    name="Ludazen", config_from_dict=LudazenConfig.from_dict, build_spec=build_ludazen_spec))

"""Typed configuration of the Ludazen decoder, read from config.json.

config.json keys (nested objects; every size and every constant that differs between models):
    architecture            "Ludazen"
    vocab, width            vocabulary and residual width
    norm.eps                eps of every RMS norm (the stream's and the latent's)
    layers[i].type          the layer's mixer: "attention" or "latent_attention"
    layers[i].mixer         "attention": heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor, original,
                            fast, slow} (absent: none)}, mask {size, keep_first (absent: 0)}
                            "latent_attention": heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}, mask {size},
                            kv_from (absent: the layer makes its own latent; j: it reads layer j's)
    layers[i].mlp           null, or kind "dense" with ff, or kind "moe" with expert.ff, router.experts, router.top
                            and shared.ff (shared absent: no expert that every token uses)
A key that is missing, or a value that no part here computes, is a `ConfigError` naming key and value.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .bidinex import _get
from .errors import ConfigError
from .loduzen import RotScalingConfig

MIXER_TYPES = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class TalkingAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotScalingConfig]
    window: int
    keep_first: int


@dataclass(frozen=True)
class WindowLatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    window: int
    kv_from: Optional[int]           # the layer whose latent and rotated key part this one reads


@dataclass(frozen=True)
class BiasedFFConfig:
    ff: int


@dataclass(frozen=True)
class SharedMoeConfig:
    ff: int
    experts: int
    top: int
    shared_ff: Optional[int]         # None: no shared expert


@dataclass(frozen=True)
class LudazenLayerConfig:
    type: str
    mixer: Any                       # TalkingAttentionConfig | WindowLatentConfig
    mlp: Any                         # BiasedFFConfig | SharedMoeConfig | None


@dataclass(frozen=True)
class LudazenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[LudazenLayerConfig, ...]
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LudazenConfig":
        layers_in = d.get("layers")
        if not isinstance(layers_in, (list, tuple)) or not layers_in:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_in):
            at = f"layers[{i}]"
            if not isinstance(L, Mapping):
                raise ConfigError(f"config.json: '{at}' must be an object")
            kind = L.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{at}.type' is {kind!r}; known mixers: {list(MIXER_TYPES)}")
            m = {"m": L.get("mixer")}
            rot_dims = _get(m, "m.rot.dims", int, minimum=0)
            if rot_dims % 2:
                raise ConfigError(f"config.json: '{at}.mixer.rot.dims' must be even, got {rot_dims}")
            base = _get(m, "m.rot.base", float)
            if not base > 0:
                raise ConfigError(f"config.json: '{at}.mixer.rot.base' must be positive, got {base}")
            window = _get(m, "m.mask.size", int, minimum=1)
            if kind == "attention":
                heads, kv = _get(m, "m.heads", int, minimum=1), _get(m, "m.kv_heads", int, minimum=1)
                if heads % kv:
                    raise ConfigError(f"config.json: '{at}.mixer': {heads} heads do not form {kv} equal groups")
                dim = _get(m, "m.dim", int, minimum=1)
                if rot_dims > dim:
                    raise ConfigError(f"config.json: '{at}.mixer.rot.dims' is {rot_dims}, more than the head's {dim}")
                scaling = None
                if _get(m, "m.rot.scaling", None, optional=True) is not None:
                    scaling = RotScalingConfig(*(_get(m, "m.rot.scaling." + k, float)
                                                 for k in ("factor", "original", "fast", "slow")))
                    if min(scaling.factor, scaling.original, scaling.fast, scaling.slow) <= 0:
                        raise ConfigError(f"config.json: '{at}.mixer.rot.scaling' wants positive numbers, got {scaling}")
                mixer = TalkingAttentionConfig(
                    heads, kv, dim, _get(m, "m.vdim", int, minimum=1), _get(m, "m.scale", float), base, rot_dims, scaling,
                    window, _get(m, "m.mask.keep_first", int, minimum=0, optional=True) or 0)
            else:
                rot_dim = _get(m, "m.rot_dim", int, minimum=2)
                if rot_dims > rot_dim:
                    raise ConfigError(f"config.json: '{at}.mixer': the rotated part has {rot_dim} numbers and rot.dims is "
                                      f"{rot_dims}")
                src = L["mixer"].get("kv_from")
                if src is not None and (isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i):
                    raise ConfigError(f"config.json: '{at}.mixer.kv_from' is {src!r}; it names an earlier layer")
                mixer = WindowLatentConfig(
                    _get(m, "m.heads", int, minimum=1), _get(m, "m.dim", int, minimum=1), rot_dim,
                    _get(m, "m.vdim", int, minimum=1), _get(m, "m.kv_rank", int, minimum=1), _get(m, "m.scale", float),
                    base, rot_dims, window, src)
                if src is not None:
                    o = layers[src]
                    if o.type != "latent_attention" or o.mixer.kv_from is not None:
                        raise ConfigError(f"config.json: '{at}.mixer.kv_from' names layer {src}, which makes no latent of its own")
                    if (o.mixer.kv_rank, o.mixer.rot_dim, o.mixer.rot_base, o.mixer.rot_dims) != \
                            (mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.rot_dims):
                        raise ConfigError(f"config.json: '{at}.mixer' reads the latent of layer {src}, whose kv_rank, rot_dim "
                                          f"or rotation is another")
            mlp = None
            if L.get("mlp") is not None:
                f = {"f": L["mlp"]}
                fk = _get(f, "f.kind", str)
                if fk not in MLP_KINDS:
                    raise ConfigError(f"config.json: '{at}.mlp.kind' is {fk!r}; known feed-forwards: {list(MLP_KINDS)}")
                if fk == "dense":
                    mlp = BiasedFFConfig(_get(f, "f.ff", int, minimum=1))
                else:
                    mlp = SharedMoeConfig(_get(f, "f.expert.ff", int, minimum=1), _get(f, "f.router.experts", int, minimum=1),
                                          _get(f, "f.router.top", int, minimum=1),
                                          _get(f, "f.shared.ff", int, minimum=1, optional=True))
                    if mlp.top > mlp.experts:
                        raise ConfigError(f"config.json: '{at}.mlp.router': top {mlp.top} of {mlp.experts} experts")
            layers.append(LudazenLayerConfig(kind, mixer, mlp))
        eos = d.get("eos_token_id")
        eos_ids = tuple(eos) if isinstance(eos, (list, tuple)) else ((int(eos),) if isinstance(eos, int) else ())
        return cls(vocab=_get(d, "vocab", int, minimum=1), width=_get(d, "width", int, minimum=1),
                   norm_eps=_get(d, "norm.eps", float), layers=tuple(layers), eos_token_ids=eos_ids,
                   bos_token_id=d.get("bos_token_id"))

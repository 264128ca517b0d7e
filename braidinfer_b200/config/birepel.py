"""Typed configuration of the Birepel decoder, read from config.json.

config.json keys (nested objects; every size and every constant that differs between models):
    architecture            "Birepel"
    vocab, width            vocabulary and residual width
    max_positions           rows of the learned table of positions (the longest sequence)
    norm.eps                eps of every RMS norm, of the unit norms of attention heads and of the memory's read-out
    layers[i].type          the layer's mixer: "attention" or "mlstm"
    layers[i].mixer         "attention": heads, kv_heads, dim, vdim, scale, q_temp {coef, every} (absent: none)
                            "mlstm": heads, dim, vdim, gate_cap
    layers[i].mlp           null, or kind "dense" with ff and limit, or kind "moe" with expert.ff, router.experts,
                            router.top
    layers[i].weights_of    j: the layer has no tensors of its own and reads layer j's (mixer, feed-forward and
                            norms), with a cache or state of its own; the rest of its entry is layer j's
A key that is missing, or a value that no part here computes, is a `ConfigError` naming key and value.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .bidinex import _get
from .errors import ConfigError

MIXER_TYPES = ("attention", "mlstm")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: Optional[float]       # None: no query temperature
    temp_every: int


@dataclass(frozen=True)
class MlstmConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoeFFConfig:
    ff: int
    experts: int
    top: int


@dataclass(frozen=True)
class BirepelLayerConfig:
    type: str
    mixer: Any                       # SinkAttentionConfig | MlstmConfig
    mlp: Any                         # DenseFFConfig | MoeFFConfig | None
    weights_of: int                  # the layer whose tensors this one reads (itself: its own)


@dataclass(frozen=True)
class BirepelConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: Tuple[BirepelLayerConfig, ...]
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BirepelConfig":
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
            if kind == "attention":
                heads, kv = _get(m, "m.heads", int, minimum=1), _get(m, "m.kv_heads", int, minimum=1)
                if heads % kv:
                    raise ConfigError(f"config.json: '{at}.mixer': {heads} heads do not form {kv} equal groups")
                coef = _get(m, "m.q_temp.coef", float, optional=True)
                every = _get(m, "m.q_temp.every", int, minimum=1, optional=coef is None)
                mixer = SinkAttentionConfig(heads, kv, _get(m, "m.dim", int, minimum=1), _get(m, "m.vdim", int, minimum=1),
                                            _get(m, "m.scale", float), coef, every or 0)
            else:
                cap = _get(m, "m.gate_cap", float)
                if not cap > 0:
                    raise ConfigError(f"config.json: '{at}.mixer.gate_cap' must be positive, got {cap}")
                mixer = MlstmConfig(_get(m, "m.heads", int, minimum=1), _get(m, "m.dim", int, minimum=1),
                                    _get(m, "m.vdim", int, minimum=1), cap)
            mlp = None
            if L.get("mlp") is not None:
                f = {"f": L["mlp"]}
                fk = _get(f, "f.kind", str)
                if fk not in MLP_KINDS:
                    raise ConfigError(f"config.json: '{at}.mlp.kind' is {fk!r}; known feed-forwards: {list(MLP_KINDS)}")
                if fk == "dense":
                    limit = _get(f, "f.limit", float)
                    if not limit > 0:
                        raise ConfigError(f"config.json: '{at}.mlp.limit' must be positive, got {limit}")
                    mlp = DenseFFConfig(_get(f, "f.ff", int, minimum=1), limit)
                else:
                    mlp = MoeFFConfig(_get(f, "f.expert.ff", int, minimum=1), _get(f, "f.router.experts", int, minimum=1),
                                      _get(f, "f.router.top", int, minimum=1))
                    if mlp.top > mlp.experts:
                        raise ConfigError(f"config.json: '{at}.mlp.router': top {mlp.top} of {mlp.experts} experts")
            wo = L.get("weights_of")
            if wo is not None and (isinstance(wo, bool) or not isinstance(wo, int) or not 0 <= wo < len(layers_in)):
                raise ConfigError(f"config.json: '{at}.weights_of' is {wo!r}; it names one of the {len(layers_in)} layers")
            layers.append(BirepelLayerConfig(kind, mixer, mlp, i if wo is None else wo))
        # a layer that borrows may name one that borrows in turn: follow to the layer that stores the tensors
        owners = []
        for i, L in enumerate(layers):
            j, seen = i, set()
            while layers[j].weights_of != j:
                if j in seen:
                    raise ConfigError(f"config.json: 'layers[{i}].weights_of' leads in a circle")
                seen.add(j)
                j = layers[j].weights_of
            owners.append(j)
        for i, j in enumerate(owners):
            if j != i and (layers[i].type, layers[i].mixer, layers[i].mlp) != (layers[j].type, layers[j].mixer, layers[j].mlp):
                raise ConfigError(f"config.json: 'layers[{i}]' reads the tensors of layer {j} but describes another layer")
        layers = [BirepelLayerConfig(L.type, L.mixer, L.mlp, owners[i]) for i, L in enumerate(layers)]
        eos = d.get("eos_token_id")
        eos_ids = tuple(eos) if isinstance(eos, (list, tuple)) else ((int(eos),) if isinstance(eos, int) else ())
        return cls(vocab=_get(d, "vocab", int, minimum=1), width=_get(d, "width", int, minimum=1),
                   max_positions=_get(d, "max_positions", int, minimum=1), norm_eps=_get(d, "norm.eps", float),
                   layers=tuple(layers), eos_token_ids=eos_ids, bos_token_id=d.get("bos_token_id"))

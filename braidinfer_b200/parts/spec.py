"""Data that describes a model: which parts each layer is made of, and the
order in which layers run.  A description holds names and numbers only; the
parts themselves are built from it by `braidinfer_b200.models.decoder`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: the name it is registered under and its sizes and constants."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (block) of a mixer, a feed-forward and norms.

    `prefix` is put before every tensor name the layer's parts ask for.
    """
    block: str
    prefix: str
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    # a part (registry LAYER_INPUTS) that the block applies to the stream after its other parts: something the
    # layer reads about each token beside the stream
    layer_input: Optional[PartSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `cache_of` names an earlier schedule entry whose
    cache this run reads instead of keeping its own.  `inject`: the model's injection
    (`ModelSpec.injection`) is applied to the stream right before this run."""
    layer: int
    cache_of: Optional[int] = None
    inject: bool = False


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, the order they run in, final norm, head."""
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_position: int = 0                      # longest sequence the model is meant for (0: not stated)
    eos_token_ids: Tuple[int, ...] = ()        # tokens that end a sequence unless the caller names others
    bos_token_id: Optional[int] = None         # put before a text prompt by the command line
    # A part (registry INJECTIONS) that mixes the embedding's output back into the stream before the runs
    # that ask for it (`ScheduleEntry.inject`): a block of layers that runs several times in a row, for one,
    # is fed the stream and the embedding's output anew at the start of every pass.
    injection: Optional[PartSpec] = None

    def validate(self) -> None:
        if self.injection is None and any(e.inject for e in self.schedule):
            raise ValueError("a schedule entry asks for the injection, and the model has none")
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, which does not exist")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(
                        f"schedule entry {i} reads the cache of entry {e.cache_of}, "
                        f"which must be an earlier entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(
                        f"schedule entry {i} reads the cache of entry {e.cache_of}, "
                        f"which has no cache of its own")


@dataclass(frozen=True)
class TensorSpec:
    """A tensor that a part needs from the model folder.

    `init` tells the random-weights mode how to draw it: "normal" is N(0, std),
    "one_plus_normal" is 1 + N(0, std).  A shape of () is one stored scalar.  `integer` marks index tables, which are
    kept as int32 whatever the run's dtype.
    """
    shape: Tuple[int, ...]
    init: str = "normal"
    std: float = 0.02
    integer: bool = False
    optional: bool = False


@dataclass(frozen=True)
class CacheRequest:
    """What a mixer needs kept for each sequence between steps.

    kind "full": keys and values of every past token; "window": of the last
    `window` tokens only.  Layers whose requests are equal share one group of
    storage.  `planes` is how many vectors of `head_dim` a token and kv head keep:
    2 for a key and a value, 1 where one vector serves as both (a latent).  `keep_first` (kind "window"): the
    sequence's first positions stay beside the window, for mixers whose queries see them at any distance.
    """
    kind: str
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    planes: int = 2
    keep_first: int = 0

    def group_key(self) -> Tuple:
        return (self.kind, self.num_kv_heads, self.head_dim, self.window, self.planes, self.keep_first)

"""Token embedding and output head.

Embedding: h[t, :] = float(E[token_t, :]), no scale (reference:
kernels/megakernel_ops.hip:1757-1768); a model may name a constant factor on the rows (`scale`) and a
norm of the scaled rows (`norm`), whose output is then the stream, and a learned vector a position that is added to
a token's row, unscaled (`positions`: the stored table's name and its number of rows).  A model may also cap its logits:
logits <- cap * tanh(logits / cap) (`softcap`).  Head: logits = W h in float32
(kernels/megakernel_ops.hip:1783-1835); W is lm_head.weight, or the embedding table
when the model ties them (crates/braidinfer-runtime/src/model/model_load.rs:388-398).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import EMBEDDINGS, HEADS, NORMS, Embedding, Head
from .linear import Linear
from .spec import TensorSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    """params: vocab_size, hidden_size, name; optional scale (a factor on the rows, default 1), norm
    (a PartSpec of a norm whose `forward` takes `in_place=True`, applied to the scaled rows) and positions
    ({"name", "max"}: a stored table [max, hidden_size]; row p is added to the token at position p of its sequence)."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = prefix + params.get("name", "model.embed_tokens.weight")
        self.scale = float(params.get("scale", 1.0))
        norm = params.get("norm")
        self.norm = NORMS.get(norm.kind)(norm.params, prefix, runtime) if norm is not None else None
        self.weight: Optional[torch.Tensor] = None
        pos = params.get("positions")
        self.pos_name = prefix + pos["name"] if pos else None
        self.max_positions = int(pos["max"]) if pos else 0
        self.uses_positions = bool(pos)
        self.pos_table: Optional[torch.Tensor] = None
        if pos and self.norm is not None:
            raise ValueError("token_embedding: a norm of the rows and a table of positions are not combined")

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = {self.name: TensorSpec((self.vocab, self.hidden))}
        if self.pos_name:
            d[self.pos_name] = TensorSpec((self.max_positions, self.hidden))
        if self.norm is not None:
            d.update(self.norm.tensor_specs())
        return d

    def load(self, tensors) -> None:
        self.weight = tensors[self.name]
        if self.norm is not None:
            self.norm.load(tensors)
        if self.pos_name:
            self.pos_table = tensors[self.pos_name]

    def forward(self, token_ids: torch.Tensor, rows: int, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        h = torch.empty((rows, self.hidden), dtype=torch.float32, device=self.rt.device)
        if self.pos_table is not None and positions is None:
            raise RuntimeError("token_embedding: this model adds a vector a position and needs the rows' positions")
        self.rt.kernels.embed(self.weight, token_ids, h, scale=self.scale, pos_table=self.pos_table,
                              positions=positions if self.pos_table is not None else None)
        if self.norm is not None:
            h = self.norm.forward(h, None, in_place=True)
        return h


@HEADS.register("linear_head")
class LinearHead(Head):
    """params: vocab_size, hidden_size, name, tied (use the embedding table, as stored: a factor that the
    embedding puts on its rows is not part of the table), softcap (a positive cap on the logits, or None)."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        # None: tied exactly when the model folder stores no head tensor.
        self.tied = params.get("tied", False)
        self.name = prefix + params.get("name", "lm_head.weight")
        self.linear = Linear(runtime, [self.name], [self.vocab], self.hidden)
        cap = params.get("softcap")
        self.softcap = float(cap) if cap else None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        if self.tied:
            return {}
        specs = self.linear.tensor_specs()
        if self.tied is None:
            specs = {n: TensorSpec(ts.shape, optional=True) for n, ts in specs.items()}
        return specs

    def load(self, tensors) -> None:
        if self.tied is None:
            self.tied = self.name not in tensors
        if not self.tied:
            self.linear.load(tensors)

    def tie(self, embedding_weight: torch.Tensor) -> None:
        self.linear.share(embedding_weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.linear.forward(x, out_dtype=torch.float32)
        if self.softcap is not None:
            self.rt.kernels.softcap(logits, self.softcap)
        return logits

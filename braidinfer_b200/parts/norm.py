"""Norms of the residual stream.

Dynamic Tanh ("dyt"): y = tanh(alpha * x) * w + b, element by element, with one stored scalar alpha, a
weight and a bias vector: no mean, no variance, nothing shared along a row (Zhu, Chen, He, LeCun, Liu:
"Transformers without Normalization", 2025).  tanh and the products are float32.

RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, plain w
(reference: kernels/megakernel_ops.hip:862-904; `1 + w` is another model family's rule,
crates/braidinfer-runtime/src/config.rs:552).  Reads the float32 residual stream, writes
the run's element type; the sum of squares and the scale are float32.  With `offset` the stored weight w is
zero-centred and applied as offset + w (offset 1: y = x * rsqrt(mean(x^2) + eps) * (1 + w)), added in float32.
`add_into(y, h)` norms a branch's float32 result y and adds it to the float32 stream h in one kernel, for
layers that norm what a sublayer returns instead of what it reads."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import NORMS, Norm
from .linear import ROW_SCALE_MAX_ROWS
from .spec import TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: width, eps, name (tensor name under the prefix), offset (added to the stored weight; default 0)."""

    accepts_deferred = True      # adds a deferred residual sum in the same kernel as the norm

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.name = prefix + params["name"]
        self.offset = float(params.get("offset", 0.0))
        if self.offset:
            self.accepts_deferred = False        # the kernels that add up partial sums apply plain weights
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.width,), init="normal" if self.offset else "one_plus_normal")}

    def add_into(self, y: torch.Tensor, h: torch.Tensor, ctx=None) -> torch.Tensor:
        """h += norm(y), both float32 [rows, width]; returns h."""
        self.rt.kernels.rmsnorm_add(h, y, self.weight, self.eps, w_offset=self.offset)
        return h

    def load(self, tensors) -> None:
        self.weight = tensors[self.name]

    def forward(self, x: torch.Tensor, ctx=None, row_index: Optional[torch.Tensor] = None,
                rows: Optional[int] = None, reader_takes_row_scale: bool = False) -> torch.Tensor:
        n = rows if rows is not None else x.shape[0]
        out = self.rt.empty(n, self.width)
        if self.offset:
            self.rt.kernels.rmsnorm(x, self.weight, out, self.eps, row_index=row_index, w_offset=self.offset)
            return out
        d = ctx.take_deferred(x) if ctx is not None else None
        if (reader_takes_row_scale and self.rt.scaled_norm and ctx is not None and row_index is None and out.dtype == torch.bfloat16
                and n <= ROW_SCALE_MAX_ROWS and self.width % 4 == 0 and self.rt.gemm_backend == "auto"):
            # a step of few tokens: x is completed, `out` = x * weight, and the scale is left to the reader.
            # The kernel works on 512 columns of a row per CTA instead of on whole rows.
            if d is not None and d[1] != "residual":
                raise RuntimeError("a norm can only complete a deferred residual sum")
            ctx.set_row_scale(out, self.rt.kernels.streamk_reduce_prep(d[0] if d is not None else None, x, self.weight,
                                                                       out, self.eps))
            return out
        if d is not None:
            handle, kind = d
            if kind != "residual":
                raise RuntimeError("a norm can only complete a deferred residual sum")
            self.rt.kernels.streamk_reduce_norm(handle, x, self.weight, out, self.eps, row_index=row_index)
        else:
            self.rt.kernels.rmsnorm(x, self.weight, out, self.eps, row_index=row_index)
        return out


@NORMS.register("dyt")
class DynamicTanh(Norm):
    """params: width, name (the weight's tensor name under the prefix; the bias is name + ".b", the scalar
    name + ".alpha")."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.width = int(params["width"])
        self.name = prefix + params["name"]
        self.weight = self.bias = self.alpha = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.width,), init="one_plus_normal"),
                self.name + ".b": TensorSpec((self.width,)),
                self.name + ".alpha": TensorSpec((), init="one_plus_normal")}

    def load(self, tensors) -> None:
        self.weight, self.bias, self.alpha = tensors[self.name], tensors[self.name + ".b"], tensors[self.name + ".alpha"]

    def forward(self, x: torch.Tensor, ctx=None, row_index: Optional[torch.Tensor] = None,
                rows: Optional[int] = None, in_place: bool = False, in_scale: float = 1.0) -> torch.Tensor:
        """`in_place`: x itself is overwritten and stays float32 (an embedding's norm: its output is the
        stream).  `in_scale`: a constant factor on x that the caller has not applied yet."""
        if in_place:
            self.rt.kernels.dyt(x, self.weight, self.bias, self.alpha, x, in_scale=in_scale)
            return x
        n = rows if rows is not None else x.shape[0]
        out = self.rt.empty(n, self.width)
        self.rt.kernels.dyt(x, self.weight, self.bias, self.alpha, out, row_index=row_index, in_scale=in_scale)
        return out

"""Gated feed-forward: down( act(gate x) * (up x) ), added to the residual; act is silu (SwiGLU) unless the
model names another (`activation`: "gelu_tanh" is the tanh form of gelu, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))))
(reference: crates/braidinfer-runtime/src/megakernel/compile_layers.rs:373-386;
kernels/megakernel_ops.hip:1474-1545 gate/up with silu as x / (1 + exp(-x)),
:1559-1602 down with the residual).  Gate and up are one stacked product; on the
tensor-core path the activation is its epilogue.

"clamped_glu": down( g * sigmoid(alpha * g) * (u + 1) ) with g = min(gate x, limit) and u = clamp(up x, -limit, limit):
a gated unit whose two branches are bounded before they meet, and whose linear branch is offset by one.

"biased_mlp": down( f(up x + b_up) ) + b_down, one hidden layer with biases and no gate.  Its activation f is the
two-piece xIELU with two stored numbers (p, q) a layer:
    f(t) = softplus(p) t^2 + t / 2                           t > 0
    f(t) = (1/2 + softplus(q)) (exp(t) - 1 - t) + t / 2      t <= 0
(Huang, Schlag: "Deriving Activation Functions Using Integration", 2024, in the form with both numbers under a
softplus).  The up bias and the activation are one float32 kernel; the down bias is one more column of the down
matrix that meets a column of ones which that kernel writes, so it costs no launch."""
from __future__ import annotations

from typing import Dict

import torch

from .base import FEED_FORWARDS, FeedForward
from .linear import Linear
from .spec import TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size, activation (default "silu"), tensor names gate_proj, up_proj, down_proj."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.activation = p.get("activation", "silu")
        from ..csrc.api import activation_code
        activation_code(self.activation)                 # an unknown name fails here, not at the first step
        self.gate_up = Linear(runtime, [prefix + p.get("gate_proj", "mlp.gate_proj.weight"),
                                        prefix + p.get("up_proj", "mlp.up_proj.weight")],
                              [self.inter, self.inter], self.hidden, gate_up=True)
        self.down = Linear(runtime, [prefix + p.get("down_proj", "mlp.down_proj.weight")], [self.hidden], self.inter)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.gate_up.tensor_specs())
        d.update(self.down.tensor_specs())
        return d

    def load(self, tensors) -> None:
        self.gate_up.load(tensors)
        self.down.load(tensors)

    def takes_row_scale(self) -> bool:
        return self.gate_up.takes_row_scale()

    def forward(self, x, residual, ctx):
        act = self.gate_up.forward(x, swiglu=True, in_scale=ctx.take_row_scale(x) if ctx is not None else None,
                                   activation=self.activation)
        return self.down.forward(act, residual=residual, defer_to=ctx)


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(FeedForward):
    """params: hidden_size, intermediate_size, limit, alpha (default 1.702), tensor names gate_proj, up_proj, down_proj."""

    plain_output = True

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.limit = float(p["limit"])
        self.alpha = float(p.get("alpha", 1.702))
        if not self.limit > 0:
            raise ValueError(f"clamped_glu: the limit must be positive, got {self.limit}")
        self.gate_up = Linear(runtime, [prefix + p.get("gate_proj", "mlp.gate"), prefix + p.get("up_proj", "mlp.up")],
                              [self.inter, self.inter], self.hidden)
        self.down = Linear(runtime, [prefix + p.get("down_proj", "mlp.down")], [self.hidden], self.inter)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.gate_up.tensor_specs())
        d.update(self.down.tensor_specs())
        return d

    def load(self, tensors) -> None:
        self.gate_up.load(tensors)
        self.down.load(tensors)

    def forward(self, x, residual, ctx):
        gu = self.gate_up.forward(x)                           # [rows, gate | up]
        act = self.rt.empty(x.shape[0], self.inter)
        self.rt.kernels.glu_clamp(gu, act, self.limit, self.alpha)
        if residual is None:
            return self.down.forward(act, out_dtype=torch.float32)
        return self.down.forward(act, residual=residual, defer_to=ctx)


@FEED_FORWARDS.register("biased_mlp")
class BiasedMLP(FeedForward):
    """params: hidden_size, intermediate_size, activation ("xielu"), tensor names up_proj, up_bias, down_proj, down_bias,
    act (the activation's two numbers)."""

    plain_output = True

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        if p.get("activation", "xielu") != "xielu":
            raise ValueError(f"biased_mlp: activation {p.get('activation')!r} is not built (xielu)")
        self.inter_pad = -(-(self.inter + 1) // 8) * 8          # the ones column, and rows that start on 16 bytes
        self.up = Linear(runtime, [prefix + p.get("up_proj", "mlp.up")], [self.inter], self.hidden)
        self.down_name = prefix + p.get("down_proj", "mlp.down")
        self.up_bias_name = prefix + p.get("up_bias", "mlp.up.b")
        self.down_bias_name = prefix + p.get("down_bias", "mlp.down.b")
        self.act_name = prefix + p.get("act", "mlp.act")
        self.down = Linear(runtime, [self.down_name], [self.hidden], self.inter_pad)
        self.up_bias = self.act_pq = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.up.tensor_specs())
        d[self.up_bias_name] = TensorSpec((self.inter,))
        d[self.down_name] = TensorSpec((self.hidden, self.inter))
        d[self.down_bias_name] = TensorSpec((self.hidden,))
        d[self.act_name] = TensorSpec((2,), std=0.5)
        return d

    def load(self, tensors) -> None:
        self.up.load(tensors)
        w, b = tensors[self.down_name], tensors[self.down_bias_name]
        if w.dtype != b.dtype:
            w, b = w.float(), b.float()
        pad = torch.zeros((self.hidden, self.inter_pad - self.inter - 1), dtype=w.dtype, device=w.device)
        self.down.share(torch.cat([w, b.view(-1, 1), pad], dim=1).contiguous())      # [hidden, ff | bias | zeros]
        self.up_bias, self.act_pq = tensors[self.up_bias_name], tensors[self.act_name]
        if self.up_bias.dtype != self.act_pq.dtype:
            self.up_bias, self.act_pq = self.up_bias.float(), self.act_pq.float()

    def takes_row_scale(self) -> bool:
        return self.up.takes_row_scale()

    def forward(self, x, residual, ctx):
        z = self.up.forward(x, in_scale=ctx.take_row_scale(x) if ctx is not None else None)
        act = self.rt.empty(x.shape[0], self.inter_pad)
        self.rt.kernels.bias_xielu(z, self.up_bias, self.act_pq, act, self.inter)
        if residual is None:
            return self.down.forward(act, out_dtype=torch.float32)
        return self.down.forward(act, residual=residual, defer_to=ctx)

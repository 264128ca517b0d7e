"""Mixture of experts: each token is sent to a few small SwiGLU feed-forwards and gets back the
weighted sum of their outputs.

    z = Wr x (float32)          s = softmax(z) over all experts
    experts form `groups` equal groups of neighbours; a group's score is its largest s; only experts of
    the `keep` best groups can be chosen; the `top` allowed experts with the largest s are chosen
    weight_k = s_k / (sum of the chosen s + 1e-20)
    out = sum_k weight_k * Wdown_k ( silu(Wgate_k x) * (Wup_k x) )
(Group-limited routing as in DeepSeek-AI, "DeepSeek-V2", 2024.)  Router scores, the choice, the weights
and the weighted sum are float32.

A step's (token, choice) pairs are sorted by expert on the device (`moe_plan`), the experts' products run
over the sorted rows tile by tile, and the weighted sum adds a token's choices in their fixed order, so
what a token gets does not depend on its neighbours in the batch.  Nothing is read back by the host, and
launch sizes follow from the step's shape alone.  A constant factor on the output (`out_mult`) rides on
the weights.

Options for other designs: `gated: False` makes an expert Wdown act(Wup x) without a gate matrix, with
`activation: "relu2"` (the square of relu) as its act.  Softmax over all experts followed by the division by the
chosen scores' sum is the softmax over the chosen logits alone, so routers that are described that way need no
mode of their own.  `scoring: "sigmoid"` scores every expert by itself, s = 1 / (1 + exp(-z)), and the chosen experts'
weights are their scores as they are.  `weight_on: "input"` lets the weight multiply what the expert reads instead
of what it returns, out = sum_k expert_k(w_k x); the first products being linear, the weight is applied to their
float32 results before the activation.  `shared` is a feed-forward part that every token also runs through (its
result is added like an expert's with weight 1).
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import FEED_FORWARDS, FeedForward
from .linear import Linear
from .spec import PartSpec, TensorSpec


@FEED_FORWARDS.register("moe")
class MixtureOfExperts(FeedForward):
    """params: hidden_size, intermediate_size (of one expert), experts, top, groups (default 1), keep
    (groups kept, default all), out_mult (default 1), gated (default True), activation ("silu" with a gate, "relu2"
    without), scoring ("softmax" | "sigmoid"), weight_on ("output" | "input"), shared (a PartSpec of a feed-forward, or
    None), and tensor names: router, and expert_gate, expert_up, expert_down as patterns with `{e}` for the expert's
    number."""

    plain_output = True

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.experts = int(p["experts"])
        self.top = int(p["top"])
        self.groups = int(p.get("groups", 1))
        self.keep = int(p.get("keep", self.groups))
        self.out_mult = float(p.get("out_mult", 1.0))
        self.gated = bool(p.get("gated", True))
        self.activation = p.get("activation", "silu" if self.gated else "relu2")
        if (self.gated, self.activation) not in ((True, "silu"), (False, "relu2")):
            raise ValueError(f"moe: experts {'with' if self.gated else 'without'} a gate and activation "
                             f"{self.activation!r} are not built (silu with a gate, relu2 without)")
        self.scoring = p.get("scoring", "softmax")
        self.weight_on = p.get("weight_on", "output")
        if self.scoring not in ("softmax", "sigmoid") or self.weight_on not in ("output", "input"):
            raise ValueError(f"moe: scoring {self.scoring!r} (softmax or sigmoid), weight_on {self.weight_on!r} (output or input)")
        if self.weight_on == "input" and not self.gated:
            raise ValueError("moe: a weight on the expert's input is built for gated experts")
        sh: PartSpec = p.get("shared")
        self.shared = FEED_FORWARDS.get(sh.kind)(sh.params, prefix, runtime) if sh is not None else None
        if self.experts % self.groups:
            raise ValueError(f"{self.experts} experts do not form {self.groups} equal groups")
        if not (1 <= self.keep <= self.groups):
            raise ValueError(f"{self.keep} groups kept of {self.groups}")
        if not (1 <= self.top <= self.keep * (self.experts // self.groups)):
            raise ValueError(f"top {self.top} of {self.keep} groups of {self.experts // self.groups} experts")
        self.router = Linear(runtime, [prefix + p.get("router", "mlp.router")], [self.experts], self.hidden)
        self.gate_names = [prefix + p.get("expert_gate", "mlp.e{e}.gate").format(e=e) for e in range(self.experts)]
        self.up_names = [prefix + p.get("expert_up", "mlp.e{e}.up").format(e=e) for e in range(self.experts)]
        self.down_names = [prefix + p.get("expert_down", "mlp.e{e}.down").format(e=e) for e in range(self.experts)]
        self.w_gate = self.w_up = self.w_down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.router.tensor_specs())
        for e in range(self.experts):
            if self.gated:
                d[self.gate_names[e]] = TensorSpec((self.inter, self.hidden))
            d[self.up_names[e]] = TensorSpec((self.inter, self.hidden))
            d[self.down_names[e]] = TensorSpec((self.hidden, self.inter))
        if self.shared is not None:
            d.update(self.shared.tensor_specs())
        return d

    def load(self, tensors) -> None:
        self.router.load(tensors)
        if self.shared is not None:
            self.shared.load(tensors)
        if self.gated:
            self.w_gate = torch.stack([tensors[n] for n in self.gate_names]).contiguous() # [experts, inter, hidden]
        self.w_up = torch.stack([tensors[n] for n in self.up_names]).contiguous()
        self.w_down = torch.stack([tensors[n] for n in self.down_names]).contiguous()     # [experts, hidden, inter]

    def tile(self, rows: int) -> int:
        """Slots a tile of the plan: 16 while an expert sees few rows, 64 beyond."""
        return 16 if rows * self.top <= 16 * self.experts else 64

    def forward(self, x, residual, ctx):
        K = self.rt.kernels
        rows = x.shape[0]
        logits = self.router.forward(x, out_dtype=torch.float32)
        idx = torch.empty((rows, self.top), dtype=torch.int32, device=x.device)
        wgt = torch.empty((rows, self.top), dtype=torch.float32, device=x.device)
        K.moe_route(logits, idx, wgt, self.groups, self.keep, mult=self.out_mult, sigmoid=self.scoring == "sigmoid")
        tile = self.tile(rows)
        plan = K.moe_plan(idx, ctx.token_seq, self.experts, tile)
        slots = plan[4] * tile
        act = self.rt.empty(slots, self.inter)
        y = self.rt.empty(slots, self.hidden)
        on_input = self.weight_on == "input"
        self._experts(x, act, y, plan, tile, wgt if on_input else None)
        if residual is None:
            residual = torch.zeros((rows, self.hidden), dtype=torch.float32, device=x.device)
        K.moe_combine(residual, y, plan, None if on_input else wgt, top=self.top)
        if self.shared is not None:
            residual = self.shared.forward(x, residual, ctx)
        return residual

    def _experts(self, x, act, y, plan, tile, in_wgt=None) -> None:
        """bfloat16 rows that start on 16 bytes run on the tensor cores, everything else on the plain kernels."""
        K = self.rt.kernels
        tc = self.rt.gemm_backend == "auto"
        w0, w1 = (self.w_gate, self.w_up) if self.gated else (self.w_up, None)
        relu2 = not self.gated
        if tc and K.moe_gemm_mma_eligible(x, w0, tile) and K.moe_gemm_mma_eligible(act, self.w_down, tile):
            K.moe_gemm_mma(x, w0, w1, act, plan, self.top, tile, relu2=relu2, in_wgt=in_wgt)
            K.moe_gemm_mma(act, self.w_down, None, y, plan, self.top, tile)
            return
        K.moe_gemm_simt(x, w0, w1, act, plan, self.top, tile, relu2=relu2, in_wgt=in_wgt)
        K.moe_gemm_simt(act, self.w_down, None, y, plan, self.top, tile)

"""Matrix memory with exponential gates (the mLSTM of Beck, Pöppel, Spanring, Auer, Prudnikova, Kopp, Klambauer,
Brandstetter, Hochreiter: "xLSTM: Extended Long Short-Term Memory", 2024): a matrix of state and a normaliser per
head instead of a cache of keys and values.

For the mixer's input x (a row per token), per head with key size dk and value size dv:
    q = Wq x * dk^-1/2,   k = Wk x,   v = Wv x,   g = Wg x
    li = cap tanh((Wi x + bi) / cap)                      log of the input gate, kept inside (-cap, cap)
    lf = log sigmoid(cap tanh((Wf x + bf) / cap))         log of the forget gate
    m_t = max(lf + m_(t-1), li)                           a running maximum that keeps the exponentials in range; m_0 = 0
    S_t = exp(lf + m_(t-1) - m_t) S_(t-1) + exp(li - m_t) k v^T          S is [dk, dv], zero at the start
    n_t = exp(lf + m_(t-1) - m_t) n_(t-1) + exp(li - m_t) k
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
    out = Wo ( concat_heads( o / sqrt(mean(o^2) + eps) ) * w * sigmoid(g) )      w: a weight per column of all heads
The gates' logits leave their product in float32; the gates, m, both factors, the recurrence, its state, the
read-out and the norm are float32 in every run.  S, n (as one more column of S whose value is always 1) and m
live in the sequence's slot of the state area and are carried from step to step, so a prompt may be cut anywhere.
Per step: one stacked product (q | k | v | g), the gates' small product, the gate kernel (walks m along each
sequence), the recurrence kernel that the other recurrent mixers use (decays and key factors given), the
read-out kernel, the output product.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import MIXERS, Mixer
from .linear import Linear
from .spec import TensorSpec


@MIXERS.register("mlstm")
class MLSTM(Mixer):
    """params: hidden_size, num_heads, dim (key size a head), vdim (value size a head), gate_cap, eps, and the tensor
    names q, k, v, g, i, f, i_bias, f_bias, norm, o (under the prefix)."""

    plain_output = True

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dk = int(p["dim"])
        self.dv = int(p["vdim"])
        self.cap = float(p["gate_cap"])
        self.eps = float(p["eps"])
        if not self.cap > 0:
            raise ValueError(f"mlstm: gate_cap must be positive, got {self.cap}")
        if self.dk > 256:
            raise ValueError(f"mlstm: key sizes up to 256 a head are built, not {self.dk}")
        H, dk, dv = self.heads, self.dk, self.dv
        self.cols = [H * dk, H * dk, H * dv, H * dv]
        self.proj = Linear(runtime, [prefix + p.get(n, "mix." + n) for n in ("q", "k", "v", "g")], self.cols, self.hidden)
        self.gates = Linear(runtime, [prefix + p.get("i", "mix.i"), prefix + p.get("f", "mix.f")], [H, H], self.hidden)
        self.bias_names = (prefix + p.get("i_bias", "mix.i.b"), prefix + p.get("f_bias", "mix.f.b"))
        self.norm_name = prefix + p.get("norm", "mix.norm")
        self.o = Linear(runtime, [prefix + p.get("o", "mix.o")], [self.hidden], H * dv)
        self.bias_i = self.bias_f = self.norm_w = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.proj.tensor_specs())
        d.update(self.gates.tensor_specs())
        d[self.bias_names[0]] = TensorSpec((self.heads,), std=1.0)
        d[self.bias_names[1]] = TensorSpec((self.heads,), std=1.0)
        d[self.norm_name] = TensorSpec((self.heads * self.dv,), init="one_plus_normal")
        d.update(self.o.tensor_specs())
        return d

    def load(self, tensors) -> None:
        self.proj.load(tensors)
        self.gates.load(tensors)
        self.o.load(tensors)
        self.bias_i, self.bias_f = tensors[self.bias_names[0]], tensors[self.bias_names[1]]
        self.norm_w = tensors[self.norm_name]

    # the state of a sequence: S with the normaliser as its last column [heads, dk, dv + 1], then m [heads]; float32
    def _m_offset(self) -> int:
        return self.heads * self.dk * (self.dv + 1) * 4

    def state_bytes(self) -> int:
        return self._m_offset() + self.heads * 4

    def forward(self, x, residual, ctx, cache, state):
        if state is None:
            raise RuntimeError("mlstm needs its state area")
        K = self.rt.kernels
        rows = x.shape[0]
        H, dk, dv = self.heads, self.dk, self.dv
        proj = self.proj.forward(x)                                     # [rows, q | k | v | g]
        c = [0]
        for n in self.cols:
            c.append(c[-1] + n)
        q, k, v, g = (proj[:, c[i]:c[i + 1]] for i in range(4))
        z = self.gates.forward(x, out_dtype=torch.float32)              # [rows, input gates | forget gates], logits
        gates = torch.empty((rows, 3 * H), dtype=torch.float32, device=x.device)     # decays | key factors | floors
        K.mlstm_gates(z, self.bias_i, self.bias_f, gates, state, self._m_offset(), ctx, H, self.cap)
        o = torch.empty((rows, H * (dv + 1)), dtype=torch.float32, device=x.device)
        K.linear_scan(q, k, v, gates[:, :H], self.bias_i, o, state, 0, ctx, H, H, dk, dv + 1, "given",
                      q_scale=dk ** -0.5, kappa=gates[:, H:2 * H], v_cols=dv)
        y = self.rt.empty(rows, H * dv)
        K.mlstm_out(o, gates[:, 2 * H:], g, self.norm_w, y, ctx.token_seq, H, dv, self.eps)
        if residual is None:
            return self.o.forward(y, out_dtype=torch.float32)
        return self.o.forward(y, residual=residual, defer_to=ctx)

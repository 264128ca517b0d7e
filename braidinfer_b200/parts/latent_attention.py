"""Latent attention: one low-rank vector per token stands for the keys and values of all heads.

For the mixer's input x (a row per token):
    q            = Wq x                      per head [dim unrotated | rot_dim rotated] numbers
    [c' ; kr']   = Wdkv x                    kv_rank + rot_dim numbers
    c            = c' / sqrt(mean(c'^2) + eps) * w_norm           (the latent)
    kr           = rotate(kr', position)     (one rotated key part, shared by all heads)
    head h:  key = [Wuk_h c ; kr],  value = Wuv_h c
    score(i, j)  = (q_u(i) . Wuk_h c(j) + rotate(q_r(i)) . kr(j)) * scale,   j <= i, softmax over j
    out          = Wo concat_h( sigmoid(Wg x)_h * sum_j p(i, j) Wuv_h c(j) )
(Multi-head latent attention as in DeepSeek-AI, "DeepSeek-V2", 2024; the output gate per head is this
part's own option.)  Only c and kr are cached: kv_rank + rot_dim numbers a token, whatever the head count.

The cache is never expanded into keys and values.  q_u . (Wuk_h c) = (Wuk_h^T q_u) . c, so each query
head is carried into the latent space (`gemm_heads` with Wuk_h^T), attention runs as multi-query
attention over the cached rows (key: the whole row; value: its first kv_rank numbers), and the head's
output is Wuv_h applied to the attended latent (`gemm_heads` again, with the gate in its epilogue).  Wuk
and Wuv are used as stored; per-head transposes are made once at load, no product of weights is formed.

A constant factor on the mixer's output (`out_mult`, a model's residual multiplier) rides on the gate.

Options for other designs: the rotation may pair neighbours (2i, 2i + 1) instead of halves (the position encoding's
`pairing`); `window` limits a query to the last `window` positions, itself included; `shared_kv` makes a layer
without a down-projection of its own: it reads the latent and the rotated key part that an earlier layer cached
(the schedule's `cache_of`), with its own queries, Wuk, Wuv, window and output; `cache_window` widens what the
cache keeps beyond the layer's own window, for readers with a longer one.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import MIXERS, POSITION_ENCODINGS, Mixer
from .linear import Linear
from .spec import CacheRequest, PartSpec, TensorSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """params: hidden_size, num_heads, dim (unrotated query/key numbers a head), rot_dim (rotated ones),
    vdim (value size a head), kv_rank, scale (on the scores), eps (of the latent's RMS norm), window
    (int | None), out_mult (default 1), gated (default True), position_encoding (a PartSpec of kind "rope"
    with head_dim = rot_dim: its rope_dim leading numbers of the rotated part turn), shared_kv (default False),
    cache_window (default: window), and the tensor names q, dkv, dkv_norm, uk, uv, g, o (under the prefix)."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dim = int(p["dim"])
        self.rot = int(p["rot_dim"])
        self.vdim = int(p["vdim"])
        self.rank = int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.window = p.get("window")
        self.out_mult = float(p.get("out_mult", 1.0))
        self.gated = bool(p.get("gated", True))
        pe: PartSpec = p["position_encoding"]
        self.pe = POSITION_ENCODINGS.get(pe.kind)(pe.params, prefix, runtime)
        if self.pe.head_dim != self.rot or getattr(self.pe, "amplitude", 1.0) != 1.0:
            raise ValueError("latent_attention rotates the rot_dim part of queries and the shared key part, without a "
                             "factor on sine and cosine")
        self.adjacent = getattr(self.pe, "pairing", "half") == "adjacent"
        self.shared_kv = bool(p.get("shared_kv", False))
        self.cache_window = p.get("cache_window") or self.window
        if self.window and self.cache_window < self.window:
            raise ValueError("latent_attention: the cache must keep at least the layer's own window")
        self.q_cols = self.heads * (self.dim + self.rot)
        self.D = self.rank + self.rot
        names, outs = [prefix + p.get("q", "mix.q")], [self.q_cols]
        if not self.shared_kv:
            names.append(prefix + p.get("dkv", "mix.dkv"))
            outs.append(self.D)
        self.gate_col = sum(outs)
        if self.gated:
            names.append(prefix + p.get("g", "mix.g"))
            outs.append(self.heads)
        self.proj = Linear(runtime, names, outs, self.hidden)          # one stacked product: q, [c' ; kr'], gate
        self.norm_name = prefix + p.get("dkv_norm", "mix.dkv.norm")
        self.uk_name = prefix + p.get("uk", "mix.uk")
        self.uv_name = prefix + p.get("uv", "mix.uv")
        self.o = Linear(runtime, [prefix + p.get("o", "mix.o")], [self.hidden], self.heads * self.vdim)
        self.norm_w = self.uk_t = self.uv = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.proj.tensor_specs())
        if not self.shared_kv:
            d[self.norm_name] = TensorSpec((self.rank,), init="one_plus_normal")
        d[self.uk_name] = TensorSpec((self.heads * self.dim, self.rank))
        d[self.uv_name] = TensorSpec((self.heads * self.vdim, self.rank))
        d.update(self.o.tensor_specs())
        d.update(self.pe.tensor_specs())
        return d

    def load(self, tensors) -> None:
        self.proj.load(tensors)
        w = self.proj.weight
        pad = -w.shape[0] % 8            # rows of zeros, so that a row of the stacked result starts on 16 bytes
        if pad:
            self.proj.weight = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)]).contiguous()
        self.o.load(tensors)
        self.pe.load(tensors)
        self.norm_w = tensors[self.norm_name] if not self.shared_kv else None
        # [heads, kv_rank, dim]: head h's matrix that carries q_u into the latent space, [out, in]
        self.uk_t = tensors[self.uk_name].view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.uv = tensors[self.uv_name].view(self.heads, self.vdim, self.rank).contiguous()

    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest("window" if self.window else "full", 1, self.D, self.cache_window if self.window else None, planes=1)

    def forward(self, x, residual, ctx, cache, state):
        if cache is None:
            raise RuntimeError("latent_attention needs a cache view")
        K = self.rt.kernels
        rows = x.shape[0]
        proj = self.proj.forward(x)                                   # [rows, q | c' kr' | gate | padding]
        q_lat = self.rt.empty(rows, self.heads, self.D)
        writable = not cache.read_only
        if self.shared_kv and writable:
            raise RuntimeError("latent_attention: a layer without a down-projection reads another layer's cache (cache_of)")
        K.latent_prep(proj, self.q_cols, self.norm_w, self.pe.inv_freq, ctx.positions, ctx.token_seq,
                      cache.page_table if writable else None, cache.storage if writable else None, q_lat,
                      self.heads, self.dim, self.rot, self.rank, self.pe.rope_dim, cache.page_size, self.eps,
                      adjacent=self.adjacent)
        q_u = proj[:, :self.q_cols].view(rows, self.heads, self.dim + self.rot)[:, :, :self.dim]
        tc = self.rt.gemm_backend == "auto"
        K.gemm_heads(q_u, self.uk_t, q_lat[:, :, :self.rank], tensor_cores=tc)
        o_lat = self.rt.empty(rows, self.heads, self.rank)
        self._attend(q_lat, o_lat, ctx, cache)
        out = self.rt.empty(rows, self.heads * self.vdim)
        gate = proj[:, self.gate_col:self.gate_col + self.heads] if self.gated else None
        if gate is None and self.out_mult != 1.0:
            raise RuntimeError("latent_attention: an output factor needs the gate's epilogue")
        K.gemm_heads(o_lat, self.uv, out.view(rows, self.heads, self.vdim), gate=gate, mult=self.out_mult, tensor_cores=tc)
        return self.o.forward(out, residual=residual, defer_to=ctx)

    def _attend(self, q_lat, o_lat, ctx, cache) -> None:
        """bfloat16 runs use the tensor-core kernel where it is built for the latent's size (prompts and decoding
        alike; steps of few tokens slice the context so that a handful of sequences still fills the machine);
        float32 runs, runs that ask for the plain kernels, and other sizes use one warp per (token, head)."""
        K = self.rt.kernels
        if self.rt.is_f32 or self.rt.attention_backend == "plain" or not K.attn_latent_mma_supports(self.rank, self.rot):
            K.attn_latent_simple(q_lat, o_lat, cache.storage, cache.page_table, ctx.positions, ctx.token_seq,
                                 self.rank, self.window, self.scale)
            return
        if ctx.rows > ctx.n_tokens:
            o_lat.zero_()                                     # rows of padding are not written by the kernel
        n_splits = 1
        if ctx.max_q_len <= 8:
            ctas = K.attn_latent_ctas(self.rank, self.rot, ctx.n_seqs, ctx.max_q_len, self.heads)
            span = min(ctx.max_kv_len, self.window) if self.window else ctx.max_kv_len
            tiles = max(1, -(-span // 32))
            n_splits = max(1, min(296 // ctas, tiles // 4, 32))      # two CTAs an SM, at least four key tiles a slice
        K.attn_latent_mma(q_lat, o_lat, cache.storage, cache.page_table, ctx.q_start, ctx.q_len, ctx.kv_before,
                          ctx.token_seq, ctx.n_seqs, ctx.max_q_len, self.rank, self.window, self.scale, n_splits=n_splits)

"""Grouped-query attention with an optional sliding window.

norm'd tokens -> q, k, v (one stacked product) -> position encoding, keys and values
into the cache -> attention over the cache -> output projection added to the residual
(reference: crates/braidinfer-runtime/src/megakernel/compile_attention.rs:79-126, 275-351;
softmax in kernels/megakernel_ops.hip:2310-2342).  Head h reads kv head h // g.  Key j is
visible to the query at position p iff j <= p and (no window or p - j < window); the
reference has no window (crates/braidinfer-runtime/src/config.rs:416).

Options that other designs use, each off unless named:
    qk_norm         every query and key head is RMS-normed over the head, with a weight of head_dim numbers
                    shared by the heads (plain weight), before the rotation
    value_from_key  there is no value projection: a token's value is its key as projected, before norm and
                    rotation (the cache then holds the rotated key and the raw one)
    scale           the factor on the scores (default head_dim^-1/2)
    sink            one more term exp(sink) in the softmax's denominator that has no value:
                    p_j = exp(s_j) / (exp(sink) + sum_i exp(s_i)); a row may so give weight to nothing
    out_mult        a constant factor on the mixer's result
    sink_name       a learned sink score a head (a stored tensor of num_heads numbers) instead of the constant `sink`
    head_gate       a gate a head on the result: head h's output is multiplied by sigmoid(Wg x)_h, Wg a stored
                    [num_heads, hidden] tensor whose rows ride in the stacked product; the attention kernels apply it
    unit_qk_eps     every query and key head is divided by its root mean square, sqrt(mean(x^2) + eps), no weight
    q_temp          {"coef", "every"}: the query at position p is multiplied by
                    1 + coef * ln(floor((p + 1) / every) + 1), a temperature that sharpens long contexts
    value_dim       the size of a value head where it differs from head_dim
    keep_first      with a window: a sequence's first keep_first positions stay visible at any distance (key j is seen from
                    position p iff j <= p and (p - j < window or j < keep_first)); they keep their true positions
    head_scale      a stored tensor of num_heads numbers: head h's scores are multiplied by head_scale[h] (float32)
    talk            a stored [num_heads, num_heads] tensor T that mixes the heads' probabilities after the softmax,
                    p'_h = sum_g T[h, g] p_g; head h applies p'_h to the values of its own kv head.  The mix is linear, so
                    every head's own probabilities are applied to the values of every kv head (the attention kernels'
                    `value_heads`) and the results are mixed afterwards, out_h = sum_g T[h, g] O[g, kv(h)] (`head_mix`)
unit_qk_eps, q_temp and value_dim without rotation are for heads that are not rotated (position encoding "none"): one kernel norms, scales and
stores.  Keys, values and queries are then padded with zeros to one head size that the attention kernels take
(max(head_dim, value_dim), rounded up to 16), which changes no score and no result.  Rotated heads whose value
size differs from head_dim (or whose size is no multiple of 16) get the same padding from rows of zeros in the
stacked projection, put there when the weights are loaded.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .base import MIXERS, POSITION_ENCODINGS, Mixer
from .linear import Linear
from .spec import CacheRequest, PartSpec, TensorSpec


@MIXERS.register("gqa_attention")
class GQAAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, window (int | None),
    position_encoding (PartSpec), and tensor names q_proj, k_proj, v_proj, o_proj; optional qk_norm
    ({"eps", "q_name", "k_name"}), value_from_key (bool), scale, sink (a score), out_mult, sink_name, head_gate,
    unit_qk_eps, q_temp ({"coef", "every"}), value_dim, keep_first, head_scale (a tensor name), talk (a tensor name)."""

    plain_output = True

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nqh = int(p["num_heads"])
        self.nkh = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.window = p.get("window")
        if self.nqh % self.nkh:
            raise ValueError(f"{self.nqh} query heads do not divide into {self.nkh} kv heads")
        pe: PartSpec = p["position_encoding"]
        self.value_from_key = bool(p.get("value_from_key", False))
        self.vd = int(p.get("value_dim") or self.hd)
        self.unit_qk_eps = float(p["unit_qk_eps"]) if p.get("unit_qk_eps") is not None else None
        qt = p.get("q_temp")
        self.q_temp = (float(qt["coef"]), int(qt["every"])) if qt else None
        if self.q_temp and self.q_temp[1] < 1:
            raise ValueError(f"gqa_attention: q_temp.every must be at least 1, got {self.q_temp[1]}")
        # heads that are normed without weights, scaled by position or of two sizes go through the kernel that
        # pads them to one size
        gated = p.get("head_gate") is not None
        self.prep = (self.unit_qk_eps is not None or self.q_temp is not None or (self.vd != self.hd and pe.kind == "none")
                     or (gated and pe.kind == "none"))
        if gated and not self.prep and not (p.get("qk_norm") is not None or self.value_from_key):
            raise ValueError("gqa_attention: a gate a head rides in the stacked product, which the plain rotation kernels "
                             "take without further columns; it goes with head norms or with heads that are not rotated")
        self.hd_pad = -(-max(self.hd, self.vd) // 16) * 16 if self.prep else self.hd
        self.keep_first = int(p.get("keep_first") or 0)
        self.head_scale_name = prefix + p["head_scale"] if p.get("head_scale") is not None else None
        self.talk_name = prefix + p["talk"] if p.get("talk") is not None else None
        self.head_scale = self.talk = None
        # rotated heads with a value size of their own, or of a size the tensor-core kernels do not take: rows of zeros in
        # the stacked projection pad every head to one size
        self.pad_rows = (not self.prep and pe.kind != "none" and not self.value_from_key and p.get("qk_norm") is None
                         and (self.vd != self.hd or (self.hd % 16 and (self.talk_name or self.keep_first))))
        if self.pad_rows:
            self.hd_pad = -(-max(self.hd, self.vd) // 16) * 16
        if self.vd != self.hd and not (self.prep or self.pad_rows):
            raise ValueError("gqa_attention: a value size of its own goes with plainly rotated heads or with heads without rotation")
        if self.keep_first and not self.window:
            raise ValueError("gqa_attention: keep_first goes with a window")
        if self.talk_name and (gated or p.get("sink") is not None or p.get("sink_name") is not None):
            raise ValueError("gqa_attention: the mix of the heads' probabilities is built for an ordinary softmax without "
                             "sink or gate")
        pe_params = dict(pe.params)
        if self.pad_rows:
            pe_params["head_dim"] = self.hd_pad          # the rotation still turns the first rope_dim numbers of a head
        self.pe = POSITION_ENCODINGS.get(pe.kind)(pe_params, prefix, runtime)
        if self.prep and (pe.kind != "none" or self.value_from_key or p.get("qk_norm") is not None):
            raise ValueError("gqa_attention: unit norms, a query temperature and a value size of its own are for heads "
                             "without rotation, weighted head norms or keys as values")
        names = [prefix + p.get("q_proj", "self_attn.q_proj.weight"), prefix + p.get("k_proj", "self_attn.k_proj.weight")]
        outs = [self.nqh * self.hd, self.nkh * self.hd]
        if not self.value_from_key:
            names.append(prefix + p.get("v_proj", "self_attn.v_proj.weight"))
            outs.append(self.nkh * self.vd)
        self.gate_col = None
        if p.get("head_gate") is not None:
            self.gate_col = sum(outs)
            names.append(prefix + p["head_gate"])
            outs.append(self.nqh)
        self.qkv = Linear(runtime, names, outs, self.hidden)
        self.o = Linear(runtime, [prefix + p.get("o_proj", "self_attn.o_proj.weight")], [self.hidden],
                        self.nqh * self.vd)
        self.sink_name = prefix + p["sink_name"] if p.get("sink_name") is not None else None
        self.head_sinks = None
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.sink = float(p["sink"]) if p.get("sink") is not None else None
        self.out_mult = float(p.get("out_mult", 1.0))
        qn = p.get("qk_norm")
        self.qk_norm = None
        if qn is not None:
            self.qk_norm = (float(qn["eps"]), prefix + qn["q_name"], prefix + qn["k_name"])
        self.q_norm_w = self.k_norm_w = None
        if (self.qk_norm or self.value_from_key) and not hasattr(self.pe, "norm_encode_and_store"):
            raise ValueError(f"position encoding '{pe.kind}' cannot norm heads or store a key as the value")

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.qkv.tensor_specs())
        d.update(self.o.tensor_specs())
        d.update(self.pe.tensor_specs())
        if self.qk_norm:
            d[self.qk_norm[1]] = TensorSpec((self.hd,), init="one_plus_normal")
            d[self.qk_norm[2]] = TensorSpec((self.hd,), init="one_plus_normal")
        if self.sink_name:
            d[self.sink_name] = TensorSpec((self.nqh,), std=1.0)
        if self.head_scale_name:
            d[self.head_scale_name] = TensorSpec((self.nqh,), init="one_plus_normal", std=0.1)
        if self.talk_name:
            d[self.talk_name] = TensorSpec((self.nqh, self.nqh), std=0.3)
        return d

    def load(self, tensors) -> None:
        self.qkv.load(tensors)
        w = self.qkv.weight
        pad = -w.shape[0] % 8            # rows of zeros, so that a row of the stacked result starts on 16 bytes
        if pad and (self.qk_norm or self.value_from_key):     # (the plain rotation kernels take rows without padding)
            self.qkv.weight = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)]).contiguous()
        if self.pad_rows:
            # every head of q, k and v padded with rows of zeros to hd_pad: no score and no result changes
            w, D = self.qkv.weight, self.hd_pad
            parts, at = [], 0
            for heads, size in ((self.nqh, self.hd), (self.nkh, self.hd), (self.nkh, self.vd)):
                blk = w[at:at + heads * size].view(heads, size, w.shape[1])
                at += heads * size
                parts.append(torch.cat([blk, torch.zeros((heads, D - size, w.shape[1]), dtype=w.dtype, device=w.device)], 1)
                             .reshape(heads * D, w.shape[1]))
            self.qkv.weight = torch.cat(parts).contiguous()
        self.o.load(tensors)
        self.pe.load(tensors)
        if self.head_scale_name:
            self.head_scale = tensors[self.head_scale_name].float().contiguous()   # scores are float32 in every run
        if self.talk_name:
            self.talk = tensors[self.talk_name].contiguous()
        if self.qk_norm:
            self.q_norm_w, self.k_norm_w = tensors[self.qk_norm[1]], tensors[self.qk_norm[2]]
        if self.sink_name:
            self.head_sinks = tensors[self.sink_name].float().contiguous()       # scores are float32 in every run

    def cache_request(self) -> Optional[CacheRequest]:
        kind = "window" if self.window else "full"
        return CacheRequest(kind, self.nkh, self.hd_pad, self.window, keep_first=self.keep_first if self.window else 0)

    def takes_row_scale(self) -> bool:
        return self.qkv.takes_row_scale()

    def forward(self, x, residual, ctx, cache, state):
        if cache is None:
            raise RuntimeError("gqa_attention needs a cache view")
        rt = self.rt
        fused = self.pe.accepts_deferred and not self.prep
        qkv = self.qkv.forward(x, defer_to=ctx if fused else None, in_scale=ctx.take_row_scale(x))
        gate = qkv[:, self.gate_col:self.gate_col + self.nqh] if self.gate_col is not None else None
        if self.prep:
            return self._forward_padded(qkv, gate, residual, ctx, cache)
        if self.qk_norm or self.value_from_key:
            self.pe.norm_encode_and_store(qkv, self.nqh, self.nkh, ctx, cache, self.q_norm_w, self.k_norm_w,
                                          self.qk_norm[0] if self.qk_norm else 0.0, self.value_from_key)
        else:
            self.pe.encode_and_store(qkv, self.nqh, self.nkh, ctx, cache)
        rows = x.shape[0]
        D = self.hd_pad
        if self.talk is not None:
            # every head's probabilities over the values of every kv head, then the mix of the heads
            wide = rt.empty(rows, self.nqh * self.nkh * D)
            self._attend(qkv, wide, ctx, cache, D, value_heads=self.nkh)
            out = rt.empty(rows, self.nqh * self.vd)
            rt.kernels.head_mix(wide, self.talk, out, ctx.token_seq, self.nqh, self.nkh, D, self.vd)
            return self._project(out, residual, ctx)
        out = rt.empty(rows, self.nqh * D)
        self._attend(qkv, out, ctx, cache, D, gate)
        if D != self.vd:
            y = rt.empty(rows, self.nqh * self.vd)
            rt.kernels.head_gate(out, None, y, self.nqh, D, self.vd)
            out = y
        return self._project(out, residual, ctx)

    def _project(self, out, residual, ctx):
        if residual is None:
            return self.o.forward(out, out_dtype=torch.float32)
        return self.o.forward(out, residual=residual, defer_to=ctx)

    def _forward_padded(self, qkv, gate, residual, ctx, cache):
        """Heads without rotation: norm, temperature and the padding to one head size in one kernel, attention over
        the padded heads, then the value columns alone go on to the output product."""
        K = self.rt.kernels
        rows, D = qkv.shape[0], self.hd_pad
        q = self.rt.empty(rows, self.nqh * D)
        coef, every = self.q_temp if self.q_temp else (0.0, 0)
        write = cache is not None and not cache.read_only
        K.head_prep_kv(qkv, q, ctx.positions, ctx.token_seq, cache.page_table if write else None,
                       cache.storage if write else None, self.nqh, self.nkh, self.hd, self.vd, D,
                       self.unit_qk_eps is not None, self.unit_qk_eps or 0.0, coef, every)
        out = self.rt.empty(rows, self.nqh * D)
        self._attend(q, out, ctx, cache, D, gate)
        if D != self.vd:
            y = self.rt.empty(rows, self.nqh * self.vd)
            K.head_gate(out, None, y, self.nqh, D, self.vd)
            out = y
        return self._project(out, residual, ctx)

    def _attend(self, qkv, out, ctx, cache, hd, gate=None, value_heads: int = 1) -> None:
        """Pick the attention kernel for this step.  float32 runs, and runs that ask for
        the plain kernels, use the one-warp-per-query kernel for everything.  bfloat16
        runs use the tcgen05 kernel for prompts (head sizes 64 and 128; "mma" as the
        backend keeps them on the mma.sync kernel, which also serves every other head
        size), and the mma.sync kernel with the context sliced for steps of few tokens,
        so that a handful of sequences still fills the machine."""
        K = self.rt.kernels
        plain = (self.rt.is_f32 or self.rt.attention_backend == "plain" or not K.attn_mma_supports(hd))
        extras = bool(self.keep_first) or self.head_scale is not None or value_heads > 1
        if plain:
            K.attn_simple(qkv, out, cache.storage, cache.page_table, ctx.positions, ctx.token_seq,
                          self.nqh, self.nkh, hd, cache.page_size, self.window, self.scale, sink=self.sink,
                          head_sinks=self.head_sinks, head_gate=gate, out_scale=self.out_mult,
                          keep_first=self.keep_first, head_scale=self.head_scale, value_heads=value_heads)
            return
        few = ctx.max_q_len <= 8
        if not few and self.rt.attention_backend == "auto" and K.attn_tc_supports(hd) and not extras:
            K.attn_tc(qkv, out, cache.storage, cache.page_table, ctx.q_start, ctx.q_len, ctx.kv_before,
                      ctx.n_seqs, ctx.max_q_len, self.nqh, self.nkh, hd, self.window, self.scale, sink=self.sink,
                      head_sinks=self.head_sinks, head_gate=gate, out_scale=self.out_mult)
            return
        n_splits = 1
        if few:
            g = self.nqh // self.nkh
            ctas = ctx.n_seqs * self.nkh * -(-g // 16) * (value_heads // K.attn_value_heads_a_launch(hd, value_heads))
            span = min(ctx.max_kv_len, self.window + self.keep_first) if self.window else ctx.max_kv_len
            tiles = max(1, -(-span // 32))
            # one wave of CTAs over the device, and at least four key tiles a slice
            n_splits = max(1, min(K.attn_decode_slots(hd, value_heads) // ctas, tiles // 4, 64))
        K.attn_mma(qkv, out, cache.storage, cache.page_table, ctx.q_start, ctx.q_len, ctx.kv_before, ctx.token_seq,
                   ctx.n_seqs, ctx.max_q_len, self.nqh, self.nkh, hd, self.window, self.scale,
                   n_splits=n_splits, few_tokens=few, sink=self.sink, head_sinks=self.head_sinks, head_gate=gate,
                   out_scale=self.out_mult, keep_first=self.keep_first, head_scale=self.head_scale,
                   value_heads=value_heads)

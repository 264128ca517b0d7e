"""A plain, slow Ludazen: float64, whole sequences, one function per mechanism, written from the design's
equations and sharing no code with the package.  It reads config.json's dictionary itself.

Notation: T tokens, x the stream [T, width], W stored [out, in] and applied as x @ W.T; position p counts from 0.
    unit(x)       = x / sqrt(mean(x^2) + eps)                     (over the last axis)
    norm(x, w)    = unit(x) * w
    layer         x += mixer(norm(x, w1));  x += ff(norm(x, w2)) (if the layer has a feed-forward)
    output        logits = Whead norm(x, wf)
Mixers: "attention" (grouped-query, partly rotated in halves with stretched frequencies, a factor a head on the
scores, a window that also keeps a sequence's first tokens, probabilities mixed across heads after the softmax) and
"latent_attention" (a low-rank latent and one rotated key part a token, rotated in neighbouring pairs, a plain
window; a layer may read the latent and key part that an earlier layer made).  Feed-forwards: a dense one with
biases and a two-piece activation, or a mixture of gated experts whose sigmoid score scales the expert's input,
with one expert that every token uses.
"""
import math

import torch

D = torch.float64


def unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    return unit(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.clamp(z, min=0.0) + torch.log1p(torch.exp(-z.abs()))


# ---------------------------------------------------------------------------------------------- rotation
def frequencies(rot):
    """(f [dims / 2], amplitude) of a rotation {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}?}."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=D)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_at(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_at(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_at(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, layout):
    """x [T, heads, n]: the first rot.dims numbers of every head turn by position * f; "half" pairs i with
    i + dims/2, "pairs" pairs 2i with 2i + 1.  The rest passes."""
    dims = int(rot["dims"])
    f, amp = frequencies(rot)
    a = positions.to(D)[:, None, None] * f[None, None, :]
    c, s = torch.cos(a) * amp, torch.sin(a) * amp
    out = x.clone()
    if layout == "half":
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    return out


# ---------------------------------------------------------------------------------------------- masks
def visible(T, size, keep_first=0):
    """[T, T] bool: query i sees key j iff j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def masked_softmax(scores, vis):
    s = torch.where(vis, scores, torch.full_like(scores, -1e300))
    e = torch.where(vis, torch.exp(s - s.max(-1, keepdim=True).values), torch.zeros_like(s))
    return e / e.sum(-1, keepdim=True)


# ---------------------------------------------------------------------------------------------- attention
def mix_heads(p, talk):
    """p [H, T, T] probabilities, talk [H, H]: p'_h = sum_g talk[h, g] p_g."""
    return torch.einsum("hg,gij->hij", talk, p)


def attention(h, w, m):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate((h @ w["q"].T).view(T, H, dk), pos, m["rot"], "half")
    k = rotate((h @ w["k"].T).view(T, G, dk), pos, m["rot"], "half")
    v = (h @ w["v"].T).view(T, G, dv)
    kv_of = torch.arange(H) // (H // G)
    scores = torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * float(m["scale"]) * w["temp"][:, None, None]
    vis = visible(T, int(m["mask"]["size"]), int(m["mask"].get("keep_first", 0)))
    p = mix_heads(masked_softmax(scores, vis[None]), w["talk"])
    out = torch.einsum("hij,jhd->ihd", p, v[:, kv_of]).reshape(T, H * dv)
    return out @ w["o"].T


# ---------------------------------------------------------------------------------------------- latent attention
def latent_and_key(h, w, m, eps):
    """(c [T, kv_rank] normed, kr [T, rot_dim] rotated): what a latent layer caches."""
    T = h.shape[0]
    r = int(m["kv_rank"])
    z = h @ w["dkv"].T
    c = norm(z[:, :r], w["dkv.norm"], eps)
    kr = rotate(z[:, None, r:], torch.arange(T), m["rot"], "pairs")[:, 0]
    return c, kr


def latent_attention(h, w, m, eps, shared=None):
    """`shared`: (c, kr) of the layer named by kv_from; None: the layer makes its own.  Returns (out, (c, kr))."""
    T = h.shape[0]
    H, dk, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = shared if shared is not None else latent_and_key(h, w, m, eps)
    q = (h @ w["q"].T).view(T, H, dk + dr)
    qu, qr = q[..., :dk], rotate(q[..., dk:], torch.arange(T), m["rot"], "pairs")
    ku = (c @ w["uk"].T).view(T, H, dk)
    v = (c @ w["uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", qu, ku) + torch.einsum("ihd,jd->hij", qr, kr)) * float(m["scale"])
    p = masked_softmax(scores, visible(T, int(m["mask"]["size"]))[None])
    out = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    return out @ w["o"].T, (c, kr)


# ---------------------------------------------------------------------------------------------- feed-forwards
def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)


def dense(h, w):
    z = h @ w["up"].T + w["up.b"]
    return xielu(z, w["act"][0], w["act"][1]) @ w["down"].T + w["down.b"]


def gated_expert(h, gate, up, down):
    g = h @ gate.T
    return (g * sigmoid(g) * (h @ up.T)) @ down.T


def route(h, router, top):
    """(chosen [T, top] by falling score, weights [T, top]): sigmoid scores, the largest chosen, not renormalised."""
    s = sigmoid(h @ router.T)
    wgt, idx = torch.topk(s, top, dim=-1)
    return idx, wgt


def moe(h, w, f):
    n, top = int(f["router"]["experts"]), int(f["router"]["top"])
    idx, wgt = route(h, w["router"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), wgt[t]):
            out[t] += gated_expert(s * h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if f.get("shared"):
        out = out + gated_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


# ---------------------------------------------------------------------------------------------- the model
def sub(weights, prefix):
    return {k[len(prefix):]: v.to(D) for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, layers_out=None):
    """Logits [T, vocab] (float64) of one sequence.  `layers_out`: a list that receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = weights["embed"].to(D)[torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        m = L["mixer"]
        h = norm(x, weights[f"l{i}.norm1"].to(D), eps)
        w = sub(weights, f"l{i}.mix.")
        if L["type"] == "attention":
            y = attention(h, w, m)
        elif L["type"] == "latent_attention":
            src = m.get("kv_from")
            y, kept[i] = latent_attention(h, w, m, eps, kept[src] if src is not None else None)
        else:
            raise ValueError(f"unknown layer type {L['type']!r}")
        x = x + y
        f = L.get("mlp")
        if f is not None:
            h = norm(x, weights[f"l{i}.norm2"].to(D), eps)
            w = sub(weights, f"l{i}.mlp.")
            x = x + (dense(h, w) if f["kind"] == "dense" else moe(h, w, f))
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, weights["final.norm"].to(D), eps) @ weights["head"].to(D).T

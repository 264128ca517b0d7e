"""A plain, slow Birepel: float64, whole sequences, one function per mechanism, written from the design's
equations and sharing no code with the package.  It reads config.json's dictionary itself.

Notation: T tokens, x the stream [T, width], W stored [out, in] and applied as x @ W.T; position p counts from 0.
    unit(x)       = x / sqrt(mean(x^2) + eps)                     (over the last axis)
    norm(x, w)    = unit(x) * (1 + w)                             (zero-centred weights)
    stream        x = E[token] + P[p]
    layer         x += norm(mixer(x), w1);  x += norm(ff(x), w2) (if the layer has a feed-forward)
    output        logits = E norm(x, wf), E the embedding table
A layer that names `weights_of: j` reads layer j's tensors.
"""
import math

import torch

D = torch.float64


def unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    return unit(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def logsigmoid(z):
    return torch.clamp(z, max=0.0) - torch.log1p(torch.exp(-z.abs()))


# ---------------------------------------------------------------------------------------------- attention
def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1), one factor a position."""
    steps = torch.div(positions.to(torch.int64) + 1, int(every), rounding_mode="floor").to(D)
    return 1.0 + coef * torch.log(steps + 1.0)


def sink_softmax(scores, visible, sink):
    """p_j = exp(s_j) / (exp(sink) + sum over visible i of exp(s_i)); scores [..., T], sink broadcastable to [..., 1]."""
    neg = torch.full_like(scores, -1e300)
    m = torch.maximum(torch.where(visible, scores, neg).max(-1, keepdim=True).values, sink)
    e = torch.where(visible, torch.exp(scores - m), torch.zeros_like(scores))
    return e / (torch.exp(sink - m) + e.sum(-1, keepdim=True))


def attention(h, w, m, eps):
    """Causal grouped-query attention without rotation: heads of q and k brought to unit root mean square, the query
    times a factor that grows with the logarithm of its position, a learned sink a head in the softmax's
    denominator, and a gate a head on the result."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, dk)
    k = (h @ w["k"].T).view(T, G, dk)
    v = (h @ w["v"].T).view(T, G, dv)
    q, k = unit(q, eps), unit(k, eps)
    pos = torch.arange(T)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(pos, qt["coef"], qt["every"])[:, None, None]
    gate = sigmoid(h @ w["g"].T)                                    # [T, H]
    visible = (pos[None, :] <= pos[:, None])                         # [query, key]
    out = torch.zeros(T, H, dv, dtype=D)
    for a in range(H):
        kv = a // (H // G)
        s = (q[:, a] @ k[:, kv].T) * m["scale"]
        p = sink_softmax(s, visible, w["sink"][a].reshape(1, 1))
        out[:, a] = (p @ v[:, kv]) * gate[:, a:a + 1]
    return out.reshape(T, H * dv) @ w["o"].T


# ---------------------------------------------------------------------------------------------- mLSTM
def capped(z, cap):
    return cap * torch.tanh(z / cap)


def memory_walk(q, k, v, li, lf, S=None, n=None, mx=None):
    """One head's matrix memory along T tokens: q, k [T, dk] (q already scaled), v [T, dv], li and lf [T] the logarithms
    of the input and forget gates.  Returns (o [T, dv], S [dk, dv], n [dk], m): the read-outs and the state after the
    last token, held in units of exp(m).  The state starts at zero and m at 0 unless given."""
    T, dk, dv = q.shape[0], q.shape[1], v.shape[1]
    S = torch.zeros(dk, dv, dtype=D) if S is None else S.clone()
    n = torch.zeros(dk, dtype=D) if n is None else n.clone()
    mx = torch.zeros((), dtype=D) if mx is None else mx.clone()
    out = torch.zeros(T, dv, dtype=D)
    for t in range(T):
        m_new = torch.maximum(lf[t] + mx, li[t])
        keep, take = torch.exp(lf[t] + mx - m_new), torch.exp(li[t] - m_new)
        S = keep * S + take * torch.outer(k[t], v[t])
        n = keep * n + take * k[t]
        mx = m_new
        den = torch.maximum((n @ q[t]).abs(), torch.exp(-mx)) + 1e-6
        out[t] = (S.T @ q[t]) / den
    return out, S, n, mx


FIRST_ANGLES = None        # a list, while a test asks how well posed a sequence's first read-outs are


def mlstm(h, w, m, eps):
    """Matrix memory with exponential gates kept in range by a running maximum (which starts at 0).  After one token
    the memory holds one outer product, and what a head reads out, once scaled to unit size, is its value times the
    SIGN of q . k: where that product is near zero, rounding decides.  `FIRST_ANGLES` collects |cos(q, k)| of the
    first token, the smallest of the heads, for tests that choose a first token on which no rounding decides."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w["q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w["k"].T).view(T, H, dk)
    v = (h @ w["v"].T).view(T, H, dv)
    li = capped(h @ w["i"].T + w["i.b"], cap)                       # [T, H] log input gate
    lf = logsigmoid(capped(h @ w["f"].T + w["f.b"], cap))           # [T, H] log forget gate
    if FIRST_ANGLES is not None:
        FIRST_ANGLES.append(((q[0] * k[0]).sum(-1).abs() / (q[0].norm(dim=-1) * k[0].norm(dim=-1)).clamp_min(1e-30)).min().item())
    out = torch.stack([memory_walk(q[:, a], k[:, a], v[:, a], li[:, a], lf[:, a])[0] for a in range(H)], 1)
    y = unit(out, eps).reshape(T, H * dv) * w["norm"] * sigmoid(h @ w["g"].T)
    return y @ w["o"].T


# ---------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h, w, f):
    lim = f["limit"]
    g = torch.clamp(h @ w["gate"].T, max=lim)
    u = torch.clamp(h @ w["up"].T, min=-lim, max=lim)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def route(z, top):
    """The `top` largest logits of every row and the softmax over those alone: (indices [T, top], weights [T, top])."""
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe_ff(h, w, f):
    E, top = f["router"]["experts"], f["router"]["top"]
    idx, wgt = route(h @ w["router"].T, top)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=D)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            a = torch.relu(h[t] @ w[f"e{e}.up"].T) ** 2
            out[t] += wgt[t, j] * (a @ w[f"e{e}.down"].T)
    return out


# ---------------------------------------------------------------------------------------------- the model
def _sub(tensors, prefix):
    return {n[len(prefix):]: t.to(D) for n, t in tensors.items() if n.startswith(prefix)}


def owner(cfg, i):
    """The layer whose tensors layer i reads."""
    seen = set()
    while cfg["layers"][i].get("weights_of") is not None and i not in seen:
        seen.add(i)
        i = cfg["layers"][i]["weights_of"]
    return i


def forward(cfg, tensors, tokens, taps=None):
    """Logits [T, vocab] (float64) of one sequence; `taps`, a list, receives the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(tokens, dtype=torch.int64)
    T = tok.shape[0]
    E = tensors["embed"].to(D)
    x = E[tok] + tensors["pos"].to(D)[:T]
    for i, L in enumerate(cfg["layers"]):
        j = owner(cfg, i)
        w = _sub(tensors, f"l{j}.mix.")
        mix = attention if L["type"] == "attention" else mlstm
        x = x + norm(mix(x, w, L["mixer"], eps), tensors[f"l{j}.norm1"].to(D), eps)
        f = L.get("mlp")
        if f is not None:
            wf = _sub(tensors, f"l{j}.mlp.")
            y = dense_ff(x, wf, f) if f["kind"] == "dense" else moe_ff(x, wf, f)
            x = x + norm(y, tensors[f"l{j}.norm2"].to(D), eps)
        if taps is not None:
            taps.append(x.clone())
    return norm(x, tensors["final.norm"].to(D), eps) @ E.T

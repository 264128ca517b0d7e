"""Birepel on the GPU: every new kernel alone against plain float64 formulas, then the whole model through the
engine (prompts whole, in portions, token by token, in unequal batches, with slots and pages used again, long
decoding, greedy generation, trace replay, the command line) against tests/plain_birepel.py."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_birepel as P
from birepel_tiny import BR_CONFIGS, folder_config, make_birepel_folder, random_config
from test_gpu_loduzen import DTYPES, ROOT, TOL, TORCH, Tally, back, dev, engine, rel, step_tables
from tiny import random_prompts, read_weights

pytestmark = pytest.mark.gpu
D = torch.float64


@pytest.fixture(scope="module")
def K():
    from braidinfer_b200.csrc.api import get_kernels
    return get_kernels(verbose=False)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("birepel")
    d = {n: make_birepel_folder(base, n) for n in BR_CONFIGS}
    d.update({n + "~": make_birepel_folder(base, n, steady=True) for n in BR_CONFIGS})
    return d


def fold(name, dtype):
    """The folder a run of this precision reads.  A float32 run reads routers drawn at random: its error is far below
    the gaps between their logits.  A bfloat16 run reads the folder whose routers rest on no close call (named with a
    tilde): one expert chosen otherwise at one position moves that position by the size of the stream, and a
    memory carries it to every later one, so no tolerance on rounding could tell it from a fault."""
    return name if dtype == "float32" else name + "~"


class Oracle:
    def __init__(self, folder):
        self.cfg, self.w, self.memo = folder_config(folder), read_weights(folder), {}

    def logits(self, tokens, w=None):
        if w is not None:
            return P.forward(self.cfg, w, list(tokens))
        key = tuple(tokens)
        if key not in self.memo:
            self.memo[key] = P.forward(self.cfg, self.w, list(tokens))
        return self.memo[key]


@pytest.fixture(scope="module")
def oracles(folders):
    return {n: Oracle(f) for n, f in folders.items()}


def paged(total, nkh, page, hd, dtype, g, n_pages=None):
    """A page table over shuffled pages for sequences of `total` tokens, and the empty cache."""
    blocks = [-(-x // page) for x in total]
    n_pages = n_pages or sum(blocks) + 2
    perm = torch.randperm(n_pages, generator=g)
    table = torch.full((len(total), max(blocks) + 1), -1, dtype=torch.int32)
    at = 0
    for s, b in enumerate(blocks):
        table[s, :b] = perm[at:at + b].to(torch.int32)
        at += b
    cache = torch.zeros(n_pages, 2, nkh, page, hd, dtype=TORCH[dtype], device="cuda")
    return table, cache


# ================================================================== kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nqh, nkh, dk, dv, unit, temp", [(4, 2, 32, 48, True, (0.5, 16)), (3, 3, 40, 40, True, None),
                                                          (2, 1, 64, 64, True, (0.1, 1)), (2, 2, 8, 24, False, (1.0, 100)),
                                                          (6, 2, 24, 8, True, (2.0, 3)), (1, 1, 16, 16, False, None),
                                                          (2, 1, 256, 136, True, (0.3, 5)), (3, 1, 20, 12, True, (0.3, 5))])
def test_unit_heads_query_temperature_padding_and_cache_write(K, dtype, nqh, nkh, dk, dv, unit, temp):
    g = torch.Generator().manual_seed(dk + dv)
    page, eps = 64, 1e-5
    hd = -(-max(dk, dv) // 16) * 16
    lengths, before = [3, 70, 1], [0, 60, 129]                   # positions 0.., across a page border, and far on
    t = step_tables(lengths, before, pad=2)
    width = nqh * dk + nkh * (dk + dv)
    src = dev(torch.randn(t.rows, -(-width // 8) * 8 + 8, generator=g) * 3, dtype)
    total = [b + n for b, n in zip(before, lengths)]
    table, cache = paged(total, nkh, page, hd, dtype, g)
    cache.fill_(7.0)
    q = torch.full((t.rows, nqh * hd), 7.0, dtype=TORCH[dtype], device="cuda")
    coef, every = temp if temp else (0.0, 0)
    K.head_prep_kv(src, q, t.positions, t.token_seq, table.cuda(), cache, nqh, nkh, dk, dv, hd, unit, eps, coef, every)
    K.check_device_errors()
    x = back(src)
    qs, ks = x[:, :nqh * dk].view(-1, nqh, dk), x[:, nqh * dk:(nqh + nkh) * dk].view(-1, nkh, dk)
    vs = x[:, (nqh + nkh) * dk:width].view(-1, nkh, dv)
    if unit:
        qs, ks = P.unit(qs, eps), P.unit(ks, eps)
    if temp:
        qs = qs * P.query_temperature(t.positions.cpu(), coef, every)[:, None, None]
    tol = 3e-6 if dtype == "float32" else 1e-2
    got_q = back(q).view(-1, nqh, hd)
    live = t.n_tokens
    assert rel(got_q[:live, :, :dk], qs[:live]) < tol and got_q[:live, :, dk:].abs().sum().item() == 0
    pos, seq = t.positions.cpu(), t.token_seq.cpu()
    for r in range(live):
        pg, off = int(table[seq[r], pos[r] // page]), int(pos[r] % page)
        row = back(cache[pg, :, :, off])                                        # [2, nkh, hd]
        assert rel(row[0, :, :dk], ks[r]) < tol and rel(row[1, :, :dv], vs[r]) < tol, r
        assert row[0, :, dk:].abs().sum().item() == 0 and row[1, :, dv:].abs().sum().item() == 0
    written = sum(lengths)
    assert (back(cache) != 7.0).any(-1).sum().item() == 2 * nkh * written      # no other place of the cache was touched


def plain_heads_attention(q, keys, vals, pos, scale, sinks, gates, nkh):
    """q [n, H, hd] at positions pos over keys, vals [total, G, hd]: causal, a sink a head, a gate a head and row."""
    n, H, hd = q.shape
    out = torch.zeros(n, H, vals.shape[-1], dtype=D)
    visible = torch.arange(keys.shape[0])[None, :] <= pos[:, None]
    for a in range(H):
        kv = a // (H // nkh)
        s = (q[:, a] @ keys[:, kv].T) * scale
        p = P.sink_softmax(s, visible, sinks[a].reshape(1, 1).to(D))
        out[:, a] = (p @ vals[:, kv]) * P.sigmoid(gates[:, a:a + 1])
    return out


@pytest.mark.parametrize("kernel", ["simple_f32", "simple_bf16", "mma_prompt", "mma_few_1", "mma_few_9", "tcgen05_prompt",
                                    "tcgen05_prompt_128"])
def test_attention_with_a_sink_a_head_and_a_gate_a_head(K, kernel):
    g = torch.Generator().manual_seed(len(kernel))
    dtype = "float32" if kernel == "simple_f32" else "bfloat16"
    nqh, nkh, hd, page, scale = 4, 2, {"tcgen05_prompt": 64, "tcgen05_prompt_128": 128}.get(kernel, 48), 64, 0.3
    few = kernel.startswith("mma_few")
    lengths, before = ([1, 2], [700, 130]) if few else ([150, 37], [0, 200])
    t = step_tables(lengths, before, pad=1)
    total = [b + n for b, n in zip(before, lengths)]
    table, cache = paged(total, nkh, page, hd, dtype, g)
    q0 = torch.randn(t.rows, nqh, hd, generator=g)
    q0[:, :, 0] = 4.0
    q = dev(q0.view(t.rows, nqh * hd), dtype)
    gates = dev(torch.randn(t.rows, nqh + 3, generator=g) * 2, dtype)              # a view with further columns
    sinks = torch.tensor([2.0, -30.0, 0.0, 5.0])                                   # of both signs; one that counts for nothing
    kv = []
    for s in range(2):
        keys = torch.randn(total[s], nkh, hd, generator=g) * 0.3
        vals = torch.randn(total[s], nkh, hd, generator=g)
        # every score sits below the sinks but two: the first key of the sequence (hundreds of tokens back) and the
        # key at the query's own place; losing either, or the sink, shows at once
        keys[:, :, 0] = -3.0
        keys[0, :, 0] = 1.5
        keys[total[s] - 1, :, 0] = 1.0
        keys, vals = keys.to(TORCH[dtype]), vals.to(TORCH[dtype])
        kv.append((keys.double(), vals.double()))
        for b in range(-(-total[s] // page)):
            pg, n = int(table[s, b]), min(page, total[s] - b * page)
            cache[pg, 0, :, :n] = keys[b * page:b * page + n].transpose(0, 1).cuda()
            cache[pg, 1, :, :n] = vals[b * page:b * page + n].transpose(0, 1).cuda()
    tb = table.cuda()
    for hs, gate in ((sinks, gates), (sinks, None), (None, gates)):
        out = torch.zeros(t.rows, nqh * hd, dtype=TORCH[dtype], device="cuda")
        kw = dict(head_sinks=hs.cuda() if hs is not None else None, head_gate=gate[:, :nqh] if gate is not None else None)
        if kernel.startswith("simple"):
            K.attn_simple(q, out, cache, tb, t.positions, t.token_seq, nqh, nkh, hd, page, None, scale, **kw)
        elif kernel.startswith("tcgen05_prompt"):
            K.attn_tc(q, out, cache, tb, t.q_start, t.q_len, t.kv_before, 2, max(lengths), nqh, nkh, hd, None, scale, **kw)
        else:
            splits = {"mma_prompt": 1, "mma_few_1": 1, "mma_few_9": 9}[kernel]
            K.attn_mma(q, out, cache, tb, t.q_start, t.q_len, t.kv_before, t.token_seq, 2, max(lengths), nqh, nkh, hd, None,
                       scale, n_splits=splits, few_tokens=few, **kw)
        K.check_device_errors()
        r0 = 0
        for s in range(2):
            n = lengths[s]
            qs = back(q[r0:r0 + n]).view(-1, nqh, hd)
            pos = torch.arange(before[s], total[s])
            gs = back(gate[r0:r0 + n, :nqh]) if gate is not None else torch.full((n, nqh), 1e9, dtype=D)
            want = plain_heads_attention(qs, kv[s][0], kv[s][1], pos, scale, hs if hs is not None else torch.full((nqh,), -1e9),
                                         gs, nkh)
            got = back(out[r0:r0 + n]).view(-1, nqh, hd)
            assert (got - want).abs().max().item() < (3e-6 if dtype == "float32" else 2.5e-2), (kernel, hs is None, gate is None, s)
            r0 += n
    # the test can tell: without the first key, without the sinks or without the gates the result is another
    last = plain_heads_attention(qs, kv[1][0], kv[1][1], pos, scale, sinks, gs, nkh)
    k2 = kv[1][0].clone()
    k2[0, :, 0] = -3.0
    assert (plain_heads_attention(qs, k2, kv[1][1], pos, scale, sinks, gs, nkh) - last).abs().max().item() > 0.05
    assert (plain_heads_attention(qs, kv[1][0], kv[1][1], pos, scale, torch.full((nqh,), -1e9), gs, nkh) - last).abs().max().item() > 0.05


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dk, dv, cap", [(3, 24, 40, 8.0), (2, 136, 8, 6.0), (1, 8, 24, 3.0), (4, 48, 70, 12.0), (2, 16, 16, 20.0)])
def test_matrix_memory_whole_in_portions_and_token_by_token(K, dtype, heads, dk, dv, cap):
    """Gates, recurrence and read-out as the mixer chains them, with the state of two sequences kept in slots between
    steps; a slot that held another sequence before starts from zero again only because a new sequence says so."""
    g = torch.Generator().manual_seed(heads * dk + dv)
    eps, lens = 1e-5, [41, 7]
    bias_i, bias_f = dev(torch.randn(heads, generator=g), dtype), dev(torch.randn(heads, generator=g) + 3, dtype)
    w = dev(1 + 0.3 * torch.randn(heads * dv, generator=g), dtype)
    seqs, want = [], []
    for n in lens:
        q, k = [dev(torch.randn(n, heads * dk, generator=g), dtype) for _ in range(2)]
        v, gate = [dev(torch.randn(n, heads * dv, generator=g), dtype) for _ in range(2)]
        z = (torch.randn(n, 2 * heads, generator=g) * 4).cuda()                 # gates' logits: float32 in every run
        z[: n // 2, heads:] += 6.0                                             # forget gates near one early, then mixed
        seqs.append((q, k, v, gate, z))
        li = P.capped(back(z)[:, :heads] + back(bias_i), cap)
        lf = P.logsigmoid(P.capped(back(z)[:, heads:] + back(bias_f), cap))
        o, st = [], []
        for a in range(heads):
            oa, S, nn, mx = P.memory_walk(back(q)[:, a * dk:(a + 1) * dk] * dk ** -0.5, back(k)[:, a * dk:(a + 1) * dk],
                                          back(v)[:, a * dv:(a + 1) * dv], li[:, a], lf[:, a])
            o.append(oa)
            st.append((S, nn, mx))
        y = P.unit(torch.stack(o, 1), eps).reshape(n, heads * dv) * back(w) * P.sigmoid(back(gate))
        want.append((y, st))
    m_off = heads * dk * (dv + 1) * 4
    sbytes = m_off + heads * 4
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    for cuts in ([[41, 7]], [[1, 1], [2, 2], [38, 4]], [[20, 0], [1, 7], [20, 0]], [[3, 2], [38, 5]], [[1, 1]] * 7 + [[34, 0]]):
        state = torch.full((4, sbytes), 255, dtype=torch.uint8, device="cuda")          # what an earlier sequence left
        at = [0, 0]
        for cut in cuts:
            live = [i for i in range(2) if cut[i]]
            t = step_tables([cut[i] for i in live], before=[at[i] for i in live], slots=[[3, 1][i] for i in live], pad=2)
            for i in live:
                if at[i] == 0:
                    state[[3, 1][i]].zero_()                                  # the manager hands a new sequence a cleared slot
            cat = lambda j: torch.cat([seqs[i][j][at[i]:at[i] + cut[i]] for i in live] + [seqs[0][j][:2] * 0])      # noqa: E731
            q, k, v, gate, z = (cat(j) for j in range(5))
            gates = torch.empty(t.rows, 3 * heads, dtype=torch.float32, device="cuda")
            K.mlstm_gates(z, bias_i, bias_f, gates, state, m_off, t, heads, cap)
            o = torch.empty(t.rows, heads * (dv + 1), dtype=torch.float32, device="cuda")
            K.linear_scan(q, k, v, gates[:, :heads], bias_i, o, state, 0, t, heads, heads, dk, dv + 1, "given",
                          q_scale=dk ** -0.5, kappa=gates[:, heads:2 * heads], v_cols=dv)
            out = torch.zeros(t.rows, heads * dv, dtype=TORCH[dtype], device="cuda")
            K.mlstm_out(o, gates[:, 2 * heads:], gate, w, out, t.token_seq, heads, dv, eps)
            r = 0
            for i in live:
                assert rel(out[r:r + cut[i]], want[i][0][at[i]:at[i] + cut[i]]) < tol, (cuts, cut, i)
                r += cut[i]
                at[i] += cut[i]
        for slot, i in ((3, 0), (1, 1)):
            S = state[slot, :m_off].contiguous().view(torch.float32).view(heads, dk, dv + 1)
            m = state[slot, m_off:].contiguous().view(torch.float32)
            for a in range(heads):
                assert rel(S[a, :, :dv], want[i][1][a][0]) < 1e-4 and rel(S[a, :, dv], want[i][1][a][1]) < 1e-4
                assert abs(m[a].item() - want[i][1][a][2].item()) < 1e-4
        assert (state[[0, 2]] == 255).all()                                   # the other slots were not touched


@pytest.mark.parametrize("dtype", DTYPES)
def test_matrix_memory_of_a_long_prompt_keeps_a_token_from_its_start(K, dtype):
    """300 tokens, walked whole (chunks side by side with a carry between them) and in portions that end on, just before
    and just after the chunks' edges.  One token near the start has an open input gate and all others nearly closed
    ones, with forget gates near one: every later read-out is that token's value, and a walk that lost it, or the
    state at a chunk's or a portion's edge, returns something else."""
    heads, dk, dv, cap, n, eps = 2, 32, 24, 10.0, 300, 1e-5
    g = torch.Generator().manual_seed(11)
    # queries of one sign and that token's key all ones: no read-out is a sum that cancels, so rounding stays rounding
    q, k = dev(torch.randn(n, heads * dk, generator=g).abs() + 0.1, dtype), dev(torch.randn(n, heads * dk, generator=g), dtype)
    v, gate = [dev(torch.randn(n, heads * dv, generator=g), dtype) for _ in range(2)]
    k[2] = dev(torch.ones(heads * dk), dtype)
    z = torch.cat([torch.full((n, heads), -6.0), torch.full((n, heads), 9.0)], 1)
    z[2, :heads] = 8.0
    z = z.cuda()
    zero, w = dev(torch.zeros(heads), dtype), dev(1 + 0.3 * torch.randn(heads * dv, generator=g), dtype)
    li, lf = P.capped(back(z)[:, :heads], cap), P.logsigmoid(P.capped(back(z)[:, heads:], cap))

    def plain(vals):
        o = [P.memory_walk(back(q)[:, a * dk:(a + 1) * dk] * dk ** -0.5, back(k)[:, a * dk:(a + 1) * dk],
                           vals[:, a * dv:(a + 1) * dv], li[:, a], lf[:, a])[0] for a in range(heads)]
        return P.unit(torch.stack(o, 1), eps).reshape(n, heads * dv) * back(w) * P.sigmoid(back(gate))

    want = plain(back(v))
    other = back(v).clone()
    other[2] = -other[2]
    assert rel(plain(other)[n - 1:], want[n - 1:]) > 0.5 and rel(plain(other)[150:151], want[150:151]) > 0.5     # token 2's value is read
    m_off = heads * dk * (dv + 1) * 4
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    for cuts in ([300], [128, 1, 63, 108], [127, 2, 171], [65, 63, 64, 108], [2, 298]):
        state = torch.zeros(1, m_off + heads * 4, dtype=torch.uint8, device="cuda")
        at = 0
        for cut in cuts:
            t = step_tables([cut], before=[at])
            sl = slice(at, at + cut)
            gates = torch.empty(t.rows, 3 * heads, dtype=torch.float32, device="cuda")
            K.mlstm_gates(z[sl], zero, zero, gates, state, m_off, t, heads, cap)
            o = torch.empty(t.rows, heads * (dv + 1), dtype=torch.float32, device="cuda")
            K.linear_scan(q[sl], k[sl], v[sl], gates[:, :heads], zero, o, state, 0, t, heads, heads, dk, dv + 1, "given",
                          q_scale=dk ** -0.5, kappa=gates[:, heads:2 * heads], v_cols=dv)
            out = torch.zeros(t.rows, heads * dv, dtype=TORCH[dtype], device="cuda")
            K.mlstm_out(o, gates[:, 2 * heads:], gate[sl], w, out, t.token_seq, heads, dv, eps)
            assert rel(out[:cut], want[sl]) < tol, (cuts, cut)
            at += cut
    K.check_device_errors()


def test_the_running_maximum_starts_at_zero_and_the_read_out_has_a_floor(K):
    """Input gates far below one at the first tokens: the maximum stays at 0 from its start (not at the first gate),
    and the read-out's denominator is its floor exp(-m); with a maximum that started at minus infinity the
    results would be hundreds of times larger."""
    heads, dk, dv, cap, n = 2, 8, 8, 30.0, 5
    g = torch.Generator().manual_seed(2)
    q, k = torch.randn(n, heads * dk, generator=g).cuda(), torch.randn(n, heads * dk, generator=g).cuda()
    v = torch.randn(n, heads * dv, generator=g).cuda()
    z = torch.cat([torch.full((n, heads), -9.0), torch.full((n, heads), 8.0)], 1).cuda()
    zero, one = torch.zeros(heads).cuda(), torch.ones(heads * dv).cuda()
    m_off = heads * dk * (dv + 1) * 4
    state = torch.zeros(1, m_off + heads * 4, dtype=torch.uint8, device="cuda")
    t = step_tables([n])
    gates = torch.empty(n, 3 * heads, dtype=torch.float32, device="cuda")
    K.mlstm_gates(z, zero, zero, gates, state, m_off, t, heads, cap)
    li, lf = P.capped(torch.full((n,), -9.0, dtype=D), cap), P.logsigmoid(P.capped(torch.full((n,), 8.0, dtype=D), cap))
    m = state[0, m_off:].contiguous().view(torch.float32)
    assert abs(m[0].item() - float(lf.sum())) < 1e-5 and m[0].item() > -0.01        # max(lf + m, li) never took li
    o = torch.empty(n, heads * (dv + 1), dtype=torch.float32, device="cuda")
    K.linear_scan(q, k, v, gates[:, :heads], zero, o, state, 0, t, heads, heads, dk, dv + 1, "given", q_scale=1.0,
                  kappa=gates[:, heads:2 * heads], v_cols=dv)
    raw = torch.empty(n, heads * dv, dtype=torch.float32, device="cuda")
    K.mlstm_out(o, gates[:, 2 * heads:], torch.full((n, heads * dv), 40.0).cuda(), one, raw, t.token_seq, heads, dv, 1e3)
    for a in range(heads):
        oa = P.memory_walk(back(q)[:, a * dk:(a + 1) * dk], back(k)[:, a * dk:(a + 1) * dk], back(v)[:, a * dv:(a + 1) * dv], li, lf)[0]
        assert oa.abs().max().item() < 0.05                                     # small: the floor, not |n . q|, divides
        want = oa / torch.sqrt((oa * oa).mean(-1, keepdim=True) + 1e3)          # an eps that leaves the size to see
        assert rel(raw[:, a * dv:(a + 1) * dv], want) < 1e-4


@pytest.mark.parametrize("dtype", DTYPES)
def test_clamped_unit_zero_centred_norms_and_learned_positions(K, dtype):
    g = torch.Generator().manual_seed(4)
    rows, inter, width, vocab, npos = 9, 72, 100, 50, 40
    gu = dev(torch.randn(rows, 2 * inter, generator=g) * 3, dtype)
    out = torch.zeros(rows, inter, dtype=TORCH[dtype], device="cuda")
    tol = 2e-6 if dtype == "float32" else 8e-3
    for limit, alpha in ((1.5, 1.702), (0.4, 1.0), (100.0, 1.702)):
        K.glu_clamp(gu, out, limit, alpha)
        a, b = back(gu)[:, :inter].clamp(max=limit), back(gu)[:, inter:].clamp(-limit, limit)
        assert rel(out, a * P.sigmoid(alpha * a) * (b + 1.0)) < tol, limit
    x = (torch.randn(rows, width, generator=g) * 5).cuda()
    w = dev(0.2 * torch.randn(width, generator=g), dtype)                        # stored around zero
    y = torch.zeros(rows, width, dtype=TORCH[dtype], device="cuda")
    K.rmsnorm(x, w, y, 1e-5, w_offset=1.0)
    assert rel(y, P.norm(back(x), back(w), 1e-5)) < tol
    h0 = torch.randn(rows, width, generator=g)
    h = h0.cuda().clone()
    K.rmsnorm_add(h, x, w, 1e-5, w_offset=1.0)
    assert rel(h, h0.double() + P.norm(back(x), back(w), 1e-5)) < 2e-6            # the stream and the sum are float32
    table, ptab = dev(torch.randn(vocab, width, generator=g), dtype), dev(torch.randn(npos, width, generator=g), dtype)
    ids = torch.randint(0, vocab, (rows,), generator=g).to(torch.int32)
    pos = torch.tensor([0, 1, 2, 39, 17, 0, 5, 38, 3], dtype=torch.int32)
    e = torch.zeros(rows, width, dtype=torch.float32, device="cuda")
    K.embed(table, ids.cuda(), e, 1.0, pos_table=ptab, positions=pos.cuda())
    assert rel(e, back(table)[ids.long()] + back(ptab)[pos.long()]) < 1e-7
    K.check_device_errors()


# ================================================================== the whole model through the engine
NAMES = ["A", "B", "C", "D"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_and_every_layer(folders, oracles, name, dtype):
    eng = engine(folders[fold(name, dtype)], dtype)
    cfg = oracles[fold(name, dtype)].cfg
    tally = Tally(dtype)
    for n, seed in ((1, 0), (2, 1), (67, 2), (200, 3)):
        toks = random_prompts(cfg["vocab"], [n], seed)[0]
        s = eng.open()
        taps = []
        got = eng.step([(s, toks)], want="all", tap=lambda i, h: taps.append(h.clone()))
        eng.close(s)
        eng.check()
        tally.add(got, oracles[fold(name, dtype)].logits(toks), (name, n))
        if n == 67:
            streams = []
            P.forward(cfg, oracles[fold(name, dtype)].w, toks, streams)
            assert len(taps) == 1 + len(streams) == 1 + len(cfg["layers"])
            for i, (a, b) in enumerate(zip(taps[1:], streams)):
                t2 = Tally(dtype)
                t2.add(a, b, (name, "after layer", i))
                t2.close()
    tally.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first_token_equals_the_prompt_whole(folders, oracles, name, dtype):
    eng = engine(folders[fold(name, dtype)], dtype)
    toks = random_prompts(oracles[fold(name, dtype)].cfg["vocab"], [150], 7)[0]
    want = oracles[fold(name, dtype)].logits(toks)
    s, tally = eng.open(), Tally(dtype)
    for t, tok in enumerate(toks):
        tally.add(eng.step([(s, [tok])], want="last"), want[t:t + 1], t)
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, cuts", [("A", [2, 62, 1, 3, 64, 18]), ("A", [63, 2, 2, 83]), ("B", [128, 22]), ("A", [1, 1, 2, 146]),
                                        ("C", [2, 2, 2, 3, 141]), ("D", [5, 60, 64, 2, 19]), ("D", [64, 64, 22]), ("B", [15, 2, 16, 2, 115])])
def test_a_prompt_in_portions(folders, oracles, dtype, name, cuts):
    eng = engine(folders[fold(name, dtype)], dtype)
    toks = random_prompts(oracles[fold(name, dtype)].cfg["vocab"], [150], 9)[0]
    want = oracles[fold(name, dtype)].logits(toks)
    s, at, tally = eng.open(), 0, Tally(dtype)
    for c in cuts:
        tally.add(eng.step([(s, toks[at:at + c])], want="all"), want[at:at + c], (at, c))
        at += c
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_requests_in_one_batch_then_decoded_together_and_slots_used_again(folders, oracles, name, dtype):
    eng = engine(folders[fold(name, dtype)], dtype, max_tokens=64 * 12, max_slots=4)
    vocab = oracles[fold(name, dtype)].cfg["vocab"]
    prompts = random_prompts(vocab, [3 + 4, 70 + 9, 1 + 2, 129 + 12], 21)
    cut = [3, 70, 1, 129]
    want = [oracles[fold(name, dtype)].logits(p) for p in prompts]
    slots = [eng.open() for _ in prompts]
    lg = eng.step([(s, p[:c]) for s, p, c in zip(slots, prompts, cut)], want="all")
    off, tally = 0, Tally(dtype)
    for i, (p, c, w) in enumerate(zip(prompts, cut, want)):
        tally.add(lg[off:off + c], w[:c], ("prompt", i))
        off += c
    live, t = list(range(4)), 0
    while live:
        lg = eng.step([(slots[i], [prompts[i][cut[i] + t]]) for i in live], want="last")
        for j, i in enumerate(live):
            tally.add(lg[j:j + 1], want[i][cut[i] + t:cut[i] + t + 1], (i, t))
        t += 1
        for i in list(live):
            if cut[i] + t == len(prompts[i]):
                eng.close(slots[i])                                  # the shorter requests end earlier
                live.remove(i)
    assert all(n == 0 for n in eng.cache.pages_in_use())
    # the freed slots (state areas) and pages serve other requests; what they held before must not show
    again = random_prompts(vocab, [66, 5], 22)
    slots = [eng.open(), eng.open()]
    lg = eng.step([(slots[0], again[0]), (slots[1], again[1])], want="all")
    tally.add(lg[:66], oracles[fold(name, dtype)].logits(again[0]), "slot used again")
    tally.add(lg[66:], oracles[fold(name, dtype)].logits(again[1]), "slot used again")
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_long_decoding_across_page_borders_and_temperature_steps(folders, oracles, name, dtype):
    eng = engine(folders[fold(name, dtype)], dtype)
    toks = random_prompts(oracles[fold(name, dtype)].cfg["vocab"], [5 + 215], 31)[0]
    want = oracles[fold(name, dtype)].logits(toks)
    s, tally = eng.open(), Tally(dtype)
    eng.step([(s, toks[:5])], want=None)
    for t in range(5, len(toks)):
        tally.add(eng.step([(s, [toks[t]])], want="last"), want[t:t + 1], t)
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "D"])
def test_a_token_far_back_still_counts(folders, oracles, name, dtype):
    """Two prompts that differ in their first token only: 300 tokens on the logits still differ, through the cache of
    keys (C has attention alone) and through the memories (D has nothing else), and the engine follows the plain
    implementation on both, in a prompt's portion and decoded."""
    cfg = oracles[fold(name, dtype)].cfg
    a = random_prompts(cfg["vocab"], [310], 77)[0]
    b = [(a[0] + 1) % cfg["vocab"]] + a[1:]
    wa, wb = oracles[fold(name, dtype)].logits(a), oracles[fold(name, dtype)].logits(b)
    assert rel(wa[290:], wb[290:]) > 0.01
    eng = engine(folders[fold(name, dtype)], dtype)
    for toks, want in ((a, wa), (b, wb)):
        s, tally = eng.open(), Tally(dtype)
        tally.add(eng.step([(s, toks[:200])], want="all"), want[:200])
        tally.add(eng.step([(s, toks[200:296])], want="all"), want[200:296])
        for t in range(296, 310):
            tally.add(eng.step([(s, [toks[t]])], want="last"), want[t:t + 1], t)
        tally.close()
        eng.close(s)
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sinks_the_gates_and_the_temperature_count_in_the_model(folders, oracles, dtype):
    """The plain implementation with the sinks far below, the gates' tensors zeroed or the temperature's steps moved by
    one gives other logits than the model's by far more than the tolerance, and the engine is on the model's side."""
    o = oracles[fold("C", dtype)]
    toks = random_prompts(o.cfg["vocab"], [140], 5)[0]
    want = o.logits(toks)
    for change in ("sink", "g"):
        w = dict(o.w)
        for n in w:
            if n.endswith(".mix." + change):
                w[n] = torch.full_like(w[n], -1e9) if change == "sink" else torch.zeros_like(w[n])
        assert rel(o.logits(toks, w), want) > 0.05, change
    cfg = json.loads(json.dumps(o.cfg))
    cfg["layers"][1]["mixer"]["q_temp"]["every"] = 101
    for L in cfg["layers"][2:]:
        L["mixer"]["q_temp"]["every"] = 101
    assert rel(P.forward(cfg, o.w, toks)[100:], want[100:]) > 0.01
    eng = engine(folders[fold("C", dtype)], dtype)
    s, tally = eng.open(), Tally(dtype)
    tally.add(eng.step([(s, toks[:97])], want="all"), want[:97])
    for t in range(97, 104):                                                # the temperature steps at position 99
        tally.add(eng.step([(s, [toks[t]])], want="last"), want[t:t + 1], t)
    tally.add(eng.step([(s, toks[104:])], want="all"), want[104:])
    tally.close()
    eng.check()


def well_posed_first_token(oracle, token):
    """The first token from `token` on after which every memory's first read-out has a sign that rounding cannot turn
    (a memory that holds one token returns its value times the sign of q . k)."""
    for t in range(token, token + oracle.cfg["vocab"]):
        P.FIRST_ANGLES = []
        try:
            P.forward(oracle.cfg, oracle.w, [t % oracle.cfg["vocab"]])
            if min(P.FIRST_ANGLES, default=1.0) > 0.05:
                return t % oracle.cfg["vocab"]
        finally:
            P.FIRST_ANGLES = None
    raise AssertionError("no first token is well posed")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10])
def test_configurations_drawn_from_a_seed(tmp_path, seed, dtype):
    """Other sizes, head counts, layer orders and constants than any written by hand: a prompt in two portions beside
    a second request, then both decoded together, against the plain implementation."""
    cfg = random_config(seed)
    # A float32 run takes the sharp gates (an input gate's logit spans the whole cap: a memory holds a few tokens out
    # of hundreds).  A bfloat16 run rounds the gates' input to 8 bits, which moves such a logit by 0.1 and a token's
    # weight in the memory by a tenth, layer upon layer: its gates are drawn milder, so that its error stays rounding.
    folder = make_birepel_folder(tmp_path, f"r{seed}", cfg=cfg, seed=100 + seed, steady=dtype == "bfloat16",
                                 gains={".mix.i": 4.0} if dtype == "bfloat16" else None)
    oracle = Oracle(folder)
    eng = engine(folder, dtype, max_tokens=64 * 8, max_slots=3)
    a, b = random_prompts(cfg["vocab"], [150, 21], seed)
    if dtype == "bfloat16":           # a float32 run resolves the sign of a small q . k; eight bits of mantissa may not
        a[0], b[0] = well_posed_first_token(oracle, a[0]), well_posed_first_token(oracle, b[0])
    wa, wb = oracle.logits(a), oracle.logits(b)
    sa, sb, tally = eng.open(), eng.open(), Tally(dtype)
    tally.add(eng.step([(sa, a[:3])], want="all"), wa[:3], "first tokens")
    lg = eng.step([(sa, a[3:135]), (sb, b[:9])], want="all")
    tally.add(lg[:132], wa[3:135], "portion")
    tally.add(lg[132:], wb[:9], "beside it")
    for t in range(12):
        lg = eng.step([(sa, [a[135 + t]]), (sb, [b[9 + t]])], want="last")
        tally.add(lg[:1], wa[135 + t:136 + t], ("decoded", t))
        tally.add(lg[1:], wb[9 + t:10 + t], ("decoded beside", t))
    tally.close()
    eng.check()


def argmax_lowest(row):
    return int((row == row.max()).nonzero()[0])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_library_entry_point(folders, oracles, name, dtype):
    import braidinfer_b200 as lib
    model = lib.load(folders[fold(name, dtype)], dtype=dtype, max_seq_len=256, max_batch=3, verbose=False)
    prompts = random_prompts(oracles[fold(name, dtype)].cfg["vocab"], [4, 61, 17, 9], 51)          # four requests, three slots
    outs = model.generate(prompts, lib.SamplingParams.greedy(), stop_tokens=(), max_new_tokens=[6, 8, 3, 5])
    for p, o, n in zip(prompts, outs, [6, 8, 3, 5]):
        assert len(o.tokens) == n
        toks = list(p)
        for t in o.tokens:
            row = oracles[fold(name, dtype)].logits(toks)[-1]
            if dtype == "float32":
                assert t == argmax_lowest(row)
            else:
                assert row[t] >= row.max() - 2 * TOL[dtype] * row.abs().max()
            toks.append(t)
    model.engine.check()


def test_a_sequence_longer_than_the_table_of_positions_is_refused(folders, oracles):
    cfg = oracles["B"].cfg
    eng = engine(folders["B"], "bfloat16", max_tokens=64 * 8)
    toks = random_prompts(cfg["vocab"], [cfg["max_positions"] + 1], 1)[0]
    s = eng.open()
    eng.step([(s, toks[:-1])], want="last")
    eng.check()                                                      # the table's last row is still a position
    with pytest.raises(Exception):
        eng.step([(s, toks[-1:])], want="last")
        eng.check()


def test_graphs_on_and_off_give_the_same_logits(folders, oracles):
    toks = random_prompts(oracles["A"].cfg["vocab"], [40], 5)[0]
    res = []
    for graphs in (True, False):
        eng = engine(folders["A"], "bfloat16", use_graphs=graphs)
        s = eng.open()
        out = [eng.step([(s, toks[:20])], want="last")]
        out += [eng.step([(s, [t])], want="last") for t in toks[20:]]
        res.append(torch.cat(out))
        if graphs:
            assert eng.graph_replays > 10
    assert torch.equal(res[0], res[1])


def test_logits_do_not_depend_on_the_batch_or_on_the_cut_beyond_rounding(folders, oracles):
    """float32: the same request alone and whole, beside others, and cut in portions gives logits equal to a few
    units in the last place of the sums."""
    eng = engine(folders["A"], "float32", max_slots=4)
    vocab = oracles["A"].cfg["vocab"]
    a, b, c = random_prompts(vocab, [90, 7, 130], 3)
    s = eng.open()
    alone = eng.step([(s, a)], want="all")
    eng.close(s)
    sa, sb, sc = eng.open(), eng.open(), eng.open()
    lg = eng.step([(sb, b), (sa, a[:50]), (sc, c)], want="all")
    part = [lg[7:57]]
    lg = eng.step([(sb, [1]), (sa, [a[50]]), (sc, [2])], want="last")
    part.append(lg[1:2])
    eng.close(sb)
    part.append(eng.step([(sa, a[51:]), ], want="all"))
    assert rel(torch.cat(part), alone.cpu()) < 2e-5
    eng.check()


def test_trace_replay_program_on_a_model_folder(folders, oracles, tmp_path):
    toks = random_prompts(oracles["A"].cfg["vocab"], [40, 9], 61)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[0][:33], "want": [0, 32]}, {"id": "b", "tokens": toks[1][:8], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [toks[0][33]], "want": [0]}, {"id": "b", "tokens": [toks[1][8]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [toks[0][34]], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": toks[0][35:], "want": [4]}], "end": ["a"]}]
    import numpy as np
    vocab = oracles["A"].cfg["vocab"]
    wa, wb = oracles["A"].logits(toks[0]), oracles["A"].logits(toks[1])
    for dtype in DTYPES:
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["A"], "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps).encode(),
                           capture_output=True, timeout=600)
        assert p.returncode == 0, p.stderr.decode()[-2000:]
        assert [l for l in p.stdout.decode().split("\n") if l.startswith("done")] == [f"done {i}" for i in range(4)]
        got = {i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab)) for i in (0, 1, 3)}
        assert not (out / "2.f32").exists()
        tol = TOL[dtype] * (1 if dtype == "float32" else 3)
        assert rel(got[0], wa[[0, 32]]) < tol and rel(got[1], torch.stack([wa[33], wb[8]])) < tol
        assert rel(got[3], wa[39:40]) < tol


def test_generate_command_line_on_a_model_folder(folders, oracles):
    env = dict(os.environ, MODEL=folders["B"], MAX_TOKENS="6", RAW="1", DTYPE="float32", MAX_SEQ_LEN="128")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "7, 200, 31, 4"], env=env, capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    toks, want = [7, 200, 31, 4], []
    for _ in range(6):
        t = argmax_lowest(oracles["B"].logits(toks)[-1])
        want.append(t)
        toks.append(t)
    assert [int(x) for x in p.stdout.split()] == want

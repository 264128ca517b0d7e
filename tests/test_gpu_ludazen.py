"""Ludazen on the GPU: every new kernel or kernel option alone against plain float64 formulas, then the whole model
through the engine (prompts whole, in portions, token by token, in unequal batches, with slots and pages used again,
long decoding past every window, greedy generation, trace replay, the command line) against tests/plain_ludazen.py."""
import copy
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_ludazen as P
from ludazen_tiny import LD_CONFIGS, _att, folder_config, make_ludazen_folder, random_config
from test_gpu_birepel import paged
from test_gpu_loduzen import DTYPES, ROOT, TOL, TORCH, Tally, back, dev, engine, rel, step_tables
from tiny import random_prompts, read_weights

pytestmark = pytest.mark.gpu
D = torch.float64
NAMES = ["A", "B", "C"]


@pytest.fixture(scope="module")
def K():
    from braidinfer_b200.csrc.api import get_kernels
    return get_kernels(verbose=False)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("ludazen")
    d = {n: make_ludazen_folder(base, n) for n in LD_CONFIGS}
    d.update({n + "~": make_ludazen_folder(base, n, steady=True) for n in LD_CONFIGS})
    return d


def fold(name, dtype):
    """The folder a run of this precision reads.  A float32 run reads routers drawn at random: its error is far below
    the gaps between their scores.  A bfloat16 run reads the folder whose routers rest on no close call (named with a
    tilde): one expert chosen otherwise at one position moves that position by the size of the stream."""
    return name if dtype == "float32" else name + "~"


class Oracle:
    def __init__(self, folder):
        self.cfg, self.w, self.memo = folder_config(folder), read_weights(folder), {}

    def logits(self, tokens, cfg=None, w=None):
        if cfg is not None or w is not None:
            return P.forward(cfg or self.cfg, w or self.w, list(tokens))
        key = tuple(tokens)
        if key not in self.memo:
            self.memo[key] = P.forward(self.cfg, self.w, list(tokens))
        return self.memo[key]


@pytest.fixture(scope="module")
def oracles(folders):
    return {n: Oracle(f) for n, f in folders.items()}


# ================================================================== kernels alone
def plain_talking_attention(q, keys, vals, pos, scale, temp, talk, nkh, size, keep):
    """q [n, H, hd] at positions pos over keys, vals [total, G, .]: windowed with kept first tokens, a factor a head, the
    heads' probabilities mixed by talk.  Returns (mixed result [n, H, vd], every head over every kv head [n, H, G, vd])."""
    n, H, _ = q.shape
    j = torch.arange(keys.shape[0])[None, :]
    vis = (j <= pos[:, None]) & ((pos[:, None] - j < size) | (j < keep))
    kv_of = torch.arange(H) // (H // nkh)
    s = torch.einsum("ihd,jhd->hij", q, keys[:, kv_of]) * scale * temp[:, None, None]
    p = P.masked_softmax(s, vis[None])
    wide = torch.einsum("hij,jcd->ihcd", p, vals)
    out = torch.einsum("hij,jhd->ihd", P.mix_heads(p, talk), vals[:, kv_of])
    return out, wide


@pytest.mark.parametrize("kernel", ["simple_f32", "simple_bf16", "mma_prompt", "mma_few_1", "mma_few_7"])
@pytest.mark.parametrize("nqh, nkh, hd, size, keep", [(4, 2, 48, 40, 3), (6, 3, 16, 64, 0), (3, 3, 48, 7, 9), (8, 4, 64, 70, 5),
                                                      (4, 4, 128, 96, 2), (2, 1, 64, 300, 1), (2, 2, 32, 1, 0), (4, 1, 32, 33, 70),
                                                      (3, 3, 96, 50, 4)])
def test_attention_with_kept_first_tokens_a_factor_a_head_and_values_of_every_kv_head(K, kernel, nqh, nkh, hd, size, keep):
    """For the last query of each sequence, the keys at the window's edge (the oldest one inside, the one just outside)
    and at the kept tokens' edge (the last kept, the first not kept) stand out: their scores are far above the others
    and their values are large, so one key let in or left out by mistake moves that row by a large part of itself."""
    g = torch.Generator().manual_seed(nqh * hd + size)
    dtype = "float32" if kernel == "simple_f32" else "bfloat16"
    few = kernel.startswith("mma_few")
    n_few = int(kernel[-1]) if few else 0
    lengths, before = ([n_few, 1], [320 - n_few, 131]) if few else ([150, 37], [0, 290])
    t = step_tables(lengths, before, pad=1)
    total = [b + n for b, n in zip(before, lengths)]
    page, scale = 64, 0.35
    table, cache = paged(total, nkh, page, hd, dtype, g)
    keys = [torch.randn(n, nkh, hd, generator=g) for n in total]
    vals = [torch.randn(n, nkh, hd, generator=g) for n in total]
    u = torch.zeros(hd)
    u[hd // 2] = 1.0                                                         # every query leans this way; planted keys too
    for s in range(2):
        last = total[s] - 1
        for j in {last - size, last - size + 1, keep - 1, keep}:
            if 0 <= j <= last:
                keys[s][j] = 12.0 * u
                vals[s][j] = 5.0 * torch.sign(torch.randn(nkh, hd, generator=g))
    for s in range(2):
        for j in range(total[s]):
            pg = int(table[s, j // page])
            cache[pg, 0, :, j % page] = dev(keys[s][j], dtype)
            cache[pg, 1, :, j % page] = dev(vals[s][j], dtype)
    q0 = torch.randn(t.rows, nqh * hd + 8, generator=g)
    q0[:, :nqh * hd] += (4.0 * u).repeat(nqh)
    q = dev(q0, dtype)
    temp = torch.rand(nqh, generator=g) * 2 + 0.5
    talk = torch.randn(nqh, nqh, generator=g)
    wide = torch.full((t.rows, nqh * nkh * hd), 7.0, dtype=TORCH[dtype], device="cuda")
    kw = dict(keep_first=keep, head_scale=temp.cuda(), value_heads=nkh)
    if kernel.startswith("simple"):
        K.attn_simple(q, wide, cache, table.cuda(), t.positions, t.token_seq, nqh, nkh, hd, page, size, scale, **kw)
    else:
        n_splits = 1 if not few else (3 if size + keep > 128 else 2)
        K.attn_mma(q, wide, cache, table.cuda(), t.q_start, t.q_len, t.kv_before, t.token_seq, t.n_seqs, t.max_q_len, nqh, nkh, hd,
                   size, scale, n_splits=n_splits, few_tokens=few, **kw)
    out = torch.empty((t.rows, nqh * hd), dtype=TORCH[dtype], device="cuda")
    K.head_mix(wide, dev(talk, dtype), out, t.token_seq, nqh, nkh, hd, hd)
    K.check_device_errors()
    tol = 2e-5 if dtype == "float32" else 3e-2
    qs = back(q)[:, :nqh * hd].view(-1, nqh, hd)
    talk_r = back(dev(talk, dtype))
    r0, shown = 0, 0.0
    for s in range(2):
        rows = slice(r0, r0 + lengths[s])
        pos = torch.arange(before[s], total[s])
        kk, vv = back(dev(keys[s], dtype)), back(dev(vals[s], dtype))
        want, want_wide = plain_talking_attention(qs[rows], kk, vv, pos, scale, temp.double(), talk_r, nkh, size, keep)
        assert rel(back(wide)[rows].view(-1, nqh, nkh, hd), want_wide) < tol, (kernel, s)
        assert rel(back(out)[rows].view(-1, nqh, hd), want) < tol * 3, (kernel, s)
        for wrong in ((size + 1, keep), (size, keep + 1), (max(size - 1, 1), keep)):        # what a fault by one would give
            other, _ = plain_talking_attention(qs[rows], kk, vv, pos, scale, temp.double(), talk_r, nkh, *wrong)
            shown = max(shown, rel(other, want))
        r0 += lengths[s]
    assert shown > 0.15                                                      # the test's inputs do show such a fault
    if not few:
        assert back(out)[t.n_tokens:].abs().sum().item() == 0                # the row of padding


@pytest.mark.parametrize("dtype", DTYPES)
def test_bias_and_two_piece_activation_with_the_ones_column(K, dtype):
    g = torch.Generator().manual_seed(2)
    rows, n, cols = 37, 70, 72
    z = dev(torch.randn(rows, n + 2, generator=g) * 3, dtype)
    b = dev(torch.randn(n, generator=g), dtype)
    for pq in ([0.3, -0.7], [-2.0, 4.0], [0.0, 0.0]):
        pqt = dev(torch.tensor(pq), dtype)
        out = torch.full((rows, cols), 7.0, dtype=TORCH[dtype], device="cuda")
        K.bias_xielu(z, b, pqt, out, n)
        want = P.xielu(back(z)[:, :n] + back(b), back(pqt)[0], back(pqt)[1])
        got = back(out)
        assert rel(got[:, :n], want) < (3e-6 if dtype == "float32" else 6e-3)
        assert (got[:, n] == 1).all() and got[:, n + 1:].abs().sum().item() == 0


@pytest.mark.parametrize("experts, top", [(5, 2), (1, 1), (4, 4), (16, 1), (40, 6)])
def test_sigmoid_routing_keeps_the_scores_as_weights(K, experts, top):
    g = torch.Generator().manual_seed(experts)
    logits = (torch.randn(33, experts, generator=g) * 3).cuda()
    idx = torch.empty((33, top), dtype=torch.int32, device="cuda")
    wgt = torch.empty((33, top), dtype=torch.float32, device="cuda")
    K.moe_route(logits, idx, wgt, 1, 1, sigmoid=True)
    s = P.sigmoid(back(logits))
    ww, wi = torch.topk(s, top, dim=-1)
    assert torch.equal(idx.cpu().long(), wi) and rel(wgt, ww) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, tile", [(9, 16), (150, 64)])
def test_experts_whose_weight_multiplies_their_input(K, dtype, rows, tile):
    g = torch.Generator().manual_seed(rows)
    experts, top, hidden, inter = 5, 2, 64, 24
    x = dev(torch.randn(rows + 1, hidden, generator=g), dtype)
    wg, wu = (dev(torch.randn(experts, inter, hidden, generator=g) * 0.3, dtype) for _ in range(2))
    wd = dev(torch.randn(experts, hidden, inter, generator=g) * 0.3, dtype)
    idx = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows + 1)]).to(torch.int32).cuda()
    wgt = (torch.rand(rows + 1, top, generator=g) * 0.9 + 0.05).cuda()
    token_seq = torch.zeros(rows + 1, dtype=torch.int32)
    token_seq[-1] = -1
    plan = K.moe_plan(idx, token_seq.cuda(), experts, tile)
    slots = plan[4] * tile
    for mma in ([False, True] if dtype == "bfloat16" else [False]):
        act = torch.empty((slots, inter), dtype=TORCH[dtype], device="cuda")
        y = torch.empty((slots, hidden), dtype=TORCH[dtype], device="cuda")
        gemm = K.moe_gemm_mma if mma else K.moe_gemm_simt
        gemm(x, wg, wu, act, plan, top, tile, in_wgt=wgt)
        gemm(act, wd, None, y, plan, top, tile)
        h = torch.zeros((rows + 1, hidden), dtype=torch.float32, device="cuda")
        K.moe_combine(h, y, plan, None, top=top)
        want = torch.zeros(rows + 1, hidden, dtype=D)
        for r in range(rows):
            for k in range(top):
                e = int(idx[r, k])
                want[r] += P.gated_expert(wgt[r, k].double().cpu() * back(x)[r:r + 1], back(wg)[e], back(wu)[e], back(wd)[e])[0]
        assert rel(h, want) < (1e-5 if dtype == "float32" else 3e-2), mma
        assert back(h)[-1].abs().sum().item() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, rot, rank, rot_dims", [(3, 16, 16, 32, 16), (1, 8, 8, 20, 8), (2, 24, 16, 64, 8)])
def test_latent_rows_rotated_in_neighbouring_pairs_and_rows_without_a_latent(K, dtype, heads, dim, rot, rank, rot_dims):
    g = torch.Generator().manual_seed(rank)
    lengths, before = [3, 70, 1], [0, 60, 129]
    t = step_tables(lengths, before, pad=1)
    page, Dl, q_cols = 64, rank + rot, heads * (dim + rot)
    total = [b + n for b, n in zip(before, lengths)]
    table, _ = paged(total, 1, page, Dl, dtype, g)
    rot_cfg = {"base": 50.0, "dims": rot_dims}
    inv = P.frequencies(rot_cfg)[0].float().cuda()
    w = dev(torch.rand(rank, generator=g) + 0.5, dtype)
    for shared in (False, True):
        width = q_cols + (0 if shared else Dl)
        proj = dev(torch.randn(t.rows, -(-width // 8) * 8, generator=g), dtype)
        cache = torch.full((int(table.max()) + 1, 1, 1, page, Dl), 7.0, dtype=TORCH[dtype], device="cuda")
        q_lat = torch.zeros((t.rows, heads, Dl), dtype=TORCH[dtype], device="cuda")
        K.latent_prep(proj, q_cols, None if shared else w, inv, t.positions, t.token_seq, None if shared else table.cuda(),
                      None if shared else cache, q_lat, heads, dim, rot, rank, rot_dims, page, 1e-6, adjacent=True)
        K.check_device_errors()
        x = back(proj)
        pos = t.positions.cpu()
        qr = P.rotate(x[:, :q_cols].view(-1, heads, dim + rot)[..., dim:], pos, rot_cfg, "pairs")
        tol = 3e-6 if dtype == "float32" else 1e-2
        live = t.n_tokens
        assert rel(back(q_lat)[:live, :, rank:], qr[:live]) < tol
        if shared:
            assert (back(cache) == 7.0).all()
            continue
        c = P.norm(x[:, q_cols:q_cols + rank], back(w), 1e-6)
        kr = P.rotate(x[:, None, q_cols + rank:q_cols + Dl], pos, rot_cfg, "pairs")[:, 0]
        seq = t.token_seq.cpu()
        for r in range(live):
            row = back(cache[int(table[seq[r], pos[r] // page]), 0, 0, int(pos[r] % page)])
            assert rel(row[:rank], c[r]) < tol and rel(row[rank:], kr[r]) < tol, r


@pytest.mark.parametrize("kernel", ["simple_f32", "simple_bf16", "mma_prompt", "mma_few"])
@pytest.mark.parametrize("rank, rot, size", [(32, 16, 24), (64, 16, 33), (64, 16, 64), (32, 16, 1), (64, 16, 129)])
def test_latent_attention_behind_a_window(K, kernel, rank, rot, size):
    g = torch.Generator().manual_seed(rank + size)
    dtype = "float32" if kernel == "simple_f32" else "bfloat16"
    few = kernel == "mma_few"
    lengths, before = ([1, 2], [250, 130]) if few else ([150, 37], [0, 200])
    t = step_tables(lengths, before, pad=0)
    heads, page, Dl, scale = 3, 64, rank + rot, 0.4
    total = [b + n for b, n in zip(before, lengths)]
    table, _ = paged(total, 1, page, Dl, dtype, g)
    cache = torch.zeros((int(table.max()) + 1, 1, 1, page, Dl), dtype=TORCH[dtype], device="cuda")
    rows_kv = [torch.randn(n, Dl, generator=g) for n in total]
    for s in range(2):                     # the oldest key inside the last query's window and the one just outside stand out
        last = total[s] - 1
        for j in (last - size, last - size + 1):
            if 0 <= j <= last:
                rows_kv[s][j, :rank] = 2.0 * torch.sign(torch.randn(rank, generator=g))
                rows_kv[s][j, rank:] = 0.0
                rows_kv[s][j, rank] = 30.0
        for j in range(total[s]):
            cache[int(table[s, j // page]), 0, 0, j % page] = dev(rows_kv[s][j], dtype)
    q0 = torch.randn(t.rows, heads, Dl, generator=g)
    q0[:, :, rank] += 4.0
    q = dev(q0, dtype)
    out = torch.zeros((t.rows, heads, rank), dtype=TORCH[dtype], device="cuda")
    if kernel.startswith("simple"):
        K.attn_latent_simple(q, out, cache, table.cuda(), t.positions, t.token_seq, rank, size, scale)
    else:
        K.attn_latent_mma(q, out, cache, table.cuda(), t.q_start, t.q_len, t.kv_before, t.token_seq, t.n_seqs, t.max_q_len, rank, size,
                          scale, n_splits=2 if few and size > 64 else 1)
    K.check_device_errors()
    tol = 2e-5 if dtype == "float32" else 3e-2
    r0, shown = 0, 0.0
    for s in range(2):
        rows = slice(r0, r0 + lengths[s])
        pos = torch.arange(before[s], total[s])
        kv = back(dev(rows_kv[s], dtype))
        j = torch.arange(total[s])[None, :]

        def plain(sz):
            vis = (j <= pos[:, None]) & (pos[:, None] - j < sz)
            p = P.masked_softmax(torch.einsum("ihd,jd->hij", back(q)[rows], kv) * scale, vis[None])
            return torch.einsum("hij,jd->ihd", p, kv[:, :rank])
        want = plain(size)
        assert rel(back(out)[rows], want) < tol, (kernel, s)
        shown = max(shown, rel(plain(size + 1), want), rel(plain(max(size - 1, 1)), want) if size > 1 else 0.0)
        r0 += lengths[s]
    assert shown > 0.15                                                      # the test's inputs do show a fault by one


# ================================================================== the model through the engine
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
                                        ("C", [2, 2, 2, 3, 141]), ("C", [5, 60, 64, 2, 19]), ("C", [64, 64, 22]), ("B", [15, 2, 16, 2, 115])])
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
    # the freed slots and pages serve other requests; what they held before must not show
    again = random_prompts(vocab, [66, 5], 22)
    slots = [eng.open(), eng.open()]
    lg = eng.step([(slots[0], again[0]), (slots[1], again[1])], want="all")
    tally.add(lg[:66], oracles[fold(name, dtype)].logits(again[0]), "slot used again")
    tally.add(lg[66:], oracles[fold(name, dtype)].logits(again[1]), "slot used again")
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_decoding_past_every_window_gives_pages_back_and_keeps_the_first(folders, oracles, name, dtype):
    eng = engine(folders[fold(name, dtype)], dtype, max_tokens=64 * 8)
    toks = random_prompts(oracles[fold(name, dtype)].cfg["vocab"], [5 + 315], 31)[0]
    want = oracles[fold(name, dtype)].logits(toks)
    s, tally = eng.open(), Tally(dtype)
    eng.step([(s, toks[:5])], want=None)
    for t in range(5, len(toks)):
        tally.add(eng.step([(s, [toks[t]])], want="last"), want[t:t + 1], t)
    tally.close()
    eng.check()
    for g in eng.cache.groups:                                       # a window's pages went back, a kept first page did not
        r = g.request
        if r.kind == "window" and r.window + 64 < 320:
            held = [b for b in g.pages.blocks[s] if b >= 0]
            assert len(held) <= -(-r.window // 64) + 1 + (1 if r.keep_first else 0)
            assert (g.pages.blocks[s][0] >= 0) == bool(r.keep_first)


def one_attention_layer(size, keep):
    return {"architecture": "Ludazen", "vocab": 120, "width": 64, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": _att(4, 2, 32, 32, 0.25, 32, 10000.0, size, keep), "mlp": None}]}


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_kept_first_token_counts_far_away_and_the_next_one_does_not(tmp_path, dtype):
    """One attention layer, a window of 16 and two kept tokens: the token at position 1 still moves the logits 200
    tokens on (in a prompt and decoded), the one at position 2 moves nothing beyond its window, to the last bit."""
    cfg = one_attention_layer(16, 2)
    folder = make_ludazen_folder(tmp_path, "kept", cfg=cfg, seed=4)
    oracle = Oracle(folder)
    base = random_prompts(cfg["vocab"], [230], 5)[0]
    res = {}
    for which, place in (("base", None), ("kept", 1), ("next", 2)):
        toks = list(base)
        if place is not None:
            toks[place] = (toks[place] + 17) % cfg["vocab"]
        eng = engine(folder, dtype)
        s = eng.open()
        lg = [eng.step([(s, toks[:200])], want="all")[40:]]
        lg += [eng.step([(s, [t])], want="last") for t in toks[200:]]
        res[which] = torch.cat(lg)
        tally = Tally(dtype)
        tally.add(res[which], oracle.logits(toks)[40:], which)
        tally.close()
        eng.check()
    assert torch.equal(res["next"], res["base"])
    d = (res["kept"] - res["base"]).double().pow(2).mean(-1).sqrt() / res["base"].double().pow(2).mean().sqrt()
    assert d.median().item() > 0.05 and (d > 0.2).double().mean().item() > 0.1, (d.median().item(), d.max().item())


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_head_factors_the_mix_of_heads_and_the_readers_window_count_in_the_model(folders, oracles, dtype):
    eng = engine(folders[fold("A", dtype)], dtype)
    o = oracles[fold("A", dtype)]
    toks = random_prompts(o.cfg["vocab"], [150], 41)[0]
    s = eng.open()
    got = eng.step([(s, toks)], want="all")
    eng.check()
    right = o.logits(toks)
    tally = Tally(dtype)
    tally.add(got, right)
    tally.close()
    w = dict(o.w)
    w["l0.mix.temp"] = torch.ones_like(w["l0.mix.temp"])
    w2 = dict(o.w)
    w2["l3.mix.talk"] = torch.eye(6, dtype=o.w["l3.mix.talk"].dtype)
    c3 = copy.deepcopy(o.cfg)
    c3["layers"][2]["mixer"]["mask"]["size"] = 24                    # the reader with its owner's window
    for wrong in (o.logits(toks, w=w), o.logits(toks, w=w2), o.logits(toks, cfg=c3)):
        e = (wrong - right).pow(2).mean(-1).sqrt() / right.pow(2).mean().sqrt()
        assert e.max().item() > (100 if dtype == "float32" else 1.2) * TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10])
def test_configurations_drawn_from_a_seed(tmp_path, seed, dtype):
    """Other sizes, head counts, layer orders, windows and constants than any written by hand: a prompt in two portions
    beside a second request, then both decoded together, against the plain implementation."""
    cfg = random_config(seed)
    folder = make_ludazen_folder(tmp_path, f"r{seed}", cfg=cfg, seed=100 + seed, steady=dtype == "bfloat16")
    oracle = Oracle(folder)
    eng = engine(folder, dtype, max_tokens=64 * 8, max_slots=3)
    a, b = random_prompts(cfg["vocab"], [150, 21], seed)
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


def test_graphs_on_and_off_give_the_same_logits(folders, oracles):
    toks = random_prompts(oracles["A~"].cfg["vocab"], [40], 5)[0]
    res = []
    for graphs in (True, False):
        eng = engine(folders["A~"], "bfloat16", use_graphs=graphs)
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
    for dtype in DTYPES:
        o = oracles[fold("A", dtype)]
        vocab = o.cfg["vocab"]
        wa, wb = o.logits(toks[0]), o.logits(toks[1])
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[fold("A", dtype)], "--dtype", dtype,
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

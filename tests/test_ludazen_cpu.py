"""Ludazen without a GPU: configuration, recipe, cache plan, page bookkeeping with kept first tokens, and the plain
implementation's mechanisms by hand."""
import copy
import math

import pytest
import torch

import plain_ludazen as P
from ludazen_tiny import LD_A, LD_B, LD_C, LD_CONFIGS, random_config
from braidinfer_b200.cache.pages import GroupPages
from braidinfer_b200.config import ConfigError, LudazenConfig
from braidinfer_b200.models import architecture_for
from braidinfer_b200.weights import tensor_specs_of

D = torch.float64


def spec_of(cfg):
    arch = architecture_for(cfg)
    return arch.build_spec(arch.config_from_dict(cfg))


def test_architecture_is_found_by_its_name_and_every_configuration_is_read():
    for cfg in LD_CONFIGS.values():
        assert architecture_for(cfg).name == "Ludazen"
        c = LudazenConfig.from_dict(cfg)
        assert c.vocab == cfg["vocab"] and len(c.layers) == len(cfg["layers"])
    c = LudazenConfig.from_dict(LD_A)
    a = c.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.rot_dims, a.window, a.keep_first) == (4, 2, 32, 48, 16, 40, 3)
    assert a.rot_scaling.factor == 8.0 and a.rot_scaling.original == 64 and c.layers[3].mixer.rot_scaling is None
    assert c.layers[3].mixer.keep_first == 0                                       # absent: nothing kept
    assert c.layers[1].mixer.kv_from is None and c.layers[2].mixer.kv_from == 1 and c.layers[2].mixer.window == 50
    assert c.layers[1].mlp.shared_ff == 40 and c.layers[3].mlp.shared_ff is None and c.layers[3].mlp.top == 4
    assert c.layers[0].mlp.ff == 72 and c.layers[2].mlp is None


@pytest.mark.parametrize("path, value", [("layers.0.type", "conv"), ("layers.0.mixer.kv_heads", 3), ("layers.0.mixer.rot.dims", 7),
                                         ("layers.0.mixer.rot.dims", 34), ("layers.0.mixer.mask.size", 0), ("layers.0.mixer.mask", None),
                                         ("layers.0.mixer.rot.scaling.factor", -1.0), ("layers.1.mlp.kind", "gated"),
                                         ("layers.1.mlp.router.top", 7), ("layers.2.mixer.kv_from", 2), ("layers.2.mixer.kv_from", 0),
                                         ("layers.2.mixer.kv_rank", 16), ("layers.1.mixer.rot_dim", None), ("norm", None),
                                         ("layers.0.mixer.scale", None), ("layers.1.mixer.vdim", None), ("layers.0.mlp.ff", None)])
def test_a_value_nothing_computes_is_an_error_that_names_its_key(path, value):
    cfg = copy.deepcopy(LD_A)
    cur = cfg
    keys = path.split(".")
    for k in keys[:-1]:
        cur = cur[int(k)] if k.isdigit() else cur[k]
    if value is None:
        del cur[keys[-1]]
    else:
        cur[keys[-1]] = value
    with pytest.raises(ConfigError) as e:
        LudazenConfig.from_dict(cfg)
    assert any(k in str(e.value) for k in [keys[-1]] + ([keys[-2], f"layers[{keys[1]}]"] if len(keys) > 1 else []))


def test_a_layer_reads_the_latent_of_a_layer_that_makes_one():
    cfg = copy.deepcopy(LD_C)
    cfg["layers"][4]["mixer"]["kv_from"] = 2                  # layer 2 reads layer 1's itself
    with pytest.raises(ConfigError):
        LudazenConfig.from_dict(cfg)


def test_recipe_names_the_tensors_of_the_design_and_the_parts_beside_the_existing_ones():
    spec = spec_of(LD_A)
    specs = tensor_specs_of(spec)
    names = set(specs)
    for n in ("embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.temp", "l0.mix.talk",
              "l0.mix.o", "l0.mlp.up", "l0.mlp.up.b", "l0.mlp.down", "l0.mlp.down.b", "l0.mlp.act", "l1.mix.q", "l1.mix.dkv",
              "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv", "l1.mix.o", "l1.mlp.router", "l1.mlp.e0.gate", "l1.mlp.e4.down",
              "l1.mlp.shared.gate", "l1.mlp.shared.up", "l1.mlp.shared.down", "l2.mix.q", "l2.mix.uk", "l2.mix.uv", "l2.mix.o",
              "l3.mlp.e3.up"):
        assert n in names, n
    for n in ("l2.mix.dkv", "l2.mix.dkv.norm", "l2.norm2", "l3.mlp.shared.gate", "l1.mix.g", "l0.mix.sink", "l1.mlp.e5.gate"):
        assert n not in names, n
    assert specs["l0.mix.q"].shape == (4 * 32, 96) and specs["l0.mix.v"].shape == (2 * 48, 96) and specs["l0.mix.o"].shape == (96, 4 * 48)
    assert specs["l0.mix.talk"].shape == (4, 4) and specs["l0.mix.temp"].shape == (4,) and specs["l0.mlp.act"].shape == (2,)
    assert specs["l1.mix.q"].shape == (3 * 32, 96) and specs["l1.mix.dkv"].shape == (48, 96) and specs["l1.mix.uk"].shape == (48, 32)
    assert specs["l2.mix.q"].shape == (2 * 40, 96) and specs["l2.mix.uv"].shape == (32, 32) and specs["head"].shape == (301, 96)
    assert [(e.layer, e.cache_of) for e in spec.schedule] == [(0, None), (1, None), (2, 1), (3, None)]
    assert [L.block for L in spec.layers] == ["prenorm_residual"] * 4
    assert [L.mixer.kind for L in spec.layers] == ["gqa_attention", "latent_attention", "latent_attention", "gqa_attention"]
    assert [L.feed_forward.kind if L.feed_forward else None for L in spec.layers] == ["biased_mlp", "moe", None, "moe"]
    moe = spec.layers[1].feed_forward.params
    assert moe["scoring"] == "sigmoid" and moe["weight_on"] == "input" and moe["shared"].kind == "swiglu"
    assert spec.layers[3].feed_forward.params["shared"] is None and not spec.head.params["tied"]
    m = spec.layers[0].mixer.params
    assert m["keep_first"] == 3 and m["window"] == 40 and m["position_encoding"].params["pairing"] == "half"
    assert spec.layers[1].mixer.params["position_encoding"].params["pairing"] == "adjacent"
    assert spec.layers[2].mixer.params["shared_kv"] and not spec.layers[1].mixer.params["shared_kv"]


def test_cache_plan_keeps_first_tokens_and_the_longest_window_of_a_latents_readers():
    from braidinfer_b200.cache import CacheManager
    from braidinfer_b200.models import DecoderModel
    from braidinfer_b200.parts.runtime import Runtime
    rt = Runtime(act_dtype=torch.bfloat16, device=torch.device("cpu"), kernels=None)
    plan = DecoderModel(spec_of(LD_A), rt).cache_plan()
    r0, r1, r2, r3 = (p[0] for p in plan)
    assert (r0.kind, r0.num_kv_heads, r0.head_dim, r0.window, r0.planes, r0.keep_first) == ("window", 2, 48, 40, 2, 3)
    assert (r1.kind, r1.num_kv_heads, r1.head_dim, r1.window, r1.planes) == ("window", 1, 48, 50, 1)   # its reader's window
    assert r2 == r1 and [p[1] for p in plan] == [None, None, 1, None] and all(p[2] == 0 for p in plan)
    assert (r3.head_dim, r3.window, r3.keep_first) == (16, 64, 0)
    plan = DecoderModel(spec_of(LD_B), rt).cache_plan()
    assert plan[1][0].head_dim == 48 and plan[1][0].keep_first == 9 and plan[2][0].head_dim == 64
    plan = DecoderModel(spec_of(LD_C), rt).cache_plan()
    assert [p[0].window for p in plan] == [70, 33, 33, 96, 33] and [p[1] for p in plan] == [None, None, 1, None, 1]
    CacheManager(plan, 256, 2, torch.bfloat16, "cpu")                       # readers and owners fit together


def test_pages_of_kept_first_tokens_stay_while_the_window_moves_on():
    g = GroupPages(16, 4, "window", window=5, keep_first=6)                  # pages of 4: the first two hold kept tokens
    g.open(0)
    g.grow(0, 30)
    g.shrink(0, 30)                                                          # positions <= 25 are dead but for the kept
    b = g.blocks[0]
    assert b[0] >= 0 and b[1] >= 0 and b[2:6] == [-1, -1, -1, -1] and b[6] >= 0 and b[7] >= 0
    assert g.pool.in_use == 4
    g.close(0)
    assert g.pool.in_use == 0
    plain = GroupPages(16, 4, "window", window=5)
    plain.open(0)
    plain.grow(0, 30)
    plain.shrink(0, 30)
    assert plain.blocks[0][:6] == [-1] * 6 and plain.pool.in_use == 2


def test_configurations_drawn_from_a_seed_are_read():
    for seed in range(40):
        cfg = random_config(seed)
        spec = spec_of(cfg)
        assert len(spec.schedule) == len(cfg["layers"]) == len(spec.layers)
        tensor_specs_of(spec)


# ---------------------------------------------------------------------------------------------- the oracle by hand
def test_window_with_kept_first_tokens_by_hand():
    v = P.visible(6, 2, 1)
    want = [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0], [1, 0, 1, 1, 0, 0], [1, 0, 0, 1, 1, 0], [1, 0, 0, 0, 1, 1]]
    assert v.tolist() == [[bool(x) for x in r] for r in want]
    assert P.visible(4, 1).tolist() == torch.eye(4, dtype=torch.bool).tolist()            # a window of one: itself
    assert P.visible(5, 100, 0).tolist() == torch.ones(5, 5).tril().bool().tolist()


def test_stretched_frequencies_by_hand():
    f, amp = P.frequencies({"base": 100.0, "dims": 8})
    assert torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=D)) and amp == 1.0
    # original 64, fast 4 turns, slow 1: d(4) = 8 ln(64 / (8 pi)) / (2 ln 100) = 0.812 -> lo 0; d(1) = 2.016 -> hi 3
    f2, amp2 = P.frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0}})
    ramp = torch.tensor([0.0, 1 / 3, 2 / 3, 1.0], dtype=D)
    assert torch.allclose(f2, f / 4.0 * ramp + f * (1 - ramp)) and abs(amp2 - (0.1 * math.log(4.0) + 1)) < 1e-12


def test_rotation_layouts_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=D)
    rot = {"base": 1.0, "dims": 4}                                           # every pair turns by the position itself
    pos = torch.tensor([1])
    c, s = math.cos(1.0), math.sin(1.0)
    half = P.rotate(x, pos, rot, "half")[0, 0]                               # pairs (0, 2) and (1, 3); 4 and 5 pass
    assert torch.allclose(half, torch.tensor([1 * c - 3 * s, 2 * c - 4 * s, 3 * c + 1 * s, 4 * c + 2 * s, 5.0, 6.0], dtype=D))
    pairs = P.rotate(x, pos, rot, "pairs")[0, 0]                             # pairs (0, 1) and (2, 3)
    assert torch.allclose(pairs, torch.tensor([1 * c - 2 * s, 2 * c + 1 * s, 3 * c - 4 * s, 4 * c + 3 * s, 5.0, 6.0], dtype=D))
    assert torch.equal(P.rotate(x, torch.tensor([0]), rot, "half"), x)


def test_attention_of_two_tokens_by_hand():
    m = {"heads": 2, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 0.5, "rot": {"base": 10.0, "dims": 0}, "mask": {"size": 5}}
    h = torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=D)
    w = {"q": torch.tensor([[1.0, 0.0], [0.0, 1.0], [2.0, 0.0], [0.0, 2.0]], dtype=D), "k": torch.eye(2, dtype=D),
         "v": torch.tensor([[1.0, 1.0]], dtype=D), "temp": torch.tensor([1.0, 3.0], dtype=D),
         "talk": torch.tensor([[1.0, 0.0], [0.5, -1.0]], dtype=D), "o": torch.eye(2, dtype=D)}
    out = P.attention(h, w, m)
    # token 1 (h = [0, 2]): keys [1, 0] and [0, 2], values 1 and 2.  head 0: q = [0, 2]: scores 0, 4 * 0.5 * 1 = 2
    # head 1: q = [0, 4]: scores 0, 8 * 0.5 * 3 = 12
    p0 = math.exp(2.0) / (1 + math.exp(2.0))
    p1 = math.exp(12.0) / (1 + math.exp(12.0))
    o0 = (1 - p0) * 1 + p0 * 2
    mixed = [0.5 * (1 - p0) - (1 - p1), 0.5 * p0 - p1]                        # head 1 applies 0.5 p_0 - p_1
    assert torch.allclose(out[1], torch.tensor([o0, mixed[0] * 1 + mixed[1] * 2], dtype=D))
    assert torch.allclose(out[0], torch.tensor([1.0, -0.5], dtype=D))          # alone: p = 1, mixed 1 and 0.5 - 1


def test_latent_attention_shares_a_latent_by_hand():
    m = {"heads": 1, "dim": 1, "rot_dim": 2, "vdim": 1, "kv_rank": 2, "scale": 1.0, "rot": {"base": 1.0, "dims": 2}, "mask": {"size": 1}}
    h = torch.tensor([[3.0, 4.0]], dtype=D)
    w = {"q": torch.tensor([[1.0, 0.0], [0.0, 0.0], [0.0, 0.0]], dtype=D),
         "dkv": torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 0.0], [0.0, 1.0]], dtype=D), "dkv.norm": torch.tensor([2.0, 1.0], dtype=D),
         "uk": torch.tensor([[1.0, 1.0]], dtype=D), "uv": torch.tensor([[1.0, -1.0]], dtype=D), "o": torch.ones(1, 1, dtype=D)}
    out, (c, kr) = P.latent_attention(h, w, m, 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(c, torch.tensor([[6.0 / r, 4.0 / r]], dtype=D)) and torch.allclose(kr, torch.tensor([[3.0, 4.0]], dtype=D))
    assert torch.allclose(out, torch.tensor([[2.0 / r]], dtype=D))             # one visible key: the value itself
    other = {"q": w["q"], "uk": w["uk"], "uv": torch.tensor([[0.0, 1.0]], dtype=D), "o": w["o"]}
    out2, kept = P.latent_attention(h, other, m, 0.0, shared=(c, kr))          # no dkv of its own
    assert torch.allclose(out2, torch.tensor([[4.0 / r]], dtype=D)) and kept[0] is c


def test_feed_forwards_by_hand():
    z = torch.tensor([2.0, -1.0, 0.0], dtype=D)
    p, q = torch.tensor(0.0, dtype=D), torch.tensor(1.0, dtype=D)
    sp0, sp1 = math.log(2.0), math.log(1 + math.e)
    want = [sp0 * 4 + 1.0, (0.5 + sp1) * (math.exp(-1.0) - 1 + 1) - 0.5, 0.0]
    assert torch.allclose(P.xielu(z, p, q), torch.tensor(want, dtype=D))
    h = torch.tensor([[1.0, -2.0]], dtype=D)
    w = {"up": torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=D), "up.b": torch.tensor([1.0, 1.0], dtype=D),
         "down": torch.tensor([[1.0, 1.0]], dtype=D), "down.b": torch.tensor([10.0], dtype=D), "act": torch.tensor([0.0, 1.0], dtype=D)}
    assert torch.allclose(P.dense(h, w), torch.tensor([[want[0] + want[1] + 10.0]], dtype=D))
    idx, wgt = P.route(torch.tensor([[1.0, 0.0]], dtype=D), torch.tensor([[0.0, 0.0], [math.log(3.0), 0.0], [-1.0, 0.0]], dtype=D), 2)
    assert idx.tolist() == [[1, 0]] and torch.allclose(wgt, torch.tensor([[0.75, 0.5]], dtype=D))        # not renormalised
    we = {"router": torch.tensor([[0.0, 0.0], [math.log(3.0), 0.0]], dtype=D)}
    for e in range(2):
        we[f"e{e}.gate"] = torch.tensor([[1.0 + e, 0.0]], dtype=D)
        we[f"e{e}.up"] = torch.tensor([[1.0, 0.0]], dtype=D)
        we[f"e{e}.down"] = torch.tensor([[1.0], [0.0]], dtype=D)
    we.update({"shared.gate": torch.tensor([[0.0, 1.0]], dtype=D), "shared.up": torch.tensor([[0.0, 1.0]], dtype=D),
               "shared.down": torch.tensor([[0.0], [1.0]], dtype=D)})
    y = P.moe(h, we, {"router": {"experts": 2, "top": 1}, "shared": {"ff": 1}})
    silu = lambda t: t / (1 + math.exp(-t))                                   # noqa: E731
    # expert 1 with weight 0.75 on its input: gate 2 * 0.75, up 0.75; the shared one sees h itself
    assert torch.allclose(y[0], torch.tensor([silu(1.5) * 0.75, silu(-2.0) * -2.0], dtype=D))

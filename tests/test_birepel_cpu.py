"""Birepel without a GPU: configuration, recipe, cache plan, and the plain implementation's mechanisms by hand."""
import copy
import math

import pytest
import torch

import plain_birepel as P
from birepel_tiny import BR_A, BR_B, BR_C, BR_CONFIGS, BR_D, random_config
from braidinfer_b200.config import BirepelConfig, ConfigError
from braidinfer_b200.models import architecture_for
from braidinfer_b200.weights import tensor_specs_of

D = torch.float64


def spec_of(cfg):
    arch = architecture_for(cfg)
    return arch.build_spec(arch.config_from_dict(cfg))


def test_architecture_is_found_by_its_name_and_every_configuration_is_read():
    for cfg in BR_CONFIGS.values():
        assert architecture_for(cfg).name == "Birepel"
        c = BirepelConfig.from_dict(cfg)
        assert c.vocab == cfg["vocab"] and len(c.layers) == len(cfg["layers"]) and c.max_positions == cfg["max_positions"]
    c = BirepelConfig.from_dict(BR_A)
    assert c.layers[0].mixer.vdim == 48 and c.layers[0].mixer.temp_every == 16 and c.layers[0].mixer.temp_coef == 0.5
    assert c.layers[1].mixer.gate_cap == 8.0 and c.layers[1].mlp.limit == 2.0 and c.layers[3].mlp is None
    assert c.layers[0].mlp.experts == 6 and c.layers[0].mlp.top == 2 and c.layers[2].weights_of == 0
    assert BirepelConfig.from_dict(BR_B).layers[1].mixer.temp_coef is None
    assert [L.weights_of for L in BirepelConfig.from_dict(BR_C).layers] == [0, 1, 1, 1]       # a chain ends at its owner


@pytest.mark.parametrize("path, value", [("layers.0.type", "conv"), ("layers.0.mixer.kv_heads", 3), ("layers.1.mixer.gate_cap", 0.0),
                                         ("layers.1.mlp.limit", -1.0), ("layers.0.mlp.kind", "gated"), ("layers.0.mlp.router.top", 7),
                                         ("layers.2.weights_of", 9), ("layers.2.mixer.heads", 2), ("norm", None), ("max_positions", None),
                                         ("layers.0.mixer.scale", None), ("layers.1.mixer.vdim", None), ("layers.0.mixer.q_temp.every", 0)])
def test_a_value_nothing_computes_is_an_error_that_names_its_key(path, value):
    cfg = copy.deepcopy(BR_A)
    cur = cfg
    keys = path.split(".")
    for k in keys[:-1]:
        cur = cur[int(k)] if k.isdigit() else cur[k]
    if value is None:
        del cur[keys[-1]]
    else:
        cur[keys[-1]] = value
    with pytest.raises(ConfigError) as e:
        BirepelConfig.from_dict(cfg)
    assert keys[-1] in str(e.value) or keys[-2] in str(e.value) or f"layers[{keys[1]}]" in str(e.value)


def test_layers_that_borrow_in_a_circle_are_refused():
    cfg = copy.deepcopy(BR_C)
    cfg["layers"][1]["weights_of"] = 3
    with pytest.raises(ConfigError):
        BirepelConfig.from_dict(cfg)


def test_recipe_names_the_tensors_of_the_design_and_the_parts_beside_the_existing_ones():
    spec = spec_of(BR_A)
    specs = tensor_specs_of(spec)
    names = set(specs)
    for n in ("embed", "pos", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.g", "l0.mix.sink",
              "l0.mix.o", "l0.mlp.router", "l0.mlp.e0.up", "l0.mlp.e5.down", "l1.mix.q", "l1.mix.i", "l1.mix.i.b", "l1.mix.f",
              "l1.mix.f.b", "l1.mix.norm", "l1.mix.g", "l1.mix.o", "l1.mlp.gate", "l1.mlp.up", "l1.mlp.down", "l3.norm1"):
        assert n in names, n
    assert not any(n.startswith("l2.") for n in names)                   # the third layer reads the first one's tensors
    assert "l3.norm2" not in names and "l0.mlp.e0.gate" not in names
    assert specs["pos"].shape == (400, 96) and specs["l0.mix.v"].shape == (2 * 48, 96) and specs["l0.mix.g"].shape == (4, 96)
    assert specs["l0.mix.o"].shape == (96, 4 * 48) and specs["l0.mix.sink"].shape == (4,) and specs["l1.mix.norm"].shape == (3 * 40,)
    assert specs["l1.mix.g"].shape == (120, 96) and specs["l1.mix.i"].shape == (3, 96) and specs["l0.mlp.e0.up"].shape == (40, 96)
    assert [e.layer for e in spec.schedule] == [0, 1, 0, 2] and len(spec.layers) == 3
    assert [L.block for L in spec.layers] == ["sublayer_norm_residual"] * 3
    assert [L.mixer.kind for L in spec.layers] == ["gqa_attention", "mlstm", "mlstm"]
    assert [L.feed_forward.kind if L.feed_forward else None for L in spec.layers] == ["moe", "clamped_glu", None]
    assert spec.layers[0].mixer_norm.params["offset"] == 1.0 and spec.final_norm.params["offset"] == 1.0
    assert spec.embedding.params["positions"] == {"name": "pos", "max": 400} and spec.head.params["tied"] and spec.max_position == 400
    assert [e.layer for e in spec_of(BR_C).schedule] == [0, 1, 1, 1]


def test_cache_plan_gives_every_run_a_cache_or_state_of_its_own():
    from braidinfer_b200.models import DecoderModel
    from braidinfer_b200.parts.runtime import Runtime
    rt = Runtime(act_dtype=torch.bfloat16, device=torch.device("cpu"), kernels=None)
    plan = DecoderModel(spec_of(BR_A), rt).cache_plan()
    assert len(plan) == 4 and all(cache_of is None for _, cache_of, _ in plan)
    req0, _, st0 = plan[0]
    assert (req0.kind, req0.num_kv_heads, req0.head_dim, req0.window, req0.planes) == ("full", 2, 48, None, 2) and st0 == 0
    assert plan[2][0] == req0                                            # the borrowing layer: the same request, another entry
    assert plan[1][0] is None and plan[1][2] == 3 * 24 * 41 * 4 + 3 * 4 and plan[3][2] == 2 * 16 * 17 * 4 + 2 * 4
    plan = DecoderModel(spec_of(BR_B), rt).cache_plan()
    assert plan[1][0].head_dim == 48                                     # heads of 40 padded to the next size the kernels take
    plan = DecoderModel(spec_of(BR_C), rt).cache_plan()
    assert [p[0].head_dim for p in plan] == [64, 128, 128, 128]
    assert all(p[0] is None for p in DecoderModel(spec_of(BR_D), rt).cache_plan())


def test_configurations_drawn_from_a_seed_are_read():
    for seed in range(30):
        cfg = random_config(seed)
        spec = spec_of(cfg)
        assert len(spec.schedule) == len(cfg["layers"])
        assert len(spec.layers) == sum(1 for L in cfg["layers"] if L.get("weights_of") is None)


# ---------------------------------------------------------------------------------------------- the oracle by hand
def test_query_temperature_by_hand():
    t = P.query_temperature(torch.tensor([0, 1, 2, 3, 4, 5, 127]), 0.5, 3)
    want = [1.0, 1.0, 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(3),
            1 + 0.5 * math.log(43)]
    assert torch.allclose(t, torch.tensor(want, dtype=D))
    assert torch.allclose(P.query_temperature(torch.tensor([0, 9]), 2.0, 1), torch.tensor([1 + 2 * math.log(2), 1 + 2 * math.log(11)], dtype=D))


def test_sink_softmax_by_hand():
    s = torch.tensor([[0.0, math.log(3.0), 5.0]], dtype=D)
    vis = torch.tensor([[True, True, False]])
    p = P.sink_softmax(s, vis, torch.tensor([[math.log(4.0)]], dtype=D))
    assert torch.allclose(p, torch.tensor([[1 / 8, 3 / 8, 0.0]], dtype=D))
    p = P.sink_softmax(s, vis, torch.tensor([[-1e9]], dtype=D))           # a sink far below: the plain softmax
    assert torch.allclose(p, torch.tensor([[0.25, 0.75, 0.0]], dtype=D))


def test_attention_of_one_token_by_hand():
    m = {"heads": 2, "kv_heads": 1, "dim": 2, "vdim": 3, "scale": 0.5, "q_temp": {"coef": 1.0, "every": 1}}
    h = torch.tensor([[1.0, 2.0]], dtype=D)
    w = {"q": torch.tensor([[3.0, 0.0], [0.0, 2.0], [1.0, 0.0], [0.0, 0.0]], dtype=D), "k": torch.eye(2, dtype=D),
         "v": torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=D), "g": torch.tensor([[0.0, 0.0], [1.0, 1.0]], dtype=D),
         "sink": torch.tensor([0.0, math.log(2.0)], dtype=D), "o": torch.eye(6, dtype=D)}
    out = P.attention(h, w, m, 0.0)
    temp = 1 + math.log(2.0)                                              # position 0: floor(1 / 1) + 1 = 2
    k = torch.tensor([1.0, 2.0]) / math.sqrt(2.5)
    q0 = torch.tensor([3.0, 4.0]) / math.sqrt(12.5) * temp
    q1 = torch.tensor([1.0, 0.0]) / math.sqrt(0.5) * temp
    v = torch.tensor([1.0, 2.0, 3.0], dtype=D)
    e0, e1 = math.exp(float(q0 @ k) * 0.5), math.exp(float(q1 @ k) * 0.5)
    want = torch.cat([v * e0 / (e0 + 1.0) * 0.5, v * e1 / (e1 + 2.0) / (1 + math.exp(-3.0))])
    assert torch.allclose(out[0], want)


def test_matrix_memory_of_two_tokens_by_hand():
    m = {"heads": 1, "dim": 1, "vdim": 2, "gate_cap": 100.0}
    h = torch.tensor([[1.0], [2.0]], dtype=D)
    one = torch.ones(1, 1, dtype=D)
    w = {"q": one, "k": one, "v": torch.tensor([[1.0], [-1.0]], dtype=D), "i": one * 0.0, "i.b": torch.tensor([math.log(2.0)], dtype=D),
         "f": one * 0.0, "f.b": torch.tensor([0.0], dtype=D), "norm": torch.ones(2, dtype=D), "g": torch.zeros(2, 1, dtype=D),
         "o": torch.eye(2, dtype=D)}
    # cap 100: the caps change nothing to six digits.  Gates in plain terms: input 2, forget 1/2 at both tokens.
    # C1 = 2 k1 v1^T = 2 [1, -1], n1 = 2;  C2 = C1 / 2 + 2 k2 v2^T = [1, -1] + 2 * 2 * [2, -2] = [9, -9], n2 = 1 + 4 = 5
    # read-out 2: q2 = 2: C2 q / max(|n2 q|, 1) = [18, -18] / 10; unit norm -> [1, -1]; times sigmoid(0) = 1/2
    out = P.mlstm(h, w, m, 0.0)
    assert torch.allclose(out, torch.tensor([[0.5, -0.5], [0.5, -0.5]], dtype=D), atol=1e-5)
    # the running maximum starts at 0, not below: a first token whose gates are small is floored by exp(-m) = 1
    w2 = dict(w)
    w2["i.b"] = torch.tensor([math.log(0.01)], dtype=D)
    w2["norm"] = torch.tensor([1.0, 1.0], dtype=D)
    S = 0.01 * 1.0 * torch.tensor([1.0, -1.0], dtype=D)                   # m_1 = max(log(1/2) + 0, log 0.01) = log(1/2)
    # held in units of exp(m_1): S' = S / 0.5, n' = 0.01 / 0.5 = 0.02; denominator max(0.02, exp(-m_1) = 2) + 1e-6
    o = (S / 0.5) / (2 + 1e-6)
    got = P.mlstm(h[:1], w2, {**m, "gate_cap": 1e4}, 1e-6)
    want = o / torch.sqrt((o * o).mean() + 1e-6) * 0.5
    assert torch.allclose(got[0], want, atol=1e-6)


def test_feed_forwards_by_hand():
    h = torch.tensor([[1.0, -2.0]], dtype=D)
    w = {"gate": torch.tensor([[5.0, 0.0], [1.0, 0.0]], dtype=D), "up": torch.tensor([[0.0, 3.0], [0.5, 0.0]], dtype=D), "down": torch.eye(2, dtype=D)}
    y = P.dense_ff(h, w, {"limit": 2.0})
    want = [2.0 / (1 + math.exp(-1.702 * 2.0)) * (-2.0 + 1.0), 1.0 / (1 + math.exp(-1.702)) * 1.5]
    assert torch.allclose(y[0], torch.tensor(want, dtype=D))
    idx, wgt = P.route(torch.tensor([[0.0, math.log(3.0), -1.0, math.log(2.0)]], dtype=D), 2)
    assert idx.tolist() == [[1, 3]] and torch.allclose(wgt, torch.tensor([[0.6, 0.4]], dtype=D))
    we = {"router": torch.tensor([[1.0, 0.0], [0.0, 0.0], [0.0, -1.0]], dtype=D)}
    for e in range(3):
        we[f"e{e}.up"] = torch.tensor([[1.0 + e, 0.0], [0.0, 1.0]], dtype=D)
        we[f"e{e}.down"] = torch.tensor([[1.0, 1.0]], dtype=D)
    y = P.moe_ff(h, we, {"router": {"experts": 3, "top": 2}})               # logits [1, 0, 2]: experts 2 and 0
    a, b = math.exp(2.0), math.exp(1.0)
    assert torch.allclose(y[0], torch.tensor([(a * 9.0 + b * 1.0) / (a + b)], dtype=D))   # relu(-2)^2 = 0 in both


def test_a_layer_that_borrows_reads_its_owners_tensors():
    cfg = copy.deepcopy(BR_A)
    assert [P.owner(cfg, i) for i in range(4)] == [0, 1, 0, 3]
    assert [P.owner(BR_C, i) for i in range(4)] == [0, 1, 1, 1]

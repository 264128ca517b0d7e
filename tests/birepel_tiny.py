"""Small Birepel configurations of the tests' own (config.json dictionaries) and helpers to write model folders
whose weights make faults show: streams of order one, peaked attention, sinks of both signs, forget gates close to
one so that a token far back still counts in a memory.

BR_A: attention whose value heads are wider than its key heads (both padded to one size), a temperature that changes
every 16 positions, a mixture of experts; a matrix memory with a dense feed-forward; the first layer's tensors used
again by a third layer with a cache of its own; a memory without a feed-forward.
BR_B: a width that is no multiple of 8 (the plain products serve it), a memory first with top = experts, one
attention head group a head (kv_heads = heads) of a size that is no multiple of 16, no temperature.
BR_C: attention layers only, head sizes the tcgen05 kernel takes (64, and keys of 128 with values of 64), one
kv head, a temperature that changes at every position, and a chain of layers that read the second layer's tensors.
BR_D: memories only (no cache of keys at all): a key size above 128, a value size that fills no tile, one head.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def _att(heads, kv, dim, vdim, scale, temp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return m


def _mem(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


BR_A: Dict = {
    "architecture": "Birepel", "vocab": 311, "width": 96, "max_positions": 400, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _att(4, 2, 32, 48, 0.3, (0.5, 16)), "mlp": _moe(40, 6, 2)},
        {"type": "mlstm", "mixer": _mem(3, 24, 40, 8.0), "mlp": _dense(136, 2.0)},
        {"type": "attention", "mixer": _att(4, 2, 32, 48, 0.3, (0.5, 16)), "mlp": _moe(40, 6, 2), "weights_of": 0},
        {"type": "mlstm", "mixer": _mem(2, 16, 16, 20.0), "mlp": None},
    ],
}

BR_B: Dict = {
    "architecture": "Birepel", "vocab": 257, "width": 100, "max_positions": 320, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mlstm", "mixer": _mem(1, 40, 20, 15.0), "mlp": _moe(24, 4, 4)},
        {"type": "attention", "mixer": _att(3, 3, 40, 40, 0.25), "mlp": _dense(60, 0.7)},
    ],
}

BR_C: Dict = {
    "architecture": "Birepel", "vocab": 200, "width": 128, "max_positions": 384, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _att(8, 1, 64, 64, 0.2, (0.1, 1)), "mlp": _dense(64, 3.0)},
        {"type": "attention", "mixer": _att(2, 1, 128, 64, 0.09, (1.0, 100)), "mlp": _moe(16, 3, 1)},
        {"type": "attention", "mixer": _att(2, 1, 128, 64, 0.09, (1.0, 100)), "mlp": _moe(16, 3, 1), "weights_of": 1},
        {"type": "attention", "mixer": _att(2, 1, 128, 64, 0.09, (1.0, 100)), "mlp": _moe(16, 3, 1), "weights_of": 2},
    ],
}

BR_D: Dict = {
    "architecture": "Birepel", "vocab": 128, "width": 64, "max_positions": 330, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mlstm", "mixer": _mem(2, 136, 8, 6.0), "mlp": None},
        {"type": "mlstm", "mixer": _mem(4, 48, 70, 12.0), "mlp": _dense(96, 1.0)},
        {"type": "mlstm", "mixer": _mem(1, 8, 24, 3.0), "mlp": _moe(32, 5, 3)},
    ],
}

BR_CONFIGS = {"A": BR_A, "B": BR_B, "C": BR_C, "D": BR_D}
BR_SEEDS = {"A": 5, "B": 19, "C": 23, "D": 43}

# factors on the drawn tensors, by the end of their names
GAINS = {"embed": 40.0, "pos": 15.0, ".mix.q": 10.0, ".mix.k": 10.0, ".mix.v": 10.0, ".mix.g": 20.0, ".mix.o": 6.0, ".mix.sink": 3.0,
         ".mix.i": 30.0, ".mix.f": 2.0, ".norm1": 10.0, ".norm2": 10.0, "final.norm": 10.0, ".mlp.gate": 8.0, ".mlp.up": 8.0,
         ".mlp.down": 8.0, ".mlp.router": 40.0, ".up": 10.0, ".down": 8.0}


def shape_weights(tensors: Dict[str, torch.Tensor], cfg: Dict = None, steady: bool = False, gains: Dict = None) -> Dict[str, torch.Tensor]:
    """The drawn tensors times their gains.  `steady`: the routers' choices rest on no close call, whatever the
    precision of the run.  The last columns of the stream, one an expert, are set apart: the table of positions and
    every norm on a sublayer's output write nothing there, so they hold what the token's embedding put there, a
    quarter times a permutation of 0 .. experts - 1 drawn for the token, and the router's row e reads column e of
    them alone, times 8.  Its logits are then exact multiples of 2 in any run, no two of a token equal, while the
    softmax over the chosen ones still mixes them (0.88 to 0.12 with two)."""
    out = {}
    table = dict(GAINS, **(gains or {}))
    for n, t in tensors.items():
        f = next((v for k, v in table.items() if n.endswith(k)), 1.0)
        x = t.float() * f
        if n.endswith(".f.b"):
            x = x + 5.0                    # forget gates near one: a memory keeps hundreds of tokens
        out[n] = x.to(t.dtype)
    if steady:
        most = max([L["mlp"]["router"]["experts"] for L in cfg["layers"] if L.get("mlp") and L["mlp"]["kind"] == "moe"] or [0])
        width = cfg["width"]
        g = torch.Generator().manual_seed(width + most)
        for n, t in out.items():
            x = t.float()
            if n == "pos":
                x[:, width - most:] = 0.0
            elif n == "embed":
                for tok in range(x.shape[0]):
                    x[tok, width - most:] = 0.25 * torch.randperm(most, generator=g).float()
            elif n.endswith(".norm1") or n.endswith(".norm2"):
                x[width - most:] = -1.0
            elif n.endswith(".mlp.router"):
                x.zero_()
                for e in range(x.shape[0]):
                    x[e, width - most + e] = 8.0
            out[n] = x.to(t.dtype)
    return out


def make_birepel_folder(tmp_path, name: str, cfg: Dict = None, seed: int = None, steady: bool = False, gains: Dict = None) -> str:
    """Write a model folder for configuration `name` (or `cfg`) with shaped random weights (`gains` replaces entries
    of `GAINS`)."""
    from braidinfer_b200.weights import open_model_folder, save_file, write_random_model
    cfg = dict(cfg if cfg is not None else BR_CONFIGS[name])
    seed = BR_SEEDS.get(name, 1) if seed is None else seed
    folder = os.path.join(str(tmp_path), f"birepel_{name}" + ("_steady" if steady else ""))
    write_random_model(cfg, folder, seed)
    tensors = {n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    save_file(shape_weights(tensors, cfg, steady, gains), os.path.join(folder, "model.safetensors"))
    return folder


def random_config(seed: int) -> Dict:
    """A configuration drawn from a seed: sizes, head counts, the order and number of layers, who reads whose tensors
    and the constants all vary, within what a test can afford."""
    import random
    r = random.Random(seed)

    def divisor(n):
        return r.choice([d for d in range(1, n + 1) if n % d == 0])

    layers = []
    for i in range(r.randint(2, 6)):
        if layers and r.random() < 0.25:
            j = r.randrange(len(layers))
            layers.append({**{k: v for k, v in layers[j].items() if k != "weights_of"}, "weights_of": j})
            continue
        u = r.random()
        mlp = None if u < 0.15 else (_dense(r.choice([24, 40, 72, 100]), r.choice([0.5, 1.5, 7.0])) if u < 0.55 else None)
        if u >= 0.55:
            experts = r.randint(1, 9)
            mlp = _moe(r.choice([8, 16, 24, 40]), experts, r.randint(1, experts))
        if r.random() < 0.5:
            heads = r.choice([1, 2, 3, 4, 6, 8])
            dim = r.choice([8, 16, 24, 32, 40, 64, 80, 128])
            temp = (r.choice([0.1, 0.3, 1.0]), r.choice([1, 2, 7, 64, 128, 1000])) if r.random() < 0.7 else None
            layers.append({"type": "attention", "mlp": mlp,
                           "mixer": _att(heads, divisor(heads), dim, r.choice([dim, dim, 8, 24, 64, 72]), r.choice([dim ** -0.5, 0.2, 0.07]), temp)})
        else:
            layers.append({"type": "mlstm", "mlp": mlp,
                           "mixer": _mem(r.randint(1, 5), r.choice([4, 8, 12, 20, 32, 40, 72, 136]), r.choice([4, 8, 12, 24, 36, 63, 64]),
                                         r.choice([2.0, 8.0, 15.0, 30.0]))})
    return {"architecture": "Birepel", "vocab": r.randint(90, 400), "width": r.choice([40, 48, 64, 72, 96, 100]),
            "max_positions": 256, "norm": {"eps": r.choice([1e-6, 1e-5])}, "layers": layers}


def folder_config(folder: str) -> Dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)

"""Small Ludazen configurations of the tests' own (config.json dictionaries) and helpers to write model folders whose
weights make faults show: streams of order one, peaked attention, head factors and mixing matrices far from one.

LD_A: attention whose value heads are wider than its key heads and whose rotation turns half a head with stretched
frequencies, three kept first tokens beside a window of 40; a latent layer with a mixture of experts and a shared
expert; a latent layer that reads the second layer's latent with a longer window, other heads and no feed-forward;
attention with a window of exactly one page, nothing kept, and top = experts without a shared expert.
LD_B: a width that is no multiple of 8 (the plain products serve it); a latent layer of one head whose window no
prompt fills; attention with one kv head a head, a head size that is no multiple of 16, more kept tokens (9) than the
window holds (7), one expert; attention with one kv head and values half as wide as keys, one kept token.
LD_C: sizes the tensor cores take: four kv heads of 64 (their values fit one launch) and of 128 (two launches), kept
tokens in both, a latent that two later layers read with shorter and equal windows.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def _att(heads, kv, dim, vdim, scale, rot_dims, base, size, keep=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": {"base": base, "dims": rot_dims}, "mask": {"size": size}}
    if keep is not None:
        m["mask"]["keep_first"] = keep
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def _lat(heads, dim, rot, vdim, rank, scale, base, size, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot}, "mask": {"size": size}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(ff, experts, top, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def _dense(ff):
    return {"kind": "dense", "ff": ff}


LD_A: Dict = {
    "architecture": "Ludazen", "vocab": 301, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _att(4, 2, 32, 48, 0.2, 16, 10000.0, 40, 3, (8.0, 64, 16.0, 2.0)), "mlp": _dense(72)},
        {"type": "latent_attention", "mixer": _lat(3, 16, 16, 24, 32, 0.2, 1000.0, 24), "mlp": _moe(24, 5, 2, 40)},
        {"type": "latent_attention", "mixer": _lat(2, 24, 16, 16, 32, 0.15, 1000.0, 50, kv_from=1), "mlp": None},
        {"type": "attention", "mixer": _att(6, 3, 16, 16, 0.3, 16, 500.0, 64), "mlp": _moe(16, 4, 4)},
    ],
}

LD_B: Dict = {
    "architecture": "Ludazen", "vocab": 257, "width": 100, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": _lat(1, 8, 8, 12, 20, 0.3, 100.0, 1000), "mlp": _dense(60)},
        {"type": "attention", "mixer": _att(3, 3, 40, 40, 0.18, 40, 3000.0, 7, 9), "mlp": _moe(20, 1, 1, 16)},
        {"type": "attention", "mixer": _att(2, 1, 64, 32, 0.12, 8, 10000.0, 300, 1, (2.0, 32, 4.0, 1.0)), "mlp": None},
    ],
}

LD_C: Dict = {
    "architecture": "Ludazen", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _att(8, 4, 64, 64, 0.12, 32, 10000.0, 70, 5, (4.0, 128, 8.0, 1.0)), "mlp": _moe(32, 8, 2, 64)},
        {"type": "latent_attention", "mixer": _lat(4, 32, 16, 32, 64, 0.15, 5000.0, 33), "mlp": _dense(136)},
        {"type": "latent_attention", "mixer": _lat(4, 32, 16, 32, 64, 0.15, 5000.0, 20, kv_from=1), "mlp": _moe(16, 3, 1, 24)},
        {"type": "attention", "mixer": _att(4, 4, 128, 128, 0.09, 128, 100000.0, 96, 2), "mlp": _dense(64)},
        {"type": "latent_attention", "mixer": _lat(2, 16, 16, 48, 64, 0.2, 5000.0, 33, kv_from=1), "mlp": None},
    ],
}

LD_CONFIGS = {"A": LD_A, "B": LD_B, "C": LD_C}
LD_SEEDS = {"A": 3, "B": 17, "C": 29}

# factors on the drawn tensors, by the end of their names (the first that fits)
GAINS = {"embed": 40.0, ".mix.q": 7.0, ".mix.k": 7.0, ".mix.v": 10.0, ".mix.o": 8.0, ".mix.dkv.norm": 1.0, ".mix.dkv": 10.0,
         ".mix.uk": 8.0, ".mix.uv": 16.0, ".mix.temp": 2.0, ".mix.talk": 2.0, ".mlp.router": 8.0, ".up.b": 10.0, ".down.b": 5.0,
         ".mlp.act": 1.0, ".gate": 8.0, ".up": 8.0, ".down": 8.0, "head": 20.0}


def shape_weights(tensors: Dict[str, torch.Tensor], cfg: Dict = None, steady: bool = False, gains: Dict = None) -> Dict[str, torch.Tensor]:
    """The drawn tensors times their gains.  `steady`: the routers' choices rest on no close call, whatever the
    precision of the run.  The last columns of the stream, one an expert, are set apart: no mixer and no feed-forward
    writes there (the rows of their last matrices and biases that would are zero), so they hold what the token's
    embedding put there, half a permutation of 1 .. experts drawn for the token, and the router's row e reads column e
    of them alone.  A token's scores then differ by a margin that rounding to eight bits does not close."""
    out = {}
    table = dict(GAINS, **(gains or {}))
    for n, t in tensors.items():
        f = next((v for k, v in table.items() if n.endswith(k)), 1.0)
        out[n] = (t.float() * f).to(t.dtype)
    if steady:
        most = max([L["mlp"]["router"]["experts"] for L in cfg["layers"] if L.get("mlp") and L["mlp"]["kind"] == "moe"] or [0])
        width = cfg["width"]
        g = torch.Generator().manual_seed(width + most)
        for n, t in out.items():
            x = t.float()
            if n == "embed":
                for tok in range(x.shape[0]):
                    x[tok, width - most:] = 0.5 * (1 + torch.randperm(most, generator=g).float())
            elif n.endswith(".norm2"):
                x[width - most:] = 1.0
            elif n.endswith(".mix.o") or n.endswith(".down"):
                x[width - most:, :] = 0.0
            elif n.endswith(".down.b"):
                x[width - most:] = 0.0
            elif n.endswith(".mlp.router"):
                x.zero_()
                for e in range(x.shape[0]):
                    x[e, width - most + e] = 4.0
            out[n] = x.to(t.dtype)
    return out


def make_ludazen_folder(tmp_path, name: str, cfg: Dict = None, seed: int = None, steady: bool = False, gains: Dict = None) -> str:
    """Write a model folder for configuration `name` (or `cfg`) with shaped random weights (`gains` replaces entries
    of `GAINS`)."""
    from braidinfer_b200.weights import open_model_folder, save_file, write_random_model
    cfg = dict(cfg if cfg is not None else LD_CONFIGS[name])
    seed = LD_SEEDS.get(name, 1) if seed is None else seed
    folder = os.path.join(str(tmp_path), f"ludazen_{name}" + ("_steady" if steady else ""))
    write_random_model(cfg, folder, seed)
    tensors = {n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    save_file(shape_weights(tensors, cfg, steady, gains), os.path.join(folder, "model.safetensors"))
    return folder


def random_config(seed: int) -> Dict:
    """A configuration drawn from a seed: sizes, head counts, the order and number of layers, windows, kept tokens,
    who reads whose latent and the constants all vary, within what a test can afford."""
    import random
    r = random.Random(seed)

    def divisor(n):
        return r.choice([d for d in range(1, n + 1) if n % d == 0])

    layers, owners = [], []
    for i in range(r.randint(2, 6)):
        u = r.random()
        mlp = None if u < 0.15 else (_dense(r.choice([24, 40, 72, 100])) if u < 0.55 else None)
        if u >= 0.55:
            experts = r.randint(1, 9)
            mlp = _moe(r.choice([8, 16, 24, 40]), experts, r.randint(1, experts), r.choice([None, 8, 24, 48]))
        v = r.random()
        if v < 0.45:
            heads = r.choice([1, 2, 3, 4, 6, 8])
            dim = r.choice([8, 16, 24, 32, 40, 64, 80, 128])
            rot = r.choice([d for d in (0, 2, 8, 16, 24, 32, 64, 128) if d <= dim] + [dim])
            scaling = (r.choice([2.0, 4.0, 16.0]), r.choice([16, 64, 512]), r.choice([8.0, 32.0]), r.choice([1.0, 2.0])) \
                if rot and r.random() < 0.6 else None
            layers.append({"type": "attention", "mlp": mlp,
                           "mixer": _att(heads, divisor(heads), dim, r.choice([dim, dim, 8, 24, 64, 72]), r.choice([dim ** -0.5, 0.2, 0.07]),
                                         rot, r.choice([100.0, 10000.0, 500000.0]), r.choice([1, 2, 5, 31, 64, 65, 100, 400]),
                                         r.choice([None, 0, 1, 4, 70]), scaling)})
        elif v < 0.75 or not owners:
            rot, rank = r.choice([2, 8, 16, 32]), r.choice([8, 16, 24, 48, 64])
            owners.append(i)
            layers.append({"type": "latent_attention", "mlp": mlp,
                           "mixer": _lat(r.randint(1, 5), r.choice([4, 8, 16, 24, 40]), rot, r.choice([4, 8, 12, 24, 36]), rank,
                                         r.choice([0.3, 0.15, 0.08]), r.choice([100.0, 10000.0]), r.choice([1, 3, 30, 64, 129, 500]))})
        else:
            j = r.choice(owners)
            o = layers[j]["mixer"]
            layers.append({"type": "latent_attention", "mlp": mlp,
                           "mixer": _lat(r.randint(1, 5), r.choice([4, 8, 16, 24, 40]), o["rot_dim"], r.choice([4, 8, 12, 24, 36]),
                                         o["kv_rank"], r.choice([0.3, 0.15, 0.08]), o["rot"]["base"],
                                         r.choice([1, 3, 30, 64, 129, 500]), kv_from=j)})
    return {"architecture": "Ludazen", "vocab": r.randint(90, 400), "width": r.choice([40, 48, 64, 72, 96, 100]),
            "norm": {"eps": r.choice([1e-6, 1e-5])}, "layers": layers}


def folder_config(folder: str) -> Dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)

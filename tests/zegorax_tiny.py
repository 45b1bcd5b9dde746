"""Small Zegorax configurations for the tests - they differ from one another in every size and option - and weights of
the tests' own making: large enough that every mechanism moves the logits (biases of order one, decays between a
memory of a few tokens and one of hundreds, routers that spread their choices, subtraction weights well away from zero)."""
from __future__ import annotations

import json
import math
import os
import random
from typing import Dict, List

import torch


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def _att(heads, kv, dim, vdim, scale, diff, rot):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff, "rot": rot}}


def _lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot, window=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def _delta(heads, kv, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(mix, mlp):
    return dict(mix, mlp=mlp)


# A: all three mixers, a looped stretch of two layers run twice, three heads a key head in the attention and value heads
#    wider than the keys', a rotation over part of a map with stretching whose blend lies inside the pairs, a window
#    shorter than a page, two heads a key head in the delta layer, a layer without feed-forward, experts of which two are chosen
TINY_A = {"architecture": "Zegorax", "vocab": 211, "width": 64, "max_positions": 320, "norm": {"eps": 1e-5},
          "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [_layer(_att(6, 2, 16, 24, 0.3, 0.35, _rot(100.0, 8, (3.0, 1.0, 6.0, 48))), _dense(72)),
                     _layer(_lat(4, 16, 8, 24, 24, 40, 0.2, _rot(50.0, 8), window=5), _moe(24, 6, 2)),
                     _layer(_delta(4, 2, 16, 24, 4), None),
                     _layer(_att(2, 2, 8, 8, 0.4, 0.1, _rot(20.0, 8)), _moe(16, 4, 1)),
                     _layer(_delta(2, 2, 24, 8, 3), _dense(40))]}
# B: nothing is a multiple of 8 (the aligned products and the tensor-core attention must find their plain forms by
#    themselves), one key head for all and one head in all, a window of one position, one tap, every expert chosen, no loop,
#    a map without rotation, a latent whose rotated part turns only in part, a delta layer first
TINY_B = {"architecture": "Zegorax", "vocab": 97, "width": 52, "max_positions": 200, "norm": {"eps": 1e-6},
          "layers": [_layer(_delta(3, 1, 10, 6, 1), _moe(10, 3, 3)),
                     _layer(_att(3, 1, 10, 6, 0.3, 0.5, _rot(7.0, 0)), _dense(36)),
                     _layer(_lat(3, 10, 6, 7, 11, 13, 0.3, _rot(30.0, 2), window=1), None),
                     _layer(_att(1, 1, 6, 9, 0.4, 0.2, _rot(500.0, 6, (8.0, 0.5, 3.0, 20))), _moe(9, 5, 2)),
                     _layer(_lat(1, 6, 2, 5, 9, 7, 0.4, _rot(2.0, 2)), _dense(18))]}
# C: sizes the tensor-core kernels take (multiples of 8), sixteen heads on one latent, key maps wider than the values, a
#    window that crosses pages of 16, one layer run three times, the loop at the very start, many experts
TINY_C = {"architecture": "Zegorax", "vocab": 130, "width": 96, "max_positions": 300, "norm": {"eps": 1e-6},
          "loop": {"start": 0, "stop": 1, "times": 3},
          "layers": [_layer(_lat(16, 16, 16, 8, 32, 48, 0.18, _rot(10000.0, 16), window=40), _moe(32, 16, 4)),
                     _layer(_att(8, 2, 32, 16, 0.15, 0.45, _rot(10000.0, 32, (2.0, 1.0, 8.0, 64))), _dense(64)),
                     _layer(_delta(4, 4, 32, 16, 4), _moe(16, 8, 2)),
                     _layer(_att(4, 4, 16, 16, 0.3, 0.25, _rot(800.0, 8)), None),
                     _layer(_delta(8, 2, 16, 32, 2), _dense(48))]}
# D: what a small real model looks like (width 256, maps of 64 and 128, a latent of 96 + 32, pages of 64): in bfloat16 the
#    products and the attention run on the tensor cores (not in TINY: its tests name it)
TINY_D = {"architecture": "Zegorax", "vocab": 500, "width": 256, "max_positions": 512, "norm": {"eps": 1e-5},
          "loop": {"start": 1, "stop": 2, "times": 2},
          "layers": [_layer(_att(4, 2, 64, 64, 0.12, 0.4, _rot(10000.0, 32, (8.0, 1.0, 4.0, 128))), _dense(512)),
                     _layer(_lat(4, 64, 32, 64, 128, 96, 0.1, _rot(10000.0, 32), window=100), _moe(128, 8, 2)),
                     _layer(_delta(4, 2, 64, 64, 4), _moe(64, 8, 2)),
                     _layer(_att(2, 1, 128, 128, 0.09, 0.2, _rot(500000.0, 128)), _dense(384))]}
TINY = {"A": (TINY_A, 41, 8), "B": (TINY_B, 42, 4), "C": (TINY_C, 43, 16)}      # config, weight seed, page size


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """float32 tensors for every name the model declares, drawn by the tensor's role (read off its name)."""
    from reinfer_b200.config.zegorax import ZegoraxConfig
    from reinfer_b200.models.zegorax import build_spec
    from reinfer_b200.parts.model import expected_params
    expected = expected_params(build_spec(ZegoraxConfig.from_dict(cfg)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, ps in expected.items():
        shape = tuple(ps.shape)
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        last = name.split(".")[-1]
        if name == "embed":
            t = n(0.8)
        elif name == "pos":
            t = n(0.3)
        elif last == "alpha":
            t = torch.rand(shape, generator=g) * 0.6 + 0.4
        elif "norm1" in name or name.startswith("final.norm"):
            t = n(0.1) if last == "b" else n(0.15, 1.0)
        elif last == "norm":
            t = n(0.15, 1.0)                # plain weights inside the mixers
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            t = n(0.35)
        elif last == "conv":
            t = n(0.5)
        elif last == "A_log":
            t = n(0.7, -1.0)
        elif last == "dt_bias":
            t = n(1.0, -1.0)
        elif last == "b" and len(shape) == 1:
            t = n(0.5)                      # projection and router biases
        elif last == "router":
            t = n(3.0 / math.sqrt(shape[1]))
        else:
            t = n(1.4 / math.sqrt(shape[-1]))
        out[name] = t.float()
    return out


def make_model_dir(path: str, which: str, store_dtype=torch.float32, cfg=None, seed=None) -> str:
    from reinfer_b200.weights.safetensors_io import write_safetensors
    base, s, _ = TINY[which] if which in TINY else (cfg, seed, None)
    cfg = cfg or base
    seed = s if seed is None else seed
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.to(store_dtype) for k, v in make_weights(cfg, seed).items()})
    return path


def sequences(which: str, lengths=None, seed=7) -> Dict[str, List[int]]:
    cfg = TINY[which][0]
    rnd = random.Random(seed)
    lengths = lengths or {"A": [5, 17, 33, 70, 40, 26, 51], "B": [1, 9, 24, 50, 90, 37, 64, 12], "C": [3, 44, 21, 60, 30]}[which]
    return {f"r{i}": [rnd.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: three to six layers in any order, head counts and sizes (also ones the tensor-core
    kernels pad or refuse), rotations over all, part or nothing of a map with and without stretching, windows from one
    position to beyond the requests, one to five taps, dense feed-forwards, mixtures or none, and a loop over any stretch."""
    rnd = random.Random(seed)
    width = rnd.choice([48, 64, 128, 192])
    layers = []
    for _ in range(rnd.randint(3, 6)):
        base = rnd.choice([10.0, 1000.0, 10000.0, 1000000.0])
        kind = rnd.choice(["attention", "latent_attention", "delta"])
        if kind == "attention":
            kv = rnd.choice([1, 2, 4])
            dim = rnd.choice([8, 12, 16, 32, 64])
            dims = rnd.choice([dim, dim // 2 // 2 * 2, 2, 0])
            scaling = (rnd.choice([2.0, 4.0, 8.0]), rnd.choice([0.5, 1.0]), rnd.choice([2.0, 4.0, 16.0]), rnd.choice([16, 64, 512])) \
                if rnd.random() < 0.7 else None
            mix = _att(kv * rnd.choice([1, 2, 3]), kv, dim, rnd.choice([8, 16, 20, 64, dim]), rnd.choice([dim ** -0.5, 0.2]),
                       rnd.choice([0.1, 0.3, 0.8]), _rot(base, dims, scaling))
        elif kind == "latent_attention":
            dim, rot_dim = rnd.choice([8, 12, 16, 32, 64]), rnd.choice([2, 8, 16, 32])
            dims = rnd.choice([rot_dim, rot_dim, max(2, rot_dim // 2 // 2 * 2)])
            mix = _lat(rnd.choice([1, 2, 4, 6, 16]), dim, rot_dim, rnd.choice([8, 16, 20, 48]), rnd.choice([12, 32, 96]),
                       rnd.choice([16, 24, 56, 64, 96]), rnd.choice([(dim + rot_dim) ** -0.5, 0.15]), _rot(base, dims),
                       window=rnd.choice([None, 1, 7, 16, 33, 64, 100, 500]))
        else:
            kv = rnd.choice([1, 2, 4])
            mix = _delta(kv * rnd.choice([1, 2]), kv, rnd.choice([8, 12, 16, 32, 64]), rnd.choice([8, 16, 20, 32, 64]), rnd.randint(1, 5))
        r = rnd.random()
        experts = rnd.choice([2, 4, 8, 16])
        mlp = None if r < 0.15 else _dense(rnd.choice([40, 64, 96])) if r < 0.5 else _moe(rnd.choice([8, 24, 32]), experts, rnd.randint(1, min(experts, 4)))
        layers.append(_layer(mix, mlp))
    cfg = {"architecture": "Zegorax", "vocab": rnd.choice([97, 300, 500]), "width": width, "max_positions": 256,
           "norm": {"eps": rnd.choice([1e-5, 1e-6])}, "layers": layers}
    if rnd.random() < 0.8:
        a = rnd.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": a, "stop": rnd.randint(a, len(layers)), "times": rnd.randint(1, 3)}
    return cfg

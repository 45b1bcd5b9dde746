"""Small Molitar configurations for the tests - they differ from one another in every size and option - and weights of
the tests' own making: large enough that every mechanism moves the logits (biases and sinks of order one, mixing weights
well inside (0, 1), norm offsets of a tenth)."""
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
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
                                                  "kv_rank": kv_rank, "scale": scale, "rot": rot}}


def _att(heads, kv, dim, vdim, scale, rot, softcap=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot, "v_mix": v_mix}
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _layer(mix, mlp):
    return dict(mix, mlp=mlp)


# A: grouped heads with value heads wider than the keys', a rotation over part of the head, a tight soft cap, three
#    value-mixing layers (the first keeps, two mix), latent layers with stretched frequencies whose ramp lies inside the
#    pairs, and one that rotates only part of its rotated width; a layer without feed-forward
TINY_A = {"architecture": "Molitar", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.7, "logit_scale": 0.8,
          "layers": [_layer(_lat(4, 16, 8, 24, 24, 40, 0.2, _rot(100.0, 8, (4.0, 16, 2.0, 0.25))), _dense(72)),
                     _layer(_att(6, 3, 16, 24, 0.3, _rot(1000.0, 8), softcap=3.0, v_mix=True), _dense(48)),
                     _layer(_lat(2, 24, 12, 16, 40, 24, 0.25, _rot(50.0, 8)), None),
                     _layer(_att(6, 3, 16, 24, 0.25, _rot(10000.0, 16), softcap=8.0, v_mix=True), _dense(40)),
                     _layer(_att(4, 4, 8, 8, 0.35, _rot(20.0, 4), v_mix=False), _dense(64)),
                     _layer(_att(3, 3, 24, 24, 0.2, _rot(300.0, 24), softcap=5.0, v_mix=True), _dense(56))]}
# B: nothing is a multiple of 8 (the aligned products and the tensor-core attention must find their plain forms by
#    themselves), one key/value head for all, only one layer says it mixes values (so it only keeps), no stretching, multiplier
#    and logit scale of 1, an attention layer first
TINY_B = {"architecture": "Molitar", "vocab": 97, "width": 52, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "logit_scale": 1.0,
          "layers": [_layer(_att(2, 1, 10, 6, 0.3, _rot(7.0, 10), softcap=2.5, v_mix=False), _dense(36)),
                     _layer(_lat(3, 10, 6, 7, 11, 13, 0.3, _rot(30.0, 6, (8.0, 8, 3.0, 0.5))), None),
                     _layer(_att(3, 1, 12, 9, 0.28, _rot(500.0, 2), v_mix=True), _dense(20)),
                     _layer(_lat(1, 6, 2, 5, 9, 7, 0.4, _rot(2.0, 2)), _dense(18))]}
# C: sixteen query heads on one latent (a full row tile of the tensor-core kernels), sizes the tensor-core kernels take
#    (multiples of 8), key heads wider than value heads, the first attention layer does not mix while two later ones do, a
#    stretching factor whose ramp covers every pair, pages of 16
TINY_C = {"architecture": "Molitar", "vocab": 130, "width": 96, "norm": {"eps": 1e-6}, "residual_mult": 0.4, "logit_scale": 2.0,
          "layers": [_layer(_lat(16, 16, 16, 8, 32, 48, 0.18, _rot(10000.0, 16, (2.0, 64, 1000.0, 0.001))), _dense(128)),
                     _layer(_att(8, 1, 32, 16, 0.2, _rot(10000.0, 32), softcap=10.0, v_mix=False), _dense(64)),
                     _layer(_att(8, 2, 32, 16, 0.15, _rot(5000.0, 16), softcap=4.0, v_mix=True), None),
                     _layer(_lat(8, 24, 8, 16, 48, 24, 0.2, _rot(100.0, 8)), _dense(64)),
                     _layer(_att(4, 2, 16, 16, 0.3, _rot(800.0, 8), v_mix=True), _dense(32))]}
# D: what a small real model looks like (width 256, heads of 128 and 64, a latent of 96 + 32, pages of 64): in bfloat16 the
#    products and the attention run on the tensor cores (not in TINY: its tests name it)
TINY_D = {"architecture": "Molitar", "vocab": 500, "width": 256, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "logit_scale": 0.25,
          "layers": [_layer(_lat(4, 64, 32, 64, 128, 96, 0.1, _rot(10000.0, 32, (4.0, 128, 16.0, 1.0))), _dense(512)),
                     _layer(_att(4, 2, 128, 64, 0.09, _rot(10000.0, 64), softcap=15.0, v_mix=True), _dense(384)),
                     _layer(_lat(8, 32, 16, 32, 64, 48, 0.15, _rot(1000.0, 16)), _dense(256)),
                     _layer(_att(4, 2, 64, 64, 0.12, _rot(10000.0, 64), softcap=30.0, v_mix=True), _dense(256))]}
TINY = {"A": (TINY_A, 41, 8), "B": (TINY_B, 42, 4), "C": (TINY_C, 43, 16)}      # config, weight seed, page size


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """float32 tensors for every name the model declares, drawn by the tensor's role (read off its name)."""
    from reinfer_b200.config.molitar import MolitarConfig
    from reinfer_b200.models.molitar import build_spec
    from reinfer_b200.parts.model import expected_params
    expected = expected_params(build_spec(MolitarConfig.from_dict(cfg)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, ps in expected.items():
        shape = tuple(ps.shape)
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        last = name.split(".")[-1]
        if name == "embed":
            t = n(0.8)
        elif last == "b":
            t = n(0.5)                      # projection biases
        elif last == "sink":
            t = n(1.5, 0.5)
        elif last == "vmix":
            t = torch.rand(shape, generator=g) * 0.6 + 0.2
        elif name.endswith("dq.norm") or name.endswith("dkv.norm"):
            t = n(0.15, 1.0)                # plain weights
        elif len(shape) == 1:
            t = n(0.1)                      # the layers' norms: stored around zero
        else:
            t = n(1.4 / math.sqrt(shape[1]))
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
    """A configuration drawn from a seed: three to six layers in any order, head counts and head sizes (also ones the
    tensor-core kernels pad or refuse), rotations over all or part of a head with and without stretching, soft caps or
    none, value mixing on any subset of the attention layers (their value sizes then agree), feed-forwards or none."""
    rnd = random.Random(seed)
    width = rnd.choice([48, 64, 128, 192])
    mix_kv, mix_vdim = rnd.choice([1, 2, 4]), rnd.choice([8, 16, 20, 64])
    layers = []
    for _ in range(rnd.randint(3, 6)):
        base = rnd.choice([10.0, 1000.0, 10000.0, 500000.0])
        if rnd.random() < 0.5:
            dim, rot_dim = rnd.choice([8, 12, 16, 32, 64]), rnd.choice([2, 8, 16, 32])
            dims = rnd.choice([rot_dim, rot_dim, max(2, rot_dim // 2)])
            scaling = (rnd.choice([2.0, 4.0, 40.0]), rnd.choice([16, 64, 2048]), rnd.choice([2.0, 32.0]), rnd.choice([0.5, 1.0])) \
                if rnd.random() < 0.7 else None
            mix = _lat(rnd.choice([1, 2, 4, 8, 16]), dim, rot_dim, rnd.choice([8, 16, 20, 64]), rnd.choice([12, 32, 96]),
                       rnd.choice([16, 24, 56, 64, 96]), rnd.choice([(dim + rot_dim) ** -0.5, 0.15]), _rot(base, dims, scaling))
        else:
            v_mix = rnd.random() < 0.6
            kv = mix_kv if v_mix else rnd.choice([1, 2, 4])
            dim = rnd.choice([8, 12, 16, 32, 48, 64, 128])
            vdim = mix_vdim if v_mix else rnd.choice([8, 16, 20, 64, 128, dim])
            dims = rnd.choice([dim, dim // 2 // 2 * 2, 2])
            mix = _att(kv * rnd.choice([1, 2, 3]), kv, dim, vdim, rnd.choice([dim ** -0.5, 0.2]), _rot(base, dims),
                       softcap=rnd.choice([None, 3.0, 20.0, 50.0]), v_mix=v_mix)
        layers.append(_layer(mix, None if rnd.random() < 0.15 else _dense(rnd.choice([40, 64, 96]))))
    return {"architecture": "Molitar", "vocab": rnd.choice([97, 300, 500]), "width": width, "norm": {"eps": rnd.choice([1e-5, 1e-6])},
            "residual_mult": rnd.choice([0.3, 0.6, 1.0]), "logit_scale": rnd.choice([0.5, 1.0, 1.7]), "layers": layers}

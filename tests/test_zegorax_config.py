"""Zegorax on the host: the configuration's parsing and its errors, the run order of a looped stretch, the model
description's tensor names and cache needs, the plain implementation's small pieces."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_zegorax as plain
import zegorax_tiny as zt
from reinfer_b200.config.errors import InvalidValue, MissingKey
from reinfer_b200.config.registry import resolve_architecture
from reinfer_b200.config.zegorax import ZegoraxConfig
from reinfer_b200.models.zegorax import build_spec
from reinfer_b200.parts.model import Model, expected_params


@pytest.mark.parametrize("cfg", [zt.TINY_A, zt.TINY_B, zt.TINY_C, zt.TINY_D] + [zt.random_config(s) for s in range(6)])
def test_round_trip_and_registry(cfg):
    arch = resolve_architecture(cfg)
    assert arch.name == "Zegorax" and arch.config_cls is ZegoraxConfig
    c = ZegoraxConfig.from_dict(cfg)
    assert ZegoraxConfig.from_dict(c.to_dict()) == c
    assert c.vocab_size == cfg["vocab"] and c.hidden_size == cfg["width"]
    assert list(c.run_order()) == plain.run_order(cfg)


def test_run_order_of_a_looped_stretch():
    c = ZegoraxConfig.from_dict(zt.TINY_A)
    assert c.run_order() == (0, 1, 2, 1, 2, 3, 4)
    m = Model(build_spec(c))
    assert [k for _, k in m.run] == ["l0", "l1", "l2", "l1#1", "l2#1", "l3", "l4"]
    d = copy.deepcopy(zt.TINY_A)
    d["loop"] = {"start": 2, "stop": 2, "times": 4}                 # an empty stretch
    assert ZegoraxConfig.from_dict(d).run_order() == (0, 1, 2, 3, 4)
    d["loop"] = {"start": 0, "stop": 5, "times": 1}
    assert ZegoraxConfig.from_dict(d).run_order() == (0, 1, 2, 3, 4)
    del d["loop"]
    assert ZegoraxConfig.from_dict(d).run_order() == (0, 1, 2, 3, 4)


@pytest.mark.parametrize("edit,error", [
    (lambda d: d.pop("vocab"), MissingKey),
    (lambda d: d.pop("max_positions"), MissingKey),
    (lambda d: d["layers"][0].__setitem__("type", "conv"), InvalidValue),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 4), InvalidValue),          # 6 heads over 4
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 18), InvalidValue),       # beyond the map
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 3), InvalidValue),
    (lambda d: d["layers"][0]["mixer"].pop("diff"), MissingKey),
    (lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), MissingKey),
    (lambda d: d["layers"][1]["mixer"]["mask"].__setitem__("size", 0), InvalidValue),
    (lambda d: d["layers"][1]["mlp"]["router"].__setitem__("top", 7), InvalidValue),
    (lambda d: d["layers"][1]["mlp"].__setitem__("kind", "sparse"), InvalidValue),
    (lambda d: d["layers"][2]["mixer"].pop("conv"), MissingKey),
    (lambda d: d["loop"].__setitem__("stop", 9), InvalidValue),
    (lambda d: d["loop"].__setitem__("times", 0), InvalidValue),
])
def test_errors_say_what_is_wrong(edit, error):
    d = copy.deepcopy(zt.TINY_A)
    edit(d)
    with pytest.raises(error):
        ZegoraxConfig.from_dict(d)


def test_tensor_names_and_shapes():
    ps = expected_params(build_spec(ZegoraxConfig.from_dict(zt.TINY_A)))
    assert tuple(ps["embed"].shape) == (211, 64) and tuple(ps["pos"].shape) == (320, 64)
    assert tuple(ps["l0.norm1.alpha"].shape) == () and tuple(ps["final.norm.b"].shape) == (64,)
    assert tuple(ps["l0.mix.q"].shape) == (6 * 2 * 16, 64) and tuple(ps["l0.mix.k"].shape) == (2 * 2 * 16, 64)
    assert tuple(ps["l0.mix.v"].shape) == (2 * 24, 64) and tuple(ps["l0.mix.g"].shape) == (6, 64) and tuple(ps["l0.mix.lk2"].shape) == (16,)
    assert tuple(ps["l0.mlp.gate.b"].shape) == (72,) and tuple(ps["l0.mlp.down.b"].shape) == (64,)
    assert tuple(ps["l1.mix.dkv"].shape) == (40 + 8, 64) and tuple(ps["l1.mix.uq"].shape) == (4 * 24, 24) and tuple(ps["l1.mix.g"].shape) == (4 * 24, 64)
    assert tuple(ps["l1.mlp.router"].shape) == (6, 64) and tuple(ps["l1.mlp.router.b"].shape) == (6,) and tuple(ps["l1.mlp.e5.gate"].shape) == (24, 64)
    assert tuple(ps["l2.mix.q.conv"].shape) == (2 * 16, 4) and tuple(ps["l2.mix.v.conv"].shape) == (4 * 24, 4)
    assert tuple(ps["l2.mix.a"].shape) == (4, 64) and tuple(ps["l2.mix.dt_bias"].shape) == (4,) and tuple(ps["l2.mix.norm"].shape) == (24,)
    assert not any(n.startswith("l2.mlp") for n in ps)              # a layer without feed-forward declares none


def test_stretched_frequencies():
    """Short waves stay, long waves are divided by the factor, and between the two the blend is linear in 1 / wavelength."""
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    f0 = plain.stretched_frequencies(16, 100.0, None)
    f1 = plain.stretched_frequencies(16, 100.0, sc)
    for a, b in zip(f0, f1):
        wave = 2 * math.pi / a
        if wave < 16:
            assert b == a
        elif wave > 64:
            assert b == a / 4
        else:
            assert a / 4 < b < a
    from reinfer_b200.parts.rope import RotaryEncoding
    got = RotaryEncoding(24, 100.0, 16, sc).table().double()
    assert torch.allclose(got, torch.tensor(f1, dtype=torch.float64), rtol=1e-6)
    assert any(a != b for a, b in zip(f0, f1)) and any(a / 4 < b < a for a, b in zip(f0, f1))


def test_plain_pieces():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 3, 8, generator=g, dtype=torch.float64)
    pos = torch.arange(5)
    fr = [0.5, 0.1]
    a = plain.rotate_half_split(x, pos, fr)
    b = plain.rotate_neighbours(x, pos, fr)
    assert torch.equal(a[0], x[0]) and torch.equal(b[0], x[0])      # position 0 turns nothing
    assert torch.equal(a[..., 4:], x[..., 4:]) and torch.equal(b[..., 4:], x[..., 4:])
    assert torch.allclose(a.norm(dim=-1), x.norm(dim=-1)) and torch.allclose(b.norm(dim=-1), x.norm(dim=-1))
    assert torch.allclose(a[2, 1, 0], x[2, 1, 0] * math.cos(1.0) - x[2, 1, 2] * math.sin(1.0))
    assert torch.allclose(b[2, 1, 0], x[2, 1, 0] * math.cos(1.0) - x[2, 1, 1] * math.sin(1.0))
    u = torch.randn(6, 2, generator=g, dtype=torch.float64)
    taps = torch.randn(2, 3, generator=g, dtype=torch.float64)
    y = plain.short_convolution(u, taps)
    assert torch.allclose(y[0], taps[:, 2] * u[0]) and torch.allclose(y[2], taps[:, 2] * u[2] + taps[:, 1] * u[1] + taps[:, 0] * u[0])
    idx, wt = plain.route(torch.eye(4, dtype=torch.float64), {"router": torch.eye(4, dtype=torch.float64) * 3, "router.b": torch.zeros(4, dtype=torch.float64)}, "", 2)
    assert idx[:, 0].tolist() == [0, 1, 2, 3] and torch.allclose(wt.sum(-1), torch.ones(4, dtype=torch.float64))

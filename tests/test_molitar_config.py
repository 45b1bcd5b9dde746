"""Host-side tests of the Molitar architecture: configuration parsing and its errors, the model description's
tensor names and shapes, which tensors a layer may leave unread, the cache layout (one keys-only row a token for a
latent layer), the stretched frequency table against the plain statement, and the plain statement against itself
(per-head keys and values rebuilt from the latent give what the absorbed form gives)."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import molitar_tiny as mt
import plain_molitar as plain
from reinfer_b200.config.errors import InvalidValue, MissingKey
from reinfer_b200.config.molitar import MolitarConfig
from reinfer_b200.config.registry import resolve_architecture


def test_round_trip_and_registry():
    for cfg in (mt.TINY_A, mt.TINY_B, mt.TINY_C, mt.TINY_D) + tuple(mt.random_config(s) for s in range(20)):
        c = MolitarConfig.from_dict(cfg)
        assert MolitarConfig.from_dict(c.to_dict()) == c
        assert resolve_architecture(c.to_dict()).config_cls is MolitarConfig
        assert c.vocab_size == cfg["vocab"] and c.hidden_size == cfg["width"]
        assert c.residual_mult == cfg["residual_mult"] and c.logit_scale == cfg["logit_scale"] and c.norm_eps == cfg["norm"]["eps"]
        assert [l.type for l in c.layers] == [l["type"] for l in cfg["layers"]]


def test_options_that_may_be_left_out():
    raw = copy.deepcopy(mt.TINY_B)
    m = raw["layers"][0]["mixer"]
    for key in ("kv_heads", "softcap", "v_mix"):
        m.pop(key, None)
    raw.pop("logit_scale")
    c = MolitarConfig.from_dict(raw)
    assert c.layers[0].mixer["kv_heads"] == c.layers[0].mixer["heads"] and c.layers[0].mixer["softcap"] is None
    assert c.layers[0].mixer["v_mix"] is False and c.logit_scale == 1.0
    assert c.layers[1].mixer["rot"]["scaling"]["factor"] == 8.0 and c.layers[3].mixer["rot"]["scaling"] is None


@pytest.mark.parametrize("change, error", [
    (lambda c: c.pop("residual_mult"), MissingKey),
    (lambda c: c.pop("norm"), MissingKey),
    (lambda c: c.pop("vocab"), MissingKey),
    (lambda c: c.update(layers=[]), MissingKey),
    (lambda c: c["layers"][0].update(type="latent"), InvalidValue),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), MissingKey),
    (lambda c: c["layers"][0]["mixer"].pop("rot"), MissingKey),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), InvalidValue),        # more than the rotated part holds
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), InvalidValue),         # pairs
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), MissingKey),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.0), InvalidValue),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), InvalidValue),            # 6 heads over 4
    (lambda c: c["layers"][1]["mixer"].update(softcap=-1.0), InvalidValue),
    (lambda c: c["layers"][1]["mixer"].update(v_mix="yes"), InvalidValue),
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), InvalidValue),               # mixes in values of another size
    (lambda c: c["layers"][1]["mixer"].update(scale=float("nan")), InvalidValue),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), InvalidValue),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), MissingKey),
])
def test_refusals(change, error):
    raw = copy.deepcopy(mt.TINY_A)
    change(raw)
    with pytest.raises(error):
        MolitarConfig.from_dict(raw)


def test_tensor_names_and_shapes():
    from reinfer_b200.models.molitar import build_spec
    from reinfer_b200.parts.model import expected_params
    spec = build_spec(MolitarConfig.from_dict(mt.TINY_A))
    exp = expected_params(spec)
    assert tuple(exp["embed"].shape) == (211, 64) and tuple(exp["final.norm"].shape) == (64,) and "head" not in exp
    # a latent layer: 4 heads of 16 + 8, values of 24, bottlenecks of 24 and 40
    assert tuple(exp["l0.mix.dq"].shape) == (24, 64) and tuple(exp["l0.mix.dq.norm"].shape) == (24,)
    assert tuple(exp["l0.mix.uq"].shape) == (4 * 24, 24) and tuple(exp["l0.mix.dkv"].shape) == (40 + 8, 64)
    assert tuple(exp["l0.mix.dkv.norm"].shape) == (40,) and tuple(exp["l0.mix.uk"].shape) == (4 * 16, 40)
    assert tuple(exp["l0.mix.uv"].shape) == (4 * 24, 40) and tuple(exp["l0.mix.o"].shape) == (64, 4 * 24)
    # a gated layer: 6 heads over 3, keys of 16, values of 24
    assert tuple(exp["l1.mix.q"].shape) == (96, 64) and tuple(exp["l1.mix.q.b"].shape) == (96,)
    assert tuple(exp["l1.mix.k"].shape) == (48, 64) and tuple(exp["l1.mix.k.b"].shape) == (48,)
    assert tuple(exp["l1.mix.v"].shape) == (72, 64) and tuple(exp["l1.mix.v.b"].shape) == (72,)
    assert tuple(exp["l1.mix.sink"].shape) == (6,) and tuple(exp["l1.mix.vmix"].shape) == ()
    assert tuple(exp["l1.mix.g"].shape) == (6 * 24, 64) and tuple(exp["l1.mix.o"].shape) == (64, 6 * 24)
    assert tuple(exp["l1.mlp.gate"].shape) == (48, 64) and tuple(exp["l1.mlp.down"].shape) == (64, 48)
    for n in ("norm1", "norm1b", "norm2", "norm2b"):
        assert tuple(exp[f"l1.{n}"].shape) == (64,)
    # a layer without feed-forward declares neither its matrices nor its norms, but a checkpoint may hold the norms
    assert not any(k.startswith("l2.mlp.") for k in exp) and "l2.norm2" not in exp
    assert {"l2.norm2", "l2.norm2b"} <= set(spec.ignorable_tensors)
    # a gated layer that mixes nothing reads no mixing weight
    assert "l4.mix.vmix" not in exp and "l4.mix.vmix" in spec.ignorable_tensors


def test_who_keeps_and_who_mixes():
    from reinfer_b200.models.molitar import build_spec
    for cfg, want in ((mt.TINY_A, {1: "first", 3: "mix", 4: None, 5: "mix"}), (mt.TINY_B, {0: None, 2: "first"}),
                      (mt.TINY_C, {1: None, 2: "first", 4: "mix"})):
        c = MolitarConfig.from_dict(cfg)
        spec = build_spec(c)
        got = {i: l.parts["mixer"][1].params["v_mix"] for i, l in enumerate(spec.layers) if c.layers[i].type == "attention"}
        assert got == want


def test_cache_layout():
    from reinfer_b200.cache.manager import group_layers
    from reinfer_b200.models.molitar import build_spec
    from reinfer_b200.parts.model import Model
    m = Model(build_spec(MolitarConfig.from_dict(mt.TINY_A)))
    paged, states = m.cache_layout()
    assert set(paged) == {f"l{i}" for i in range(6)} and not states
    assert (paged["l0"].kv_heads, paged["l0"].head_dim, paged["l0"].value_dim) == (1, 48, 0)       # [latent | rotated key], no value rows
    assert (paged["l2"].kv_heads, paged["l2"].head_dim, paged["l2"].value_dim) == (1, 36, 0)
    assert (paged["l1"].kv_heads, paged["l1"].head_dim, paged["l1"].value_dim) == (3, 16, 24)
    assert all(p.window is None and p.chunk is None for p in paged.values())
    assert len(group_layers(paged)) >= 1


@pytest.mark.parametrize("seed", range(6))
def test_stretched_frequencies(seed):
    import random
    from reinfer_b200.parts.rope import PairRotary
    rnd = random.Random(seed)
    rot = {"base": rnd.choice([10.0, 1e4, 2.5e5]), "dims": rnd.choice([2, 8, 32, 64]),
           "scaling": {"factor": rnd.choice([2.0, 8.0, 40.0]), "original": rnd.choice([16, 2048, 4096]), "fast": rnd.choice([2.0, 32.0]),
                       "slow": rnd.choice([0.25, 1.0])}}
    enc = PairRotary(rot["dims"], rot["base"], rot["scaling"])
    f, mag = plain.rotary_frequencies(rot)
    assert (enc.table().double() - f).abs().max() <= 1e-7 * f.abs().max()
    assert enc.magnitude == pytest.approx(0.1 * math.log(rot["scaling"]["factor"]) + 1.0) and mag == pytest.approx(enc.magnitude)


def test_latent_keys_can_stay_in_the_latent():
    """The plain statement rebuilds every head's keys and values from the latent; the engine keeps the latent and moves
    the per-head maps to the query and to the output.  Both are the same sums (float64)."""
    g = torch.Generator().manual_seed(3)
    T, H, dn, dr, dv, r, scale = 12, 3, 10, 4, 6, 7, 0.3
    q = torch.randn(T, H, dn + dr, generator=g, dtype=torch.float64)
    c = torch.randn(T, r, generator=g, dtype=torch.float64)
    kr = torch.randn(T, dr, generator=g, dtype=torch.float64)
    uk = torch.randn(H * dn, r, generator=g, dtype=torch.float64)
    uv = torch.randn(H * dv, r, generator=g, dtype=torch.float64)
    k = plain.lin(c, uk).view(T, H, dn)
    v = plain.lin(c, uv).view(T, H, dv)
    for h in range(H):
        rebuilt = plain.causal_softmax_head(q[:, h], torch.cat([k[:, h], kr], -1), v[:, h], scale)
        q_abs = torch.cat([q[:, h, :dn] @ uk[h * dn:(h + 1) * dn], q[:, h, dn:]], -1)             # [T, r + dr]
        latent = plain.causal_softmax_head(q_abs, torch.cat([c, kr], -1), c, scale)                 # values: the latent itself
        assert (plain.lin(latent, uv[h * dv:(h + 1) * dv]) - rebuilt).abs().max() < 1e-12

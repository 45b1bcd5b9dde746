"""Zegorax's mechanisms one at a time.  The kernels that came with the design against the formulas of
tests/plain_zegorax.py on inputs of the tests' own making, and one-layer models (one mixer, one kind of feed-forward)
through the engine with weights made so that a fault shows: a softmax so sharp that one far key carries a row, windows
whose edge falls before, on and behind a page border, a memory that decays over hundreds of tokens."""
from __future__ import annotations

import math
import random

import pytest
import torch

import plain_zegorax as plain
import tiny
import zegorax_tiny as zt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _close(got, want, tol, what=""):
    err = (got.double().cpu() - want.double()).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err <= tol, f"{what}: {err:.3e} of the scale (limit {tol})"


# ---------------------------------------------------------------- kernels
@pytest.mark.parametrize("dims,dk,dv,QH,KH", [(8, 16, 24, 6, 2), (0, 10, 6, 3, 1), (12, 12, 8, 2, 2), (32, 32, 16, 16, 4)])
def test_half_split_rotation_and_store(dims, dk, dv, QH, KH):
    """q and k heads turned in pairs (i, i + dims/2) with stretched frequencies, the rest of a head passing; q to its
    tensor, k and v into the token's cache slot."""
    from reinfer_b200 import ops
    from reinfer_b200.parts.rope import RotaryEncoding
    g = torch.Generator().manual_seed(dims + dk)
    T, page, pages = 9, 4, 5
    x = torch.randn(T, (QH + KH) * dk + KH * dv + 3, generator=g)
    pos = torch.tensor([0, 1, 2, 3, 50, 51, 7, 300, 1000], dtype=torch.int32)
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    enc = RotaryEncoding(dk, 1000.0, dims, sc) if dims else None
    freq = None
    if enc is not None:
        enc.prepare(DEV)
        freq = enc.inv_freq
    fr = plain.stretched_frequencies(dims, 1000.0, sc)
    if dims:
        _close(freq, torch.tensor(fr), 1e-6, "frequencies")
    slots = torch.tensor([3, 0, 19, 7, 8, 9, 12, 1, 16], dtype=torch.int32)
    q = torch.empty(T, QH, dk, device=DEV)
    cache = torch.zeros(pages, KH * page * (dk + dv), device=DEV)
    ops.rotary_heads_append(x.to(DEV), None, pos.to(DEV), freq, dims, 1.0, slots.to(DEV), q, cache, QH, KH, dk, dv, page, half_split=True)
    xd = x.double()
    wq = plain.rotate_half_split(xd[:, :QH * dk].view(T, QH, dk), pos, fr)
    wk = plain.rotate_half_split(xd[:, QH * dk:(QH + KH) * dk].view(T, KH, dk), pos, fr)
    wv = xd[:, (QH + KH) * dk:(QH + KH) * dk + KH * dv].view(T, KH, dv)
    _close(q, wq, 2e-5, "queries")
    c = cache.cpu()
    for t in range(T):
        p, o = divmod(int(slots[t]), page)
        keys = c[p, :KH * page * dk].view(KH, page, dk)[:, o]
        vals = c[p, KH * page * dk:].view(KH, page, dv)[:, o]
        _close(keys, wk[t], 2e-5, "keys")
        _close(vals, wv[t], 1e-6, "values")


@pytest.mark.parametrize("H,G,dv", [(6, 2, 24), (1, 1, 9), (8, 8, 64), (4, 1, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_differential_output_stage(H, G, dv, dtype):
    from reinfer_b200 import ops
    g = torch.Generator().manual_seed(H * dv)
    T, R = 7, H // G
    a = torch.randn(T, G, 2, R, dv, generator=g).to(dtype)              # [key head, map, head of the group]
    gate = torch.randn(T, H + 3, generator=g)
    lam, eps, diff = 0.62, 1e-5, 0.3
    out = torch.empty(T, H, dv, dtype=dtype, device=DEV)
    ops.diff_heads(a.to(DEV).view(T, 2 * H, dv), out, lam, eps, 1.0 - diff, H, G, dv, gate.to(DEV)[:, 1:1 + H])
    ad = a.double()
    o = (ad[:, :, 0] - lam * ad[:, :, 1]).reshape(T, H, dv)
    want = plain.rms(o, eps) * (1.0 - diff) * torch.sigmoid(gate[:, 1:1 + H].double())[:, :, None]
    _close(out.float(), want, 1e-5 if dtype == torch.float32 else 1e-2, "combined heads")


@pytest.mark.parametrize("n,top,h", [(16, 2, 64), (3, 3, 52), (5, 1, 40), (64, 6, 128)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_by_chosen_logits(n, top, h, dtype):
    """The largest logits (with their bias) are chosen and softmaxed among themselves; everything else gets zero."""
    from reinfer_b200 import ops
    g = torch.Generator().manual_seed(n + top)
    T = 37
    x = torch.randn(T, h, generator=g).to(dtype)
    w = (torch.randn(n, h, generator=g) * 0.4).to(dtype)
    b = torch.randn(n, generator=g)
    gates, ident = ops.moe_router(x.to(DEV), w.to(DEV), b.to(DEV), n, top, mode="chosen_logits")
    assert ident is None
    idx, wt = plain.route(x.double(), {"router": w.double(), "router.b": b.double()}, "", top)
    want = torch.zeros(T, n, dtype=torch.float64).scatter_(1, idx, wt)
    _close(gates, want, 1e-5, "gates")
    assert ((gates > 0).sum(1) == top).all()
    z = torch.randn(T, n, generator=g)
    gates2, _ = ops.moe_route(z.to(DEV), b.to(DEV), n, top, mode="chosen_logits")
    val, idx = torch.topk(z.double() + b.double(), top, dim=-1)
    _close(gates2, torch.zeros(T, n, dtype=torch.float64).scatter_(1, idx, torch.softmax(val, -1)), 1e-6, "gates from logits")


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_activation_with_biases_and_expert_weights(act, dtype):
    from reinfer_b200 import ops
    g = torch.Generator().manual_seed(3)
    T, E, ff = 11, 5, 12
    F = E * ff
    gu = torch.randn(T, 2 * F + 4, generator=g) * 2
    bias = torch.randn(2 * F, generator=g)
    gates = torch.rand(T, E, generator=g) * (torch.rand(T, E, generator=g) < 0.5)
    f = plain.silu if act == "silu" else plain.gelu_tanh
    gd, bd = gu[:, :2 * F].double(), bias.double()
    for with_bias, with_gates in ((True, False), (False, True), (True, True), (False, False)):
        out = torch.empty(T, F, dtype=dtype, device=DEV)
        ops.glu_act(gu.to(DEV)[:, :2 * F], out, act, bias.to(DEV) if with_bias else None, gates.to(DEV) if with_gates else None, ff)
        bb = bd if with_bias else torch.zeros_like(bd)
        want = f(gd[:, :F] + bb[:F]) * (gd[:, F:] + bb[F:])
        if with_gates:
            want = want * gates.double().repeat_interleave(ff, dim=1)
        _close(out.float(), want, 1e-5 if dtype == torch.float32 else 1e-2, f"{act} bias {with_bias} gates {with_gates}")


@pytest.mark.parametrize("T", [1, 8, 40, 100, 300, 700])
@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_gated_pair_product_with_the_activation_in_its_epilogue(T, act):
    """The tensor-core product of the gated pair at the token counts of its kernels (split over a cluster, streaming,
    persistent) with biases, either activation and a weight per token and expert: against 64-bit sums of the same
    bfloat16 operands."""
    from reinfer_b200 import ops
    g = torch.Generator().manual_seed(T)
    K, E, ff = 192, 5, 72
    F = E * ff
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    bias = torch.randn(2 * F, generator=g) * 0.5
    gates = torch.rand(T, E, generator=g) * (torch.rand(T, E, generator=g) < 0.5)
    f = plain.silu if act == "silu" else plain.gelu_tanh
    z = x.double() @ w.double().t()
    for with_bias, with_gates in ((True, False), (False, True), (True, True), (False, False)):
        out = torch.empty(T, F, dtype=torch.bfloat16, device=DEV)
        assert ops.gemm_bf16_swiglu(x.to(DEV), w.to(DEV), out, act=act, bias=bias.to(DEV) if with_bias else None,
                                    gates=gates.to(DEV) if with_gates else None, ff=ff)
        bb = bias.double() if with_bias else torch.zeros(2 * F, dtype=torch.float64)
        want = f(z[:, :F] + bb[:F]) * (z[:, F:] + bb[F:])
        if with_gates:
            want = want * gates.double().repeat_interleave(ff, dim=1)
        _close(out.float(), want, 1e-2, f"{act} bias {with_bias} gates {with_gates}")
        if with_gates:
            assert (out.float().cpu()[gates.repeat_interleave(ff, dim=1) == 0] == 0).all()


@pytest.mark.parametrize("T,E,top,h,ff", [(300, 8, 2, 64, 72), (257, 4, 1, 128, 128), (1000, 16, 4, 192, 200), (130, 6, 3, 64, 8)])
def test_experts_over_rows_sorted_by_expert(T, E, top, h, ff):
    """The grouped form of a gated mixture (only the chosen pairs are computed) against 64-bit sums over the same bfloat16
    operands, with inner widths that are no multiple of a tile (a tile of weight rows then reaches into the next
    expert's) and with experts that nobody chose."""
    from reinfer_b200 import ops
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, h, generator=g).to(torch.bfloat16)
    wg = (torch.randn(E, ff, h, generator=g) * h ** -0.5).to(torch.bfloat16)
    wu = (torch.randn(E, ff, h, generator=g) * h ** -0.5).to(torch.bfloat16)
    wd = (torch.randn(E, h, ff, generator=g) * ff ** -0.5).to(torch.bfloat16)
    z = torch.randn(T, E, generator=g)
    z[:, 1] = -50.0                                                # an expert that nobody chooses
    val, idx = torch.topk(z, top, dim=-1)
    gates = torch.zeros(T, E).scatter_(1, idx, torch.softmax(val, -1))
    want = torch.zeros(T, h, dtype=torch.float64)
    for e in range(E):
        rows = (gates[:, e] > 0).nonzero().flatten()
        if len(rows):
            xe = x[rows].double()
            inner = (plain.silu(xe @ wg[e].double().t()) * (xe @ wu[e].double().t())).to(torch.bfloat16).double()
            want[rows] += gates[rows, e:e + 1].double() * (inner @ wd[e].double().t())
    base = torch.randn(T, h, generator=g)
    w_gu = torch.cat([wg.reshape(E * ff, h), wu.reshape(E * ff, h)]).contiguous().to(DEV)
    w_down = wd.permute(1, 0, 2).reshape(h, E * ff).contiguous().to(DEV)
    for store in (False, True):
        dst = base.clone().to(DEV)
        assert ops.moe_grouped_experts(x.to(DEV), gates.to(DEV), top, w_gu, w_down, ff, "silu", dst, store=store)
        _close(dst, want if store else want + base.double(), 5e-3, f"store {store}")
    assert ops.status_word() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_per_head_maps_with_a_gate(dtype):
    from reinfer_b200 import ops
    g = torch.Generator().manual_seed(8)
    T, H, n_in, n_out = 70, 3, 24, 20
    x = torch.randn(T, H, n_in, generator=g).to(dtype)
    w = (torch.randn(H, n_out, n_in, generator=g) * 0.3).to(dtype)
    gate = torch.randn(T, H * n_out + 5, generator=g)
    y = torch.empty(T, H, n_out, dtype=dtype, device=DEV)
    ops.heads_linear(x.to(DEV), w.to(DEV), y, gate=gate.to(DEV)[:, :H * n_out])
    want = torch.einsum("thi,hoi->tho", x.double(), w.double()) * torch.sigmoid(gate[:, :H * n_out].double()).view(T, H, n_out)
    _close(y.float(), want, 1e-5 if dtype == torch.float32 else 1e-2, "gated maps")


def test_delta_rule_with_one_decay_a_head():
    """The recurrence kernel with a gate per head against the plain loop, over a request cut into steps."""
    from reinfer_b200 import ops
    g = torch.Generator().manual_seed(21)
    T, H, G, dk, dv = 45, 4, 2, 12, 10
    q, k = torch.randn(T, G * dk, generator=g), torch.randn(T, G * dk, generator=g)
    v = torch.randn(T, H * dv, generator=g)
    z, zb = torch.randn(T, H, generator=g), torch.randn(H, generator=g)
    b_pre, a_log = torch.randn(T, H, generator=g), torch.randn(H, generator=g) * 0.5 - 1.0
    state = torch.zeros(2, H, dk, dv, device=DEV)
    out = torch.empty(T, H, dv, device=DEV)
    at = 0
    for n in (1, 2, 20, 17, 5):                                   # the same request, portion by portion, in slot 1
        sl = slice(at, at + n)
        ops.recurrence("delta_gated_state", "exp_softplus", q[sl].to(DEV), k[sl].to(DEV), v[sl].to(DEV), z[sl].contiguous().to(DEV),
                       zb.to(DEV), state, out[sl], torch.tensor([0, n], dtype=torch.int32, device=DEV),
                       torch.tensor([1], dtype=torch.int32, device=DEV), 1, H, G, dk, dv, q_scale=dk ** -0.5, unit_qk=True,
                       b_pre=b_pre[sl].contiguous().to(DEV), rate=a_log.to(DEV), max_q_len=n, gate_per_head=True)
        at += n
    qd, kd = plain.unit(q.double().view(T, G, dk)) * dk ** -0.5, plain.unit(k.double().view(T, G, dk))
    vd = v.double().view(T, H, dv)
    decay = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(z.double() + zb.double()))
    beta = torch.sigmoid(b_pre.double())
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    for h in range(H):
        S = torch.zeros(dk, dv, dtype=torch.float64)
        for t in range(T):
            S = decay[t, h] * S
            S = S + torch.outer(kd[t, h // (H // G)], beta[t, h] * (vd[t, h] - S.t() @ kd[t, h // (H // G)]))
            want[t, h] = S.t() @ qd[t, h // (H // G)]
    _close(out, want, 2e-5, "read-outs")
    assert state[0].abs().max().item() == 0.0


# ---------------------------------------------------------------- one-layer models through the engine
def _one_layer(mix, mlp, width=64, vocab=101, positions=800, eps=1e-5, loop=None):
    cfg = {"architecture": "Zegorax", "vocab": vocab, "width": width, "max_positions": positions, "norm": {"eps": eps},
           "layers": [dict(mix, mlp=mlp)]}
    if loop:
        cfg["loop"] = loop
    return cfg


def _run_cuts(tmp_path, cfg, seqs, page, dtype, tol, seed=3, tail=40, sizes=(37, 2, 64, 3, 70, 5, 2, 11), edit=None):
    from reinfer_b200.engine import Engine, StepEntry
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    d = zt.make_model_dir(str(tmp_path / f"m{dtype}"), "X", store, cfg=cfg, seed=seed)
    if edit is not None:
        from reinfer_b200.weights.safetensors_io import write_safetensors
        w = {k: v.to(store) for k, v in edit(zt.make_weights(cfg, seed)).items()}
        write_safetensors(str(tmp_path / f"m{dtype}" / "model.safetensors"), w)
    raw, w = plain.read_model(d)
    want = {r: plain.forward(raw, w, t) for r, t in seqs.items()}
    for steps in (tiny.cut_whole(seqs), tiny.cut_tail_one_by_one(seqs, tail=tail), tiny.cut_portions(seqs, sizes=sizes),
                  tiny.cut_mixed(seqs, seed=seed)):
        e = Engine.from_model_dir(d, dtype=dtype, page_size=page, max_tokens=tiny.pool_tokens_needed(steps, page), max_num_seqs=4)
        done, errs = {}, []
        for entries, end in steps:
            lg = e.step([StepEntry(r, t, wnt) for r, t, wnt in entries]).double().cpu()
            row = 0
            for r, t, wnt in entries:
                for kk in wnt:
                    ref = want[r][done.get(r, 0) + kk]
                    errs.append((lg[row] - ref).abs().max().item() / ref.abs().max().item())
                    row += 1
                done[r] = done.get(r, 0) + len(t)
            for r in end:
                e.finish(r)
                done.pop(r, None)
        e.check_guards()
        e.check_status()
        assert e.cache.free_pages() == e.cache.total_pages()
        errs = torch.tensor(errs)
        if dtype == "float32":
            assert errs.max().item() <= tol, f"worst row {errs.max().item():.3e} at {int(errs.argmax())}"
        else:
            assert torch.isfinite(errs).all() and errs.median().item() <= tol / 3 and (errs <= tol).float().mean().item() >= 0.95, \
                f"median {errs.median().item():.3e}, within tolerance {(errs <= tol).float().mean().item():.3f}"


def _seqs(vocab, lengths, seed):
    rnd = random.Random(seed)
    return {f"r{i}": [rnd.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


MIXERS = {
    "attention": zt._att(6, 2, 16, 24, 0.3, 0.35, zt._rot(100.0, 8, (3.0, 1.0, 6.0, 48))),
    "attention_odd": zt._att(3, 3, 10, 6, 0.3, 0.6, zt._rot(7.0, 4)),
    "latent": zt._lat(4, 16, 8, 24, 24, 40, 0.2, zt._rot(50.0, 8), window=21),
    "latent_odd": zt._lat(3, 10, 6, 7, 11, 13, 0.3, zt._rot(30.0, 2)),
    "delta": zt._delta(4, 2, 16, 24, 4),
    "delta_odd": zt._delta(3, 1, 10, 6, 2),
}
FFS = {"none": None, "dense": zt._dense(40), "moe": zt._moe(16, 6, 2)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("ff", list(FFS))
@pytest.mark.parametrize("mixer", list(MIXERS))
def test_one_mixer_and_one_feed_forward(tmp_path, mixer, ff, dtype):
    if ff != "moe" and mixer.endswith("_odd") and dtype == "bfloat16":
        pytest.skip("covered by the other combinations")
    width = 52 if mixer.endswith("_odd") else 64
    cfg = _one_layer(MIXERS[mixer], FFS[ff], width=width)
    _run_cuts(tmp_path, cfg, _seqs(101, [1, 9, 50, 90, 37], 5), 8, dtype, 1e-4 if dtype == "float32" else 4e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "latent"])
def test_a_far_key_among_hundreds(tmp_path, kind, dtype):
    """A softmax so sharp (a scale ten times the usual) that single keys carry a row, over 600 tokens: a key that is
    lost, shifted or read from the wrong page changes rows outright.  Prompts, portions and decoded tokens."""
    mix = zt._att(4, 2, 16, 16, 2.5, 0.3, zt._rot(10000.0, 16, (4.0, 1.0, 4.0, 64))) if kind == "attention" else \
        zt._lat(4, 16, 8, 16, 24, 32, 2.0, zt._rot(10000.0, 8))
    cfg = _one_layer(mix, None)
    _run_cuts(tmp_path, cfg, _seqs(101, [600, 333], 9), 16, dtype, 2e-4 if dtype == "float32" else 6e-2, tail=48,
              sizes=(130, 2, 64, 3, 257, 5))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 2, 15, 16, 17, 33, 64])
def test_keys_just_inside_and_just_outside_the_window(tmp_path, window, dtype):
    """Windows whose edge falls before, on and behind a border of 16-token pages, with a sharp softmax: the key that just
    left the window would change the row if it were still seen, and so would the oldest one inside if it were not.  Every
    position of prompts longer than the window, in one step, in portions and decoded one by one."""
    if dtype == "bfloat16" and window not in (16, 17, 33):
        pytest.skip("32-bit covers it")
    cfg = _one_layer(zt._lat(2, 16, 8, 16, 24, 32, 1.5, zt._rot(100.0, 8), window=window), None)
    _run_cuts(tmp_path, cfg, _seqs(101, [window + 2, 3 * window + 40, 70], window), 16, dtype, 2e-4 if dtype == "float32" else 6e-2,
              tail=window + 5, sizes=(window, 2, 16, 3, window + 1, 5))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_memory_hundreds_of_tokens_old(tmp_path, dtype):
    """Decays close to one (a half-life of hundreds of tokens): what the first tokens wrote still shapes the last rows,
    so a state that is lost, reset or mixed up between requests shows; the convolution's window crosses every cut."""
    def slow(w):
        w["l0.mix.A_log"] = torch.full_like(w["l0.mix.A_log"], -5.0)
        w["l0.mix.dt_bias"] = torch.full_like(w["l0.mix.dt_bias"], -1.0)
        return w
    cfg = _one_layer(zt._delta(4, 2, 16, 16, 4), zt._dense(32))
    _run_cuts(tmp_path, cfg, _seqs(101, [500, 41, 260], 4), 16, dtype, 2e-4 if dtype == "float32" else 6e-2, tail=64,
              sizes=(3, 2, 100, 64, 5, 2, 129), edit=slow)


def test_a_looped_layer_has_a_memory_per_pass(tmp_path):
    """One layer of each kind run three times in a row: the passes share weights, never caches or states."""
    for name in ("attention", "latent", "delta"):
        cfg = _one_layer(MIXERS[name], FFS["moe"], loop={"start": 0, "stop": 1, "times": 3})
        _run_cuts(tmp_path / name, cfg, _seqs(101, [30, 75], 6), 8, "float32", 1e-4)

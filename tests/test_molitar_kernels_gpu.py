"""Each mechanism of the Molitar layers alone, on the device, against the plain statement of tests/plain_molitar.py:
the pair rotation and its stretched frequency table, the latent preparation (two norms, the shared rotated key, the
store into a keys-only page), the preparation of biased, rotated heads with value mixing, the per-head linear maps,
the attention with soft cap, sink, values inside the keys and output gate (a far key among hundreds, page borders,
prompt portions and single tokens, plain and tensor-core kernels, a batch of unequal requests), and the norms whose
weights are stored around zero."""
from __future__ import annotations

import math
from types import SimpleNamespace

import pytest
import torch

import plain_molitar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _gen(seed):
    return torch.Generator().manual_seed(seed)


ROTS = [{"base": 10000.0, "dims": 16}, {"base": 500000.0, "dims": 32, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 0.5}},
        {"base": 50.0, "dims": 8, "scaling": {"factor": 40.0, "original": 16, "fast": 2.0, "slow": 0.25}}, {"base": 7.0, "dims": 2},
        {"base": 100.0, "dims": 12, "scaling": {"factor": 2.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
        {"base": 1000.0, "dims": 24, "scaling": {"factor": 8.0, "original": 32, "fast": 1000.0, "slow": 0.001}}]


# ------------------------------------------------------------------ rotation
@pytest.mark.parametrize("rot", ROTS)
def test_frequency_table_and_magnitude(rot):
    from reinfer_b200.parts.rope import PairRotary
    enc = PairRotary(rot["dims"], rot["base"], rot.get("scaling"))
    f, mag = plain.rotary_frequencies(rot)
    assert (enc.table().double() - f).abs().max() <= 1e-7 * f.abs().max()
    assert abs(enc.magnitude - mag) < 1e-12
    if rot.get("scaling"):
        plain_f, _ = plain.rotary_frequencies({"base": rot["base"], "dims": rot["dims"]})
        assert (f <= plain_f * (1 + 1e-12)).all() and (f >= plain_f / rot["scaling"]["factor"] * (1 - 1e-12)).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rot", ROTS)
@pytest.mark.parametrize("extra", [0, 5, 8])
def test_pairs_are_rotated_and_the_rest_passes(dtype, rot, extra):
    from reinfer_b200 import ops
    from reinfer_b200.parts.rope import PairRotary
    g = _gen(rot["dims"] + extra)
    T, H, width = 9, 3, rot["dims"] + extra
    enc = PairRotary(rot["dims"], rot["base"], rot.get("scaling"))
    enc.prepare(DEV)
    positions = torch.tensor([0, 1, 2, 63, 64, 65, 500, 4097, 30000], dtype=torch.int32)
    big = torch.randn(T, H, width + 6, generator=g).to(dtype)              # heads inside a wider row: strides of their own
    src = big[:, :, 3:3 + width]
    ref = plain.rotate_pairs(src.double(), positions, rot)
    dst = torch.full((T, H, width + 2), 5.0, dtype=dtype, device=DEV)
    ops.rotate_pairs(big.to(DEV)[:, :, 3:3 + width], dst[:, :, :width], positions.to(DEV), enc.freq, rot["dims"], enc.magnitude)
    out = dst.double().cpu()
    # float32 angles of tens of thousands of radians carry an absolute error of ~1e-3 in the fastest pairs
    tol = 4e-3 if dtype == torch.float32 else 2e-2
    assert (out[:, :, :width] - ref).abs().max() <= tol * ref.abs().max()
    small = positions <= 65
    assert (out[small][:, :, :width] - ref[small]).abs().max() <= (2e-5 if dtype == torch.float32 else 1e-2) * ref.abs().max()
    assert torch.equal(out[:, :, rot["dims"]:width], src.double()[:, :, rot["dims"]:])      # the rest passes bit for bit
    assert (out[:, :, width:] == 5.0).all()
    # position 0 turns nothing, but the factor on cosine stays
    assert (out[0, :, :rot["dims"]] - src.double()[0, :, :rot["dims"]] * enc.magnitude).abs().max() <= tol * ref.abs().max()


# ------------------------------------------------------------------ latent preparation
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("na,nc,nr,rot,page", [(24, 40, 8, ROTS[2], 8), (11, 13, 6, {"base": 30.0, "dims": 6}, 4), (128, 96, 32, ROTS[1], 64),
                                               (9, 7, 2, ROTS[3], 4), (40, 24, 12, ROTS[2], 16), (1536, 512, 64, {"base": 1e4, "dims": 64}, 64)])
def test_latent_rows_are_normed_rotated_and_stored(dtype, na, nc, nr, rot, page):
    from reinfer_b200 import ops
    from reinfer_b200.parts.rope import PairRotary
    g = _gen(na + nc)
    T, eps, pages = 11, 1e-5, 7
    enc = PairRotary(rot["dims"], rot["base"], rot.get("scaling"))
    enc.prepare(DEV)
    x = torch.randn(T, na + nc + nr + 3, generator=g) * 3.0                 # float32 sums of the projection, in a wider row
    wa, wc = torch.randn(na, generator=g) * 0.2 + 1.0, torch.randn(nc, generator=g) * 0.2 + 1.0
    positions = torch.tensor([0, 1, 7, 8, 9, 63, 64, 100, 129, 2, 3], dtype=torch.int32)
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    slots[4] = -1                                                             # an inert row stores nothing
    a_ref = plain.norm_plain(x[:, :na].double(), wa.double(), eps)
    c_ref = plain.norm_plain(x[:, na:na + nc].double(), wc.double(), eps)
    r_ref = plain.rotate_pairs(x[:, na + nc:na + nc + nr].double().reshape(T, 1, nr), positions, rot)[:, 0]
    a_out = torch.empty(T, na, dtype=dtype, device=DEV)
    cache = torch.full((pages, page * (nc + nr)), 77.0, dtype=dtype, device=DEV)
    ops.latent_prep(x.to(DEV)[:, :na + nc + nr], na, nc, nr, wa.to(DEV), wc.to(DEV), eps, positions.to(DEV), enc.freq, rot["dims"],
                    enc.magnitude, slots.to(DEV), a_out, cache, page)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert (a_out.double().cpu() - a_ref).abs().max() <= tol * a_ref.abs().max()
    c = cache.double().cpu().view(pages * page, nc + nr)
    touched = torch.zeros(pages * page, dtype=torch.bool)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        touched[s] = True
        assert (c[s, :nc] - c_ref[t]).abs().max() <= tol * c_ref.abs().max()
        assert (c[s, nc:] - r_ref[t]).abs().max() <= tol * r_ref.abs().max()
    assert (c[~touched] == 77.0).all()
    # without slots only the queries' bottleneck is made
    again = torch.empty_like(a_out)
    ops.latent_prep(x.to(DEV)[:, :na + nc + nr], na, nc, nr, wa.to(DEV), wc.to(DEV), eps, positions.to(DEV), enc.freq, rot["dims"],
                    enc.magnitude, None, again, cache, page)
    assert torch.equal(again, a_out)


# ------------------------------------------------------------------ biased, rotated heads with value mixing
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("QH,KH,dk,dv,rot,page", [(6, 3, 16, 24, {"base": 1000.0, "dims": 8}, 8), (2, 1, 10, 6, {"base": 7.0, "dims": 10}, 4),
                                                  (4, 2, 128, 64, {"base": 1e4, "dims": 64}, 64), (3, 3, 24, 24, ROTS[5], 8),
                                                  (8, 2, 32, 16, {"base": 5000.0, "dims": 2}, 16), (5, 5, 7, 3, {"base": 3.0, "dims": 4}, 4)])
def test_heads_get_bias_rotation_and_mixed_values(dtype, QH, KH, dk, dv, rot, page):
    from reinfer_b200 import ops
    from reinfer_b200.parts.rope import PairRotary
    g = _gen(QH * dk + dv)
    T, pages = 10, 6
    enc = PairRotary(rot["dims"], rot["base"], rot.get("scaling"))
    enc.prepare(DEV)
    n = (QH + KH) * dk + KH * dv
    x = torch.randn(T, n + QH * dv, generator=g) * 2.0                      # q | k | v | gate
    bias = torch.randn(n, generator=g)
    positions = torch.tensor([0, 1, 2, 15, 16, 17, 64, 300, 1000, 5], dtype=torch.int32)
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    slots[7] = -1
    xb = x[:, :n].double() + bias.double()
    q_ref = plain.rotate_pairs(xb[:, :QH * dk].reshape(T, QH, dk), positions, rot)
    k_ref = plain.rotate_pairs(xb[:, QH * dk:(QH + KH) * dk].reshape(T, KH, dk), positions, rot)
    v_own = xb[:, (QH + KH) * dk:].reshape(T, KH, dv)
    lam = torch.tensor([0.37])
    v_other = torch.randn(T, KH, dv, generator=g)
    tol = 2e-4 if dtype == torch.float32 else 1e-2

    def look(cache, v_ref):
        c = cache.double().cpu()
        touched = torch.zeros_like(c, dtype=torch.bool)
        for t in range(T):
            s = int(slots[t])
            if s < 0:
                continue
            pg, off = s // page, s % page
            for hh in range(KH):
                a = (hh * page + off) * dk
                assert (c[pg, a:a + dk] - k_ref[t, hh]).abs().max() <= tol * k_ref.abs().max()
                b = KH * page * dk + (hh * page + off) * dv
                assert (c[pg, b:b + dv] - v_ref[t, hh]).abs().max() <= tol * v_ref.abs().max()
                touched[pg, a:a + dk] = True
                touched[pg, b:b + dv] = True
        assert (c[~touched] == 77.0).all()

    for vmix in (0, 1, 2):
        q_out = torch.empty(T, QH, dk, dtype=dtype, device=DEV)
        cache = torch.full((pages, KH * page * (dk + dv)), 77.0, dtype=dtype, device=DEV)
        v_first = None
        if vmix == 1:
            v_first = torch.full((T, KH * dv), -3.0, dtype=torch.float32, device=DEV)
        elif vmix == 2:
            v_first = v_other.reshape(T, KH * dv).float().to(DEV)
        ops.rotary_heads_append(x.to(DEV), bias.to(DEV), positions.to(DEV), enc.freq, rot["dims"], enc.magnitude, slots.to(DEV), q_out, cache,
                                QH, KH, dk, dv, page, vmix, lam.to(DEV) if vmix == 2 else None, v_first)
        assert (q_out.double().cpu() - q_ref).abs().max() <= tol * q_ref.abs().max()
        if vmix == 2:
            look(cache, (1.0 - lam.double()) * v_own + lam.double() * v_other.double())
        else:
            look(cache, v_own)
        if vmix == 1:                                        # the kept values: 32-bit, with bias, also of the row that stores nothing
            assert (v_first.double().cpu().view(T, KH, dv) - v_own).abs().max() <= 1e-6 * v_own.abs().max()
    # no bias, no slots: the queries alone
    q2 = torch.empty(T, QH, dk, dtype=dtype, device=DEV)
    ops.rotary_heads_append(x.to(DEV), None, positions.to(DEV), enc.freq, rot["dims"], enc.magnitude, None, q2, cache, QH, KH, dk, dv, page)
    ref2 = plain.rotate_pairs(x[:, :QH * dk].double().reshape(T, QH, dk), positions, rot)
    assert (q2.double().cpu() - ref2).abs().max() <= tol * ref2.abs().max()


# ------------------------------------------------------------------ per-head linear maps
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,n_in,n_out", [(1, 4, 16, 40), (5, 3, 10, 13), (40, 16, 16, 48), (70, 8, 64, 96), (33, 2, 24, 24), (64, 1, 6, 7)])
def test_every_head_has_its_own_matrix(dtype, T, H, n_in, n_out):
    from reinfer_b200 import ops
    g = _gen(T + n_in)
    big = torch.randn(T, H, n_in + 8, generator=g).to(dtype)
    w = (torch.randn(H, n_out, n_in, generator=g) / math.sqrt(n_in)).to(dtype)
    x = big[:, :, :n_in]
    ref = torch.einsum("thi,hoi->tho", x.double(), w.double())
    y = torch.full((T, H, n_out + 8), 9.0, dtype=dtype, device=DEV)
    ops.heads_linear(big.to(DEV)[:, :, :n_in], w.to(DEV), y[:, :, 8:])
    out = y.double().cpu()
    assert (out[:, :, 8:] - ref).abs().max() <= (1e-5 if dtype == torch.float32 else 1e-2) * ref.abs().max()
    assert (out[:, :, :8] == 9.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,n_in,n_out,n_tail,rot_dims", [(1, 4, 16, 40, 8, 8), (70, 3, 24, 13, 6, 4), (130, 16, 128, 200, 64, 64),
                                                          (9, 2, 72, 64, 16, 0), (65, 5, 8, 136, 10, 10)])
def test_heads_map_carries_a_rotated_tail_and_ignores_the_batch(dtype, T, H, n_in, n_out, n_tail, rot_dims):
    """The columns behind a head's inputs go behind its outputs, rotated by position; a token alone gives the very bits it
    gives among the others (rows beyond a tile's end, tiles of unequal fill)."""
    from reinfer_b200 import ops
    from reinfer_b200.parts.rope import PairRotary
    g = _gen(T * 3 + n_in + n_tail)
    rot = {"base": 1000.0, "dims": rot_dims, "scaling": None}
    enc = PairRotary(dims=rot_dims, base=rot["base"], scaling=None)
    enc.prepare(DEV)
    x = torch.randn(T, H, n_in + n_tail, generator=g).to(dtype)
    w = (torch.randn(H, n_out, n_in, generator=g) / math.sqrt(n_in)).to(dtype)
    positions = torch.randint(0, 3000, (T,), generator=g, dtype=torch.int32)
    ref = torch.cat([torch.einsum("thi,hoi->tho", x[:, :, :n_in].double(), w.double()),
                     plain.rotate_pairs(x[:, :, n_in:].float(), positions, rot).double()], dim=2)   # angles in 32-bit, as the design has them
    y = torch.empty(T, H, n_out + n_tail, dtype=dtype, device=DEV)
    tail = (positions.to(DEV), enc.freq, rot_dims, enc.magnitude)
    ops.heads_linear(x.to(DEV), w.to(DEV), y, tail=tail)
    assert (y.double().cpu() - ref).abs().max() <= (1e-5 if dtype == torch.float32 else 1e-2) * ref.abs().max()
    for t in sorted({0, T // 2, T - 1}):
        one = torch.empty(1, H, n_out + n_tail, dtype=dtype, device=DEV)
        ops.heads_linear(x[t:t + 1].to(DEV), w.to(DEV), one, tail=(positions[t:t + 1].to(DEV), enc.freq, rot_dims, enc.magnitude))
        assert torch.equal(one[0], y[t])


# ------------------------------------------------------------------ attention: soft cap, sink, values inside the keys, gate
def _paged(k, v, page, KH, dk, dv, pages_total, table):
    """Scatter k [n, KH, dk] and v [n, KH, dv] (None: the pages hold keys only) into a cache [pages][K | V] by a block table."""
    dvs = 0 if v is None else dv
    cache = torch.full((pages_total, KH * page * (dk + dvs)), float("nan"), dtype=k.dtype)
    for pos in range(k.shape[0]):
        pg, off = table[pos // page], pos % page
        for h in range(KH):
            a = (h * page + off) * dk
            cache[pg, a:a + dk] = k[pos, h]
            if v is not None:
                b = KH * page * dk + (h * page + off) * dv
                cache[pg, b:b + dv] = v[pos, h]
    return cache


def _plain_attention(q, k, v, scale, softcap, sink, gate):
    """q [n, QH, dk], k [n, KH, dk], v [n, KH, dv] in float64 through the plain one-head function."""
    QH, KH = q.shape[1], k.shape[1]
    heads = [plain.causal_softmax_head(q[:, h], k[:, h // (QH // KH)], v[:, h // (QH // KH)], scale, softcap,
                                       None if sink is None else sink[h].double()) for h in range(QH)]
    out = torch.stack(heads, dim=1)
    return out if gate is None else out * torch.sigmoid(gate.double()).view(out.shape)


def _ctx(lo, hi):
    T = hi - lo
    return SimpleNamespace(tok_entry=torch.zeros(T, dtype=torch.int32, device=DEV), positions=torch.arange(lo, hi, dtype=torch.int32, device=DEV),
                           n_decode=1 if T == 1 else 0, n_entries=1, q_start=[0, T], start_pos=[lo], max_kv_len=hi, decode_kv_tiles=None,
                           cu_q=torch.tensor([0, T], dtype=torch.int32, device=DEV), kv_len=torch.tensor([hi], dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("QH,KH,dk,dv,page,softcap,sink,gate,v_in_k", [
    (6, 3, 16, 24, 8, 3.0, True, True, False),          # everything at once, value heads wider than the keys'
    (2, 1, 10, 6, 4, 2.5, True, True, False),           # sizes no tensor-core kernel takes
    (4, 2, 128, 64, 64, 15.0, True, True, False),
    (8, 2, 128, 128, 16, 12.0, True, True, False),      # heads of 128: prompts go to the tcgen05 kernel
    (4, 4, 128, 128, 64, 0.0, True, False, False),
    (4, 1, 128, 128, 16, 8.0, False, False, False),
    (2, 2, 128, 128, 8, 0.0, False, True, False),
    (4, 2, 96, 48, 16, 0.0, True, False, False),        # a sink alone
    (8, 1, 32, 16, 16, 4.0, False, False, False),       # a cap alone
    (4, 4, 64, 64, 64, 0.0, False, True, False),        # a gate alone
    (16, 1, 64, 48, 16, 0.0, False, False, True),       # one shared key row, the values are its first columns
    (3, 1, 13, 7, 4, 0.0, False, False, True),
    (8, 1, 128, 96, 64, 0.0, False, False, True),
    (4, 1, 192, 128, 64, 0.0, False, False, True),
    (2, 1, 40, 24, 8, 5.0, True, True, True)])
def test_attention_options_see_what_they_should(dtype, QH, KH, dk, dv, page, softcap, sink, gate, v_in_k):
    """The very first key of the request is made to stand out (hundreds of keys back): without a cap it takes every row,
    with a cap its score is bounded and the other keys and the sink keep their shares.  Whole prompt, token by token,
    and pieces that end at page borders and inside pages, against the plain statement."""
    from reinfer_b200 import ops
    g = _gen(QH * dk + dv + page)
    n, scale = 330, (0.3 if dk <= 32 else dk ** -0.5)
    q = torch.randn(n, QH, dk, generator=g)
    k = torch.randn(n, KH, dk, generator=g)
    q[:, :, dk - 1] = 2.0
    k[0, :, dk - 1] = 10.0 / scale                           # a score of 20 above the others' few units
    q, k = q.to(dtype), k.to(dtype)
    v = k[:, :, :dv].clone() if v_in_k else torch.randn(n, KH, dv, generator=g).to(dtype)
    # a sink as large as the largest score that can be (the cap, or the far key's 20): it takes about half
    sink_w = (torch.randn(QH, generator=g) + (softcap or 20.0)).float() if sink else None
    gate_x = torch.randn(n, QH * dv + 5, generator=g).float() * 2.0 if gate else None          # rows wider than the gate
    n_pages = -(-n // page)
    table = torch.randperm(n_pages + 3, generator=g)[:n_pages].tolist()
    cache = _paged(k, None if v_in_k else v, page, KH, dk, dv, n_pages + 3, table).to(DEV)
    group = SimpleNamespace(block_table=torch.tensor([table], dtype=torch.int32, device=DEV), page_size=page)
    ref = _plain_attention(q.double(), k.double(), v.double(), scale, softcap or None, sink_w, None if gate_x is None else gate_x[:, :QH * dv])
    ungated = _plain_attention(q.double(), k.double(), v.double(), scale, softcap or None, sink_w, None)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    gate_dev = None if gate_x is None else gate_x.to(DEV)

    def run(lo, hi):
        more = ops.AttentionExtras(softcap=softcap, sink=None if sink_w is None else sink_w.to(DEV), v_in_k=v_in_k,
                                   gate=None if gate_dev is None else gate_dev[lo:hi, :QH * dv])
        out = torch.empty(hi - lo, QH, dv, dtype=dtype, device=DEV)
        ops.biased_attention(_ctx(lo, hi), q[lo:hi].contiguous().to(DEV), cache, group, out, QH, KH, dk, dv, 0, scale, None, more=more)
        return out.double().cpu()

    whole = run(0, n)
    assert (whole - ref).abs().max() <= tol * ref.abs().max()
    one_by_one = torch.cat([run(i, i + 1) for i in list(range(0, 70)) + list(range(n - 40, n))])
    assert (one_by_one - torch.cat([ref[:70], ref[n - 40:]])).abs().max() <= tol * ref.abs().max()
    cuts = sorted(set(c for c in [0, 2, page, 2 * page + 1, 3 * page, n // 2, n // 2 + 2, n - page - 1, n] if 0 <= c <= n))
    pieces = torch.cat([run(a, b) for a, b in zip(cuts, cuts[1:])])
    assert (pieces - ref).abs().max() <= tol * ref.abs().max()
    # what the plain statement itself says, so that the test shows something
    if not softcap and not sink:
        assert (ungated[n - 1, 0] - v[0, 0].double()).abs().max() < 1e-3 * v.abs().max()      # the far key takes the row
    if sink:
        no_sink = _plain_attention(q.double(), k.double(), v.double(), scale, softcap or None, None, None)
        assert (no_sink - ungated).abs().max() > 0.05 * ungated.abs().max()                    # the sink takes a visible share
        assert (ungated[0].abs() < no_sink[0].abs() + 1e-12).all()                             # also of the first token, which sees itself only
    if softcap:
        free = _plain_attention(q.double(), k.double(), v.double(), scale, None, sink_w, None)
        assert (free - ungated).abs().max() > 0.05 * ungated.abs().max()


def test_a_long_prompt_over_one_wide_key_head_takes_the_narrow_tiles():
    """A key head wider than 128 that holds its values (a latent of 104 + 56 rotated, 32 query heads): a prompt long enough
    that its row tiles fill the device six times over runs on the kernel shape with tiles of 32 keys, a shorter one on
    tiles of 64.  Both against the plain statement, whole and in two portions, with the first key standing out."""
    from reinfer_b200 import ops
    QH, KH, dk, dv, page, dtype = 32, 1, 160, 104, 16, torch.bfloat16
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    row_tiles = -(-6 * sms // (QH // 16))                      # 16 heads a row tile: QH / 16 CTAs per tile of 4 tokens
    n = 4 * row_tiles + 40
    g = _gen(n)
    scale = dk ** -0.5
    q = torch.randn(n, QH, dk, generator=g)
    k = torch.randn(n, KH, dk, generator=g)
    q[:, :, dk - 1] = 2.0
    k[0, :, dk - 1] = 6.0 / scale                              # a score of 12 above the others' few units
    q, k = q.to(dtype), k.to(dtype)
    v = k[:, :, :dv].clone()
    n_pages = -(-n // page)
    table = torch.randperm(n_pages + 2, generator=g)[:n_pages].tolist()
    cache = _paged(k, None, page, KH, dk, dv, n_pages + 2, table).to(DEV)
    group = SimpleNamespace(block_table=torch.tensor([table], dtype=torch.int32, device=DEV), page_size=page)
    ref = _plain_attention(q.float(), k.float(), v.float(), scale, None, None, None).double()
    assert (ref[n - 1, 0] - v[0, 0].double()).abs().max() < 0.05 * v.abs().max()               # the far key takes most of the last row

    def run(lo, hi):
        more = ops.AttentionExtras(softcap=0.0, sink=None, v_in_k=True, gate=None)
        out = torch.empty(hi - lo, QH, dv, dtype=dtype, device=DEV)
        ops.biased_attention(_ctx(lo, hi), q[lo:hi].contiguous().to(DEV), cache, group, out, QH, KH, dk, dv, 0, scale, None, more=more)
        return out.double().cpu()

    tol = 2e-2 * ref.abs().max()
    assert (run(0, n) - ref).abs().max() <= tol                                                  # narrow tiles
    assert (torch.cat([run(0, 37), run(37, n)]) - ref).abs().max() <= tol                       # 37 tokens on tiles of 64, the rest narrow
    half = n // 2
    assert (torch.cat([run(0, half), run(half, n)]) - ref).abs().max() <= tol                   # both halves on tiles of 64


def test_a_batch_of_unequal_requests_equals_each_alone():
    """Three requests in one launch - two single tokens at different lengths and a portion - against each by itself,
    with cap, sink and gate, and with the values inside one shared key row."""
    from reinfer_b200 import ops
    g = _gen(9)
    lens, new = [77, 130, 52], [1, 1, 20]
    for QH, KH, dk, dv, page, v_in_k in ((6, 2, 32, 16, 8, False), (8, 1, 48, 32, 16, True)):
        for dtype in (torch.float32, torch.bfloat16):
            qs = [torch.randn(n, QH, dk, generator=g).to(dtype) for n in lens]
            ks = [torch.randn(n, KH, dk, generator=g).to(dtype) for n in lens]
            vs = [kk[:, :, :dv].clone() if v_in_k else torch.randn(kk.shape[0], KH, dv, generator=g).to(dtype) for kk in ks]
            sink_w = None if v_in_k else torch.randn(QH, generator=g).float() + 1.0
            gates = None if v_in_k else [torch.randn(n, QH * dv, generator=g).float() for n in lens]
            softcap = 0.0 if v_in_k else 2.0
            pages = [-(-n // page) for n in lens]
            perm = torch.randperm(sum(pages) + 2, generator=g).tolist()
            tables, at = [], 0
            for p in pages:
                tables.append(perm[at:at + p])
                at += p
            stored = dk if v_in_k else dk + dv
            cache = torch.full((sum(pages) + 2, KH * page * stored), float("nan"), dtype=dtype)
            for kk, vv, tb in zip(ks, vs, tables):
                part = _paged(kk, None if v_in_k else vv, page, KH, dk, dv, cache.shape[0], tb)
                for pg in tb:
                    cache[pg] = part[pg]
            bt = torch.full((3, max(pages)), -1, dtype=torch.int32)
            for e, tb in enumerate(tables):
                bt[e, :len(tb)] = torch.tensor(tb, dtype=torch.int32)
            group = SimpleNamespace(block_table=bt.to(DEV), page_size=page)
            q_cat = torch.cat([qq[n - m:] for qq, n, m in zip(qs, lens, new)]).contiguous().to(DEV)
            gate_cat = None if gates is None else torch.cat([gg[n - m:] for gg, n, m in zip(gates, lens, new)]).contiguous().to(DEV)
            cu = [0, 1, 2, 22]
            ctx = SimpleNamespace(tok_entry=torch.tensor([0, 1] + [2] * 20, dtype=torch.int32, device=DEV),
                                  positions=torch.tensor([lens[0] - 1, lens[1] - 1] + list(range(lens[2] - 20, lens[2])), dtype=torch.int32, device=DEV),
                                  n_decode=2, n_entries=3, q_start=cu, start_pos=[lens[0] - 1, lens[1] - 1, lens[2] - 20], max_kv_len=max(lens),
                                  decode_kv_tiles=None, cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                                  kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV))
            out = torch.empty(22, QH, dv, dtype=dtype, device=DEV)
            more = ops.AttentionExtras(softcap=softcap, sink=None if sink_w is None else sink_w.to(DEV), v_in_k=v_in_k, gate=gate_cat)
            ops.biased_attention(ctx, q_cat, cache.to(DEV), group, out, QH, KH, dk, dv, 0, 0.2, None, more=more)
            out = out.double().cpu()
            at = 0
            for e, (qq, kk, vv, n, m) in enumerate(zip(qs, ks, vs, lens, new)):
                ref = _plain_attention(qq.double(), kk.double(), vv.double(), 0.2, softcap or None, sink_w, None if gates is None else gates[e])[n - m:]
                assert (out[at:at + m] - ref).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2) * ref.abs().max()
                at += m


# ------------------------------------------------------------------ norms whose weights are stored around zero
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("h", [52, 64, 200, 1030])
def test_offset_norm_and_output_norm(dtype, h):
    """rms(x) * (1 + w) * gain before a sublayer, and x += m * rms(y) * (1 + w) behind it; the weight tensor is small
    (a hundredth), so a factor of w instead of 1 + w would show at once."""
    from reinfer_b200.parts.base import build_part
    from reinfer_b200.parts.spec import PartSpec
    g = _gen(h)
    T, eps, mult, gain = 7, 1e-5, 0.3, 0.5
    w = (torch.randn(h, generator=g) * 0.01).to(dtype)
    x = torch.randn(T, h, generator=g) * 4.0
    y = torch.randn(T, h, generator=g) * 0.2
    ctx = SimpleNamespace(dtype=dtype, device=torch.device(DEV), norm_ahead=None, fresh_residual=False)
    pre = build_part("norm", PartSpec("rmsnorm", {"width": h, "eps": eps, "weight_name": "", "unit_offset": True, "gain": gain}, "n"))
    pre.bind({"": w.to(DEV)})
    assert pre.weight.dtype == torch.float32
    ref = plain.norm_offset(x.double(), w.double(), eps) * gain
    got = pre.forward(ctx, x.to(DEV))
    got = got.rows if hasattr(got, "rows") else got
    assert (got.double().cpu() - ref).abs().max() <= (1e-5 if dtype == torch.float32 else 1e-2) * ref.abs().max()
    post = build_part("norm", PartSpec("rms_out", {"width": h, "eps": eps, "mult": mult, "weight_name": "", "unit_offset": True}, "n"))
    post.bind({"": w.to(DEV)})
    stream = x.to(DEV).clone()
    post.add(ctx, stream, y.to(DEV), None)
    want = x.double() + mult * plain.norm_offset(y.double(), w.double(), eps)
    assert (stream.double().cpu() - want).abs().max() <= 1e-5 * want.abs().max()              # the stream is 32-bit in every dtype


@pytest.mark.parametrize("h", [52, 64, 200, 1030, 2048])
@pytest.mark.parametrize("stack", [1, 3])
def test_output_norm_leaves_the_next_norm_its_rows(h, stack):
    """The output norm's kernel can leave what the norm that reads the stream next needs - the new stream times that
    norm's weight, and the row's sum of squares - and the stream itself is the same bits with and without."""
    from reinfer_b200 import ops
    g = _gen(h + stack)
    T, eps, mult = 5, 1e-5, 0.4
    w = torch.randn(h, generator=g).float() * 0.1 + 1.0
    w_next = torch.randn(h, generator=g).float() * 0.1 + 1.0
    x = torch.randn(T, h, generator=g) * 3.0
    y = torch.randn(stack, T, h, generator=g) * 0.3
    ys = y.double().sum(0)
    want = x.double() + mult * ys / torch.sqrt((ys * ys).mean(-1, keepdim=True) + eps) * w.double()
    alone, both = x.to(DEV).clone(), x.to(DEV).clone()
    assert ops.residual_outnorm(alone, y.to(DEV), w.to(DEV), eps, mult) is None
    rows, sumsq = ops.residual_outnorm(both, y.to(DEV), w.to(DEV), eps, mult, next_w=w_next.to(DEV))
    assert torch.equal(alone, both)
    assert (both.double().cpu() - want).abs().max() <= 1e-5 * want.abs().max()
    assert (rows.double().cpu() - want * w_next.double()).abs().max() <= 1e-2 * want.abs().max()
    total = sumsq.double().sum(-1).cpu()
    assert ((total - (want * want).sum(-1)).abs() <= 1e-5 * (want * want).sum(-1)).all()

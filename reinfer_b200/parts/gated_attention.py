"""Softmax attention with grouped key/value heads and five options on top of the plain form, each a parameter:

    q, k, v = W h + b                            projections with biases (`bias=True`), value heads of their own size
    rotation                                     a registered position encoding over the first dimensions of q and k
                                                 (kind `rope_pairs`: neighbouring pairs)
    score   = cap * tanh(q . k * scale / cap)    `softcap` (None: q . k * scale)
    softmax with a sink                          `sink=True`: a learned number per head joins the denominator as
                                                 exp(sink_h); it has no key and no value, is neither scaled nor capped
    value mixing                                 `v_mix`: "first" - the layer's values (with bias) are kept for the step's
                                                 tokens; "mix" - v <- (1 - lambda) v + lambda v_first with the learned lambda
                                                 (tensor `vmix`) before v is cached; the layers of a model that say so share
                                                 the first one's values of the same token (through `ctx.shared`)
    output gate                                  `gate=True`: the heads' outputs are multiplied by sigmoid(W_g h)

Position i sees every j <= i.  The projections q, k, v (and g) are one product with the rows concatenated at load;
it leaves 32-bit sums, to which `rotary_heads_append` adds the biases, applies the rotation and the mixing, and
rounds once on the way to the queries' tensor and the cache.  Soft cap, sink and gate are options of the attention
kernels (`ops.AttentionExtras`), so the gate costs no pass of its own.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Mixer, PagedKVSpec, build_part, register_part
from .linear import matmul, matmul_into_residual, takes_row_scaled
from .spec import PartSpec

V_FIRST_KEY = "gated_attention.v_first"


class GatedAttention(Mixer):
    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, position: Optional[dict] = None,
                 bias: bool = True, softcap: Optional[float] = None, sink: bool = True, v_mix: Optional[str] = None,
                 gate: bool = True, names=None):
        self.hidden, self.QH, self.KH, self.dk, self.dv = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        if self.KH <= 0 or self.QH % self.KH:
            raise ValueError(f"gated attention: {self.QH} query heads over {self.KH} key/value heads")
        self.scale = float(scale)
        self.softcap = float(softcap) if softcap else 0.0
        if v_mix not in (None, "first", "mix"):
            raise ValueError(f"gated attention: v_mix {v_mix!r} (None, 'first' or 'mix')")
        self.bias, self.sink, self.v_mix, self.gate = bool(bias), bool(sink), v_mix, bool(gate)
        pos = dict(position) if position else None
        self.position = build_part("position", PartSpec(pos.pop("kind"), pos)) if pos else None
        self.rot = int(getattr(self.position, "dims", 0)) if self.position is not None else 0
        if self.rot > self.dk:
            raise ValueError(f"gated attention: {self.rot} rotated dimensions in heads of {self.dk}")
        self.w_in = self.w_o = self.b_in = self.sink_w = self.lam = None

    def param_specs(self):
        h, QH, KH, dk, dv = self.hidden, self.QH, self.KH, self.dk, self.dv
        out = {"q": ParamSpec((QH * dk, h)), "k": ParamSpec((KH * dk, h)), "v": ParamSpec((KH * dv, h)), "o": ParamSpec((h, QH * dv))}
        if self.bias:
            out.update({"q.b": ParamSpec((QH * dk,), std=0.1), "k.b": ParamSpec((KH * dk,), std=0.1), "v.b": ParamSpec((KH * dv,), std=0.1)})
        if self.sink:
            out["sink"] = ParamSpec((QH,), std=1.0)
        if self.v_mix is not None:
            out["vmix"] = ParamSpec((), std=0.3)               # the first layer's is never read
        if self.gate:
            out["g"] = ParamSpec((QH * dv, h))
        return out

    def cache_spec(self):
        return PagedKVSpec(self.KH, self.dk, None, None if self.dv == self.dk else self.dv)

    def bind(self, t):
        mats = [t["q"], t["k"], t["v"]] + ([t["g"]] if self.gate else [])
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = t["o"]
        self.b_in = torch.cat([t["q.b"].float(), t["k.b"].float(), t["v.b"].float()]).contiguous() if self.bias else None
        self.sink_w = t["sink"].float().contiguous() if self.sink else None
        self.lam = t["vmix"].float().reshape(1).contiguous() if self.v_mix == "mix" else None

    def prepare(self, device, dtype) -> None:
        if self.position is not None:
            self.position.prepare(device)

    @property
    def takes_row_scaled(self) -> bool:
        return takes_row_scaled(self.w_in)

    def forward(self, ctx, xn, residual, cache):
        T, QH, KH, dk, dv = xn.shape[0], self.QH, self.KH, self.dk, self.dv
        g = cache.group
        act, dev = ctx.dtype, ctx.device
        proj = matmul(ctx, xn, self.w_in, out_dtype=torch.float32)                 # [T, q | k | v | g], 32-bit sums
        vmix, v_first = 0, None
        if self.v_mix == "first":
            vmix = 1
            v_first = ctx.shared[V_FIRST_KEY] = torch.empty((T, KH * dv), dtype=torch.float32, device=dev)
        elif self.v_mix == "mix":
            v_first = ctx.shared.get(V_FIRST_KEY)
            if v_first is None or v_first.shape != (T, KH * dv):
                raise ValueError("gated attention: a layer that mixes values needs an earlier layer that keeps its own, of the same size")
            vmix = 2
        q = torch.empty((T, QH, dk), dtype=act, device=dev)
        freq = self.position.freq if self.position is not None else None
        mag = self.position.magnitude if self.position is not None else 1.0
        ops.rotary_heads_append(proj, self.b_in, ctx.positions, freq, self.rot, mag, g.kv_slot if cache.write else None, q, cache.kv,
                                QH, KH, dk, dv, g.page_size, vmix, self.lam, v_first)
        gate = proj[:, (QH + KH) * dk + KH * dv:] if self.gate else None
        more = ops.AttentionExtras(softcap=self.softcap, sink=self.sink_w, gate=gate)
        heads = torch.empty((T, QH, dv), dtype=act, device=dev)
        ops.biased_attention(ctx, q, cache.kv, g, heads, QH, KH, dk, dv, 0, self.scale, None, more=more)
        return matmul_into_residual(ctx, heads.view(T, QH * dv), self.w_o, residual)


register_part("mixer", "gated_attention", GatedAttention)

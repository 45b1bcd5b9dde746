"""Differential attention: every head runs TWO softmax maps over the same values and subtracts the second from the first.

    q = W_q h      [H heads x (map 1: dim | map 2: dim)]       k = W_k h   [G key heads x (map 1 | map 2)]
    v = W_v h      [G value heads x vdim], shared by the two maps of the heads of its group
    rotation       a registered position encoding over the first dimensions of every map of q and k
    a_m = softmax(q_m . k_m * scale) v          causal, m = 1, 2
    o   = a_1 - lambda a_2,   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff        one number for the layer
    o  <- o / sqrt(mean(o^2) + eps) * (1 - diff)                                      per head, no weight
    o  <- o * sigmoid(W_g h)_head               `gate=True`: one number per token and head
    out = W_o [heads side by side]

To the attention kernels a map is a head: 2H query heads of size `dim` over 2G key heads, ordered so that their plain
grouping pairs the right ones - map m of head g R + r (R = H / G) is query head (2g + m) R + r and reads key head
2g + m.  W_q's rows are permuted to that order at load and W_v's rows are repeated so that both key heads of a group
find the group's values; nothing in a kernel knows of maps.  The output stage (`ops.diff_heads`) undoes the order.
The projections (and the gate) are one product with 32-bit sums; `rotary_heads_append` rotates, rounds once and stores.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Mixer, PagedKVSpec, build_part, register_part
from .linear import matmul, matmul_into_residual, takes_row_scaled
from .spec import PartSpec


class DifferentialAttention(Mixer):
    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, diff: float, eps: float,
                 position: Optional[dict] = None, gate: bool = True):
        self.hidden, self.H, self.G, self.d, self.dv = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        if self.G <= 0 or self.H % self.G:
            raise ValueError(f"differential attention: {self.H} heads over {self.G} key heads")
        self.scale, self.diff, self.eps, self.gate = float(scale), float(diff), float(eps), bool(gate)
        pos = dict(position) if position else None
        self.position = build_part("position", PartSpec(pos.pop("kind"), pos)) if pos else None
        self.w_in = self.w_o = None
        self.lam = 0.0

    def param_specs(self):
        h, H, G, d, dv = self.hidden, self.H, self.G, self.d, self.dv
        out = {"q": ParamSpec((H * 2 * d, h)), "k": ParamSpec((G * 2 * d, h)), "v": ParamSpec((G * dv, h)), "o": ParamSpec((h, H * dv))}
        for n in ("lq1", "lk1", "lq2", "lk2"):
            out[n] = ParamSpec((d,), std=0.1)
        if self.gate:
            out["g"] = ParamSpec((H, h))
        return out

    def cache_spec(self):
        # a map's keys are a key head; the group's values stand beside both
        return PagedKVSpec(2 * self.G, self.d, None, None if self.dv == self.d else self.dv)

    def bind(self, t):
        H, G, d, dv, R = self.H, self.G, self.d, self.dv, self.H // self.G
        # query rows [g, r, m, :] -> [g, m, r, :]
        wq = t["q"].view(G, R, 2, d, -1).permute(0, 2, 1, 3, 4).reshape(2 * H * d, -1)
        wv = t["v"].view(G, 1, dv, -1).expand(G, 2, dv, -1).reshape(2 * G * dv, -1)
        mats = [wq, t["k"], wv] + ([t["g"]] if self.gate else [])
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        rows = sum(m.shape[0] for m in mats)
        if -rows % 8:
            mats.append(torch.zeros((-rows % 8, mats[0].shape[1]), dtype=mats[0].dtype, device=mats[0].device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = t["o"]
        f = {n: t[n].double() for n in ("lq1", "lk1", "lq2", "lk2")}
        lam = torch.exp((f["lq1"] * f["lk1"]).sum().float()) - torch.exp((f["lq2"] * f["lk2"]).sum().float()) + self.diff
        self.lam = float(lam)

    def prepare(self, device, dtype) -> None:
        if self.position is not None:
            self.position.prepare(device)

    @property
    def takes_row_scaled(self) -> bool:
        return takes_row_scaled(self.w_in)

    def forward(self, ctx, xn, residual, cache):
        T, H, G, d, dv = xn.shape[0], self.H, self.G, self.d, self.dv
        g = cache.group
        act, dev = ctx.dtype, ctx.device
        proj = matmul(ctx, xn, self.w_in, out_dtype=torch.float32)                 # [T, q | k | v v | g], 32-bit sums
        q = torch.empty((T, 2 * H, d), dtype=act, device=dev)
        freq, rot = self.position.fused_rotary() if self.position is not None else (None, 0)
        ops.rotary_heads_append(proj, None, ctx.positions, freq, rot, 1.0, g.kv_slot if cache.write else None, q, cache.kv,
                                2 * H, 2 * G, d, dv, g.page_size, half_split=True)
        maps = torch.empty((T, 2 * H, dv), dtype=act, device=dev)
        ops.biased_attention(ctx, q, cache.kv, g, maps, 2 * H, 2 * G, d, dv, 0, self.scale, None)
        at = 2 * (H + G) * d + 2 * G * dv
        gate = proj[:, at:at + H] if self.gate else None
        heads = torch.empty((T, H * dv), dtype=act, device=dev)
        ops.diff_heads(maps, heads, self.lam, self.eps, 1.0 - self.diff, H, G, dv, gate)
        return matmul_into_residual(ctx, heads, self.w_o, residual)


register_part("mixer", "diff_attention", DifferentialAttention)

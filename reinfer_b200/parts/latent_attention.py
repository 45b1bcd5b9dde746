"""Attention whose keys and values are rebuilt from one small latent vector per token:

    a   = rms(W_dq h) * w_q                       the queries' bottleneck (`q_rank`), an RMS norm with a plain weight inside
    q   = W_uq a                                  per head [dim unrotated | rot_dim rotated]
    c,r = split(W_dkv h)                          c (`kv_rank`) is normalised, rms(c) * w_kv; r (`rot_dim`) is rotated and is
                                                  ONE key part for all heads
    k_h = [W_uk,h c | rot(r)],   v_h = W_uv,h c
    score_h(i, j) = (q_h,plain . W_uk,h c_j + rot(q_h,rot) . rot(r_j)) * scale,   j <= i,   ordinary softmax
    `window`: position i sees only the j with i - j < window (pages that the window has passed go back to the pool)
    `gate`:   the heads' outputs are multiplied, element by element, by sigmoid(W_g h) (tensor `g`) before W_o

Only [c | rot(r)] of a token is cached: kv_rank + rot_dim numbers, whatever the head count.  The per-head maps are
moved to the query's side (q_h,plain . W_uk,h c = (W_uk,h^T q_h,plain) . c, and sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j),
so the attention kernels see ONE key/value head of size kv_rank + rot_dim whose values are the first kv_rank columns of
its keys (`AttentionExtras(v_in_k=True)`), shared by all query heads: each cached row is read once for all heads.  The
rotation is a registered position encoding (kind `rope_pairs`: neighbouring pairs, optional frequency stretching).
`scale` is used as given.

Launches: fused projection [W_dq; W_dkv] -> `latent_prep` (both norms, the shared key's rotation, the cache store) ->
W_uq -> per-head W_uk^T on the plain part with the rotation of the rotated part behind it (`heads_linear`, one launch for
all heads) -> attention -> per-head W_uv (`heads_linear`, whose epilogue applies the gate) -> output projection.  The
bottleneck rows (and the gate's) reach their readers as 32-bit sums.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Mixer, PagedKVSpec, build_part, register_part
from .linear import matmul, matmul_into_residual, takes_row_scaled
from .spec import PartSpec


class LatentAttention(Mixer):
    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int, scale: float,
                 eps: float, position: Optional[dict] = None, window: Optional[int] = None, gate: bool = False):
        self.hidden, self.H, self.dn, self.dr, self.dv = int(hidden), int(heads), int(dim), int(rot_dim), int(vdim)
        self.rq, self.rkv, self.scale, self.eps = int(q_rank), int(kv_rank), float(scale), float(eps)
        if min(self.H, self.dn, self.dv, self.rq, self.rkv) <= 0 or self.dr < 0:
            raise ValueError("latent attention: sizes must be positive")
        self.window, self.gate = (int(window) if window else None), bool(gate)
        if self.window is not None and self.window <= 0:
            raise ValueError(f"latent attention: a window of {window} positions")
        pos = dict(position) if position else None
        self.position = build_part("position", PartSpec(pos.pop("kind"), pos)) if pos else None
        self.rot = int(getattr(self.position, "dims", 0)) if self.position is not None else 0
        if self.rot > self.dr:
            raise ValueError(f"latent attention: {self.rot} rotated dimensions in a part of {self.dr}")
        self.w_in = self.w_uq = self.w_absorb = self.w_uv = self.w_o = self.qw = self.kvw = None

    def param_specs(self):
        h, H = self.hidden, self.H
        out = {"dq": ParamSpec((self.rq, h)), "dq.norm": ParamSpec((self.rq,), init="norm"),
               "uq": ParamSpec((H * (self.dn + self.dr), self.rq)),
               "dkv": ParamSpec((self.rkv + self.dr, h)), "dkv.norm": ParamSpec((self.rkv,), init="norm"),
               "uk": ParamSpec((H * self.dn, self.rkv)), "uv": ParamSpec((H * self.dv, self.rkv)),
               "o": ParamSpec((h, H * self.dv))}
        if self.gate:
            out["g"] = ParamSpec((H * self.dv, h))
        return out

    def cache_spec(self):
        # one head of [c | rot(r)]; no value rows of their own
        return PagedKVSpec(1, self.rkv + self.dr, self.window, 0)

    def bind(self, t):
        mats = [t["dq"], t["dkv"]] + ([t["g"]] if self.gate else [])
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_uq = t["uq"]
        # the keys' per-head map on the query's side: [H, kv_rank, dim] so that q_abs = w_absorb[h] q_plain
        self.w_absorb = t["uk"].view(self.H, self.dn, self.rkv).transpose(1, 2).contiguous()
        self.w_uv = t["uv"].view(self.H, self.dv, self.rkv).contiguous()
        self.w_o = t["o"]
        self.qw, self.kvw = t["dq.norm"].float().contiguous(), t["dkv.norm"].float().contiguous()

    def prepare(self, device, dtype) -> None:
        if self.position is not None:
            self.position.prepare(device)

    @property
    def takes_row_scaled(self) -> bool:
        return takes_row_scaled(self.w_in)

    def forward(self, ctx, xn, residual, cache):
        T, H, dn, dr, dv, rq, rkv = xn.shape[0], self.H, self.dn, self.dr, self.dv, self.rq, self.rkv
        g = cache.group
        act, dev = ctx.dtype, ctx.device
        freq = self.position.freq if self.position is not None else None
        mag = self.position.magnitude if self.position is not None else 1.0
        proj = matmul(ctx, xn, self.w_in, out_dtype=torch.float32)                 # [T, q_rank | kv_rank | rot_dim (| gate)], 32-bit sums
        a = torch.empty((T, rq), dtype=act, device=dev)
        ops.latent_prep(proj, rq, rkv, dr, self.qw, self.kvw, self.eps, ctx.positions, freq, self.rot, mag,
                        g.kv_slot if cache.write else None, a, cache.kv, g.page_size)
        q = matmul(ctx, a, self.w_uq).view(T, H, dn + dr)
        qf = torch.empty((T, H, rkv + dr), dtype=act, device=dev)                  # [W_uk^T q_plain | rot(q_rot)] per head
        ops.heads_linear(q, self.w_absorb, qf, tail=(ctx.positions, freq, self.rot, mag))     # the rotated part rides along
        lat = torch.empty((T, H, rkv), dtype=act, device=dev)
        ops.biased_attention(ctx, qf, cache.kv, g, lat, H, 1, rkv + dr, rkv, self.window or 0, self.scale, None,
                             more=ops.AttentionExtras(v_in_k=True))
        heads = torch.empty((T, H, dv), dtype=act, device=dev)
        at = rq + rkv + dr
        ops.heads_linear(lat, self.w_uv, heads, gate=proj[:, at:at + H * dv] if self.gate else None)
        return matmul_into_residual(ctx, heads.view(T, H * dv), self.w_o, residual)


register_part("mixer", "latent_attention", LatentAttention)

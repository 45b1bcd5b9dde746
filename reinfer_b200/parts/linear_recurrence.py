"""Mixers whose memory is a matrix state per (request, head) that moves on token by token
(csrc/recurrence.cu): S [dk, dv] in float32 in the request's slot, zero at admission.

  gla            gated linear attention:  S <- diag(a) S + k v^T,  o = S^T q,  q scaled by dk^-1/2,
                 a = sigmoid(W_a2 W_a1 h + b)^(1/tau) per key channel; o per head over its root mean
                 square, times a weight shared by the heads, times silu(W_g h); then W_o.
  general_delta  the generalised delta rule:  with the unit key u = k/|k|,
                 S <- diag(w) S - (a*u)(u^T S) + k v^T (both from the old state),  o = S^T r;
                 w = exp(-c sigmoid(W_w2 tanh(W_w1 h) + w0)), c = exp(-1/2);  a = sigmoid(W_a h + b);
                 o per head over its root mean square, times a weight over all heads, times sigmoid(W_g h).
  channel_delta  the gated delta rule with a decay per key channel:  q, k, v through a short causal
                 convolution and silu; q, k to unit vectors (q also times dk^-1/2);
                 S <- g S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T q;
                 g = exp(-exp(A_log[h]) softplus(W_a2 W_a1 h + dt_bias)),  beta = sigmoid(W_b h);
                 o per head over its root mean square, times a shared weight, times sigmoid(W_g2 W_g1 h).

  head_delta     the gated delta rule with ONE decay per head and token: as channel_delta, but
                 g = exp(-exp(A_log[h]) softplus(W_a h + dt_bias[h])) is a scalar of the head, and the read-out
                 is gated by silu(W_g h) (full rank).

Every input projection of a mixer is one product with the rows of its matrices concatenated at load
(padded to a multiple of 8 rows so that slices of the result can feed the next product); gates,
decays, unit vectors and the state are float32 in both precisions.  All read the step's entries from
the device tables only, so decode steps are captured in graphs.  `out_scale` multiplies the mixer's
result (applied before the output projection's input is rounded).
"""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Mixer, SlotStateSpec, register_part
from .linear import matmul, matmul_into_residual
from .shortconv import ShortConv


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.float().contiguous()


class _RecurrentMixer(Mixer):
    steps_from_device_tables = True

    def _fuse(self, tensors, names: List[str]) -> None:
        """One matrix of the named projections' rows, in order; `self.cols[name]` = (first column, width) of the
        product's result.  Rows are padded with zeros to a multiple of 8."""
        mats = [tensors[n] for n in names]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.cols: Dict[str, Tuple[int, int]] = {}
        at = 0
        for n, m in zip(names, mats):
            self.cols[n] = (at, m.shape[0])
            at += m.shape[0]
        pad = -at % 8
        if pad:
            mats.append(torch.zeros((pad, mats[0].shape[1]), dtype=mats[0].dtype, device=mats[0].device))
        self.w_in = torch.cat(mats, dim=0).contiguous()

    def _col(self, proj: torch.Tensor, name: str, upto: str = None) -> torch.Tensor:
        a, n = self.cols[name]
        if upto is not None:
            b, m = self.cols[upto]
            n = b + m - a
        return proj[:, a:a + n]


class GatedLinearAttention(_RecurrentMixer):
    def __init__(self, hidden: int, heads: int, dim: int, vdim: int, tau: float, decay_rank: int, eps: float,
                 out_scale: float = 1.0):
        self.hidden, self.H, self.dk, self.dv = int(hidden), int(heads), int(dim), int(vdim)
        self.tau, self.rank, self.eps, self.out_scale = float(tau), int(decay_rank), float(eps), float(out_scale)
        if self.tau <= 0:
            raise ValueError("gla: tau must be positive")

    def param_specs(self):
        h, H, dk, dv, r = self.hidden, self.H, self.dk, self.dv, self.rank
        return {"q": ParamSpec((H * dk, h)), "k": ParamSpec((H * dk, h)), "v": ParamSpec((H * dv, h)),
                "g": ParamSpec((H * dv, h)), "o": ParamSpec((h, H * dv)), "norm": ParamSpec((dv,), init="norm"),
                "a1": ParamSpec((r, h)), "a2": ParamSpec((H * dk, r), std=0.5), "a2.b": ParamSpec((H * dk,), std=1.0)}

    def state_spec(self):
        return SlotStateSpec((self.H, self.dk, self.dv), "float32")

    def bind(self, t):
        self._fuse(t, ["q", "k", "v", "g", "a1"])
        self.w_a2, self.w_o = t["a2"], t["o"]
        self.a2_bias, self.norm_w = _f32(t["a2.b"]), _f32(t["norm"])

    def forward(self, ctx, xn, residual, cache):
        T, H, dk, dv = xn.shape[0], self.H, self.dk, self.dv
        proj = matmul(ctx, xn, self.w_in)
        z = matmul(ctx, self._col(proj, "a1"), self.w_a2, out_dtype=torch.float32)
        o = torch.empty((T, H, dv), dtype=torch.float32, device=proj.device)
        ops.recurrence("diagonal", "sigmoid_root", self._col(proj, "q"), self._col(proj, "k"), self._col(proj, "v"),
                       z, self.a2_bias, cache.state, o, ctx.cu_q, ctx.entry_slot, ctx.n_entries, H, H, dk, dv,
                       gate_param=1.0 / self.tau, q_scale=dk ** -0.5, max_q_len=ctx.max_q_len)
        y = torch.empty((T, H * dv), dtype=proj.dtype, device=proj.device)
        ops.head_norm_gate(o, self.norm_w, self._col(proj, "g"), y, H, dv, self.eps, "silu", self.out_scale)
        return matmul_into_residual(ctx, y, self.w_o, residual)


class GeneralDeltaRule(_RecurrentMixer):
    DECAY_SCALE = math.exp(-0.5)

    def __init__(self, hidden: int, heads: int, dim: int, decay_rank: int, eps: float, out_scale: float = 1.0):
        self.hidden, self.H, self.d = int(hidden), int(heads), int(dim)
        self.rank, self.eps, self.out_scale = int(decay_rank), float(eps), float(out_scale)

    def param_specs(self):
        h, n, r = self.hidden, self.H * self.d, self.rank
        return {"r": ParamSpec((n, h)), "k": ParamSpec((n, h)), "v": ParamSpec((n, h)), "g": ParamSpec((n, h)),
                "a": ParamSpec((n, h)), "a.b": ParamSpec((n,), std=1.0),
                "w1": ParamSpec((r, h)), "w2": ParamSpec((n, r), std=0.5), "w0": ParamSpec((n,), std=1.0),
                "norm": ParamSpec((n,), init="norm"), "o": ParamSpec((h, n))}

    def state_spec(self):
        return SlotStateSpec((self.H, self.d, self.d), "float32")

    def bind(self, t):
        self._fuse(t, ["r", "k", "v", "g", "a", "w1"])
        self.w_w2, self.w_o = t["w2"], t["o"]
        self.w0, self.a_bias, self.norm_w = _f32(t["w0"]), _f32(t["a.b"]), _f32(t["norm"])

    def forward(self, ctx, xn, residual, cache):
        T, H, d = xn.shape[0], self.H, self.d
        proj = matmul(ctx, xn, self.w_in)
        low = self._col(proj, "w1")
        ops.tanh_(low)
        z = matmul(ctx, low, self.w_w2, out_dtype=torch.float32)
        o = torch.empty((T, H, d), dtype=torch.float32, device=proj.device)
        ops.recurrence("delta_old_state", "exp_sigmoid", self._col(proj, "r"), self._col(proj, "k"), self._col(proj, "v"),
                       z, self.w0, cache.state, o, ctx.cu_q, ctx.entry_slot, ctx.n_entries, H, H, d, d,
                       gate_param=self.DECAY_SCALE, a_pre=self._col(proj, "a"), a_bias=self.a_bias, max_q_len=ctx.max_q_len)
        y = torch.empty((T, H * d), dtype=proj.dtype, device=proj.device)
        ops.head_norm_gate(o, self.norm_w, self._col(proj, "g"), y, H, d, self.eps, "sigmoid", self.out_scale)
        return matmul_into_residual(ctx, y, self.w_o, residual)


class ChannelGatedDeltaRule(_RecurrentMixer):
    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, decay_rank: int,
                 gate_rank: int, eps: float, out_scale: float = 1.0):
        self.hidden, self.H, self.G, self.dk, self.dv = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        if self.G <= 0 or self.H % self.G:
            raise ValueError(f"channel_delta: {self.H} heads over {self.G} key heads")
        self.rank_a, self.rank_g, self.eps, self.out_scale = int(decay_rank), int(gate_rank), float(eps), float(out_scale)
        self.conv = ShortConv(("q.conv", "k.conv", "v.conv"), (self.G * self.dk, self.G * self.dk, self.H * self.dv), conv)

    def param_specs(self):
        h, H, G, dk, dv = self.hidden, self.H, self.G, self.dk, self.dv
        out = {"q": ParamSpec((G * dk, h)), "k": ParamSpec((G * dk, h)), "v": ParamSpec((H * dv, h)),
               "b": ParamSpec((H, h)), "A_log": ParamSpec((H,), std=0.5), "norm": ParamSpec((dv,), init="norm"),
               "a1": ParamSpec((self.rank_a, h)), "a2": ParamSpec((H * dk, self.rank_a), std=0.5),
               "dt_bias": ParamSpec((H * dk,), std=1.0),
               "g1": ParamSpec((self.rank_g, h)), "g2": ParamSpec((H * dv, self.rank_g), std=0.5),
               "o": ParamSpec((h, H * dv))}
        out.update(self.conv.param_specs())
        return out

    def state_spec(self):
        return {"S": SlotStateSpec((self.H, self.dk, self.dv), "float32"), "conv": self.conv.state_spec()}

    def bind(self, t):
        self._fuse(t, ["q", "k", "v", "a1", "g1", "b"])
        self.conv.bind(t)
        self.w_a2, self.w_g2, self.w_o = t["a2"], t["g2"], t["o"]
        self.dt_bias, self.a_log, self.norm_w = _f32(t["dt_bias"]), _f32(t["A_log"]), _f32(t["norm"])

    def forward(self, ctx, xn, residual, cache):
        T, H, G, dk, dv = xn.shape[0], self.H, self.G, self.dk, self.dv
        proj = matmul(ctx, xn, self.w_in)
        y = self.conv.forward(ctx, self._col(proj, "q", upto="v"), cache.state["conv"], silu=True)
        z = matmul(ctx, self._col(proj, "a1"), self.w_a2, out_dtype=torch.float32)
        gate = matmul(ctx, self._col(proj, "g1"), self.w_g2)
        o = torch.empty((T, H, dv), dtype=torch.float32, device=proj.device)
        ops.recurrence("delta_gated_state", "exp_softplus", y[:, :G * dk], y[:, G * dk:2 * G * dk], y[:, 2 * G * dk:],
                       z, self.dt_bias, cache.state["S"], o, ctx.cu_q, ctx.entry_slot, ctx.n_entries, H, G, dk, dv,
                       q_scale=dk ** -0.5, unit_qk=True, b_pre=self._col(proj, "b"), rate=self.a_log, max_q_len=ctx.max_q_len)
        out = torch.empty((T, H * dv), dtype=proj.dtype, device=proj.device)
        ops.head_norm_gate(o, self.norm_w, gate, out, H, dv, self.eps, "sigmoid", self.out_scale)
        return matmul_into_residual(ctx, out, self.w_o, residual)


class HeadGatedDeltaRule(_RecurrentMixer):
    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, eps: float, out_scale: float = 1.0):
        self.hidden, self.H, self.G, self.dk, self.dv = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        if self.G <= 0 or self.H % self.G:
            raise ValueError(f"head_delta: {self.H} heads over {self.G} key heads")
        self.eps, self.out_scale = float(eps), float(out_scale)
        self.conv = ShortConv(("q.conv", "k.conv", "v.conv"), (self.G * self.dk, self.G * self.dk, self.H * self.dv), conv)

    def param_specs(self):
        h, H, G, dk, dv = self.hidden, self.H, self.G, self.dk, self.dv
        out = {"q": ParamSpec((G * dk, h)), "k": ParamSpec((G * dk, h)), "v": ParamSpec((H * dv, h)),
               "a": ParamSpec((H, h), std=0.1), "b": ParamSpec((H, h)), "g": ParamSpec((H * dv, h)),
               "A_log": ParamSpec((H,), std=0.5), "dt_bias": ParamSpec((H,), std=1.0),
               "norm": ParamSpec((dv,), init="norm"), "o": ParamSpec((h, H * dv))}
        out.update(self.conv.param_specs())
        return out

    def state_spec(self):
        return {"S": SlotStateSpec((self.H, self.dk, self.dv), "float32"), "conv": self.conv.state_spec()}

    def bind(self, t):
        self._fuse(t, ["q", "k", "v", "g", "b"])
        self.conv.bind(t)
        self.w_a, self.w_o = t["a"], t["o"]
        self.dt_bias, self.a_log, self.norm_w = _f32(t["dt_bias"]), _f32(t["A_log"]), _f32(t["norm"])

    def forward(self, ctx, xn, residual, cache):
        T, H, G, dk, dv = xn.shape[0], self.H, self.G, self.dk, self.dv
        proj = matmul(ctx, xn, self.w_in)
        z = matmul(ctx, xn, self.w_a, out_dtype=torch.float32)              # the decay's pre-activation, one a head: 32-bit sums
        y = self.conv.forward(ctx, self._col(proj, "q", upto="v"), cache.state["conv"], silu=True)
        o = torch.empty((T, H, dv), dtype=torch.float32, device=proj.device)
        ops.recurrence("delta_gated_state", "exp_softplus", y[:, :G * dk], y[:, G * dk:2 * G * dk], y[:, 2 * G * dk:],
                       z, self.dt_bias, cache.state["S"], o, ctx.cu_q, ctx.entry_slot, ctx.n_entries, H, G, dk, dv,
                       q_scale=dk ** -0.5, unit_qk=True, b_pre=self._col(proj, "b"), rate=self.a_log, max_q_len=ctx.max_q_len,
                       gate_per_head=True)
        out = torch.empty((T, H * dv), dtype=proj.dtype, device=proj.device)
        ops.head_norm_gate(o, self.norm_w, self._col(proj, "g"), out, H, dv, self.eps, "silu", self.out_scale)
        return matmul_into_residual(ctx, out, self.w_o, residual)


register_part("mixer", "head_delta", HeadGatedDeltaRule)
register_part("mixer", "gla", GatedLinearAttention)
register_part("mixer", "general_delta", GeneralDeltaRule)
register_part("mixer", "channel_delta", ChannelGatedDeltaRule)

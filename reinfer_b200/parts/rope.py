"""Rotary position encoding, half-split pairing (p, p + rot/2):
angle = pos * theta^(-2p/rot); x'[p] = x[p] cos - x[p+rot/2] sin;
x'[p+rot/2] = x[p] sin + x[p+rot/2] cos   (crates/kernels/src/refs.rs:25-37,
crates/cuda/kernels/dense_kernels.cu:127-170).  The reference evaluates powf per
element on the device; here theta^(-2p/rot) is tabulated once in double precision
and rounded to float32, the angle and its sine and cosine are float32 on the device.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from .base import PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    """`scaling` = {factor, low, high, original} stretches the slow pairs by wavelength: with l = 2 pi / f, a frequency
    with l < original / high stays, one with l > original / low becomes f / factor, and between the two it is
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""

    def __init__(self, head_dim: int, theta: float, rotary_dim: int = 0, scaling: Optional[dict] = None):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) or self.head_dim
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary width {self.rotary_dim} of head_dim {self.head_dim}")
        self.scaling = None
        if scaling:
            self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")}
            if min(self.scaling.values()) <= 0 or self.scaling["high"] == self.scaling["low"]:
                raise ValueError(f"rotation: scaling {scaling}")
        self.inv_freq = None

    def table(self) -> torch.Tensor:
        f = [self.theta ** (-2.0 * p / self.rotary_dim) for p in range(self.rotary_dim // 2)]
        sc = self.scaling
        if sc:
            for p, fp in enumerate(f):
                wave = 2.0 * math.pi / fp
                if wave > sc["original"] / sc["low"]:
                    f[p] = fp / sc["factor"]
                elif wave >= sc["original"] / sc["high"]:
                    s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                    f[p] = (1.0 - s) * fp / sc["factor"] + s * fp
        return torch.tensor(f, dtype=torch.float64).to(torch.float32)

    def prepare(self, device) -> None:
        self.inv_freq = self.table().to(device)

    def fused_rotary(self):
        return self.inv_freq, self.rotary_dim

    def table_key(self):
        sc = tuple(sorted(self.scaling.items())) if self.scaling else None
        return ("rope", self.theta, self.rotary_dim, sc)

    def apply(self, ctx, q, k, positions) -> None:
        """The unfused form, for a mixer that does not take `fused_rotary()`: q [T, QH, d] and k [T, KH, d]
        are rotated in place (through the same kernel, with the head norm and the cache switched off)."""
        for x in (q, k):
            T, heads, d = x.shape
            out = torch.empty_like(x)
            ops.qknorm_rope_append(x.reshape(T, heads * d), None, None, self.inv_freq, positions, None, out, None,
                                   heads, 0, d, self.rotary_dim, 1, 0.0)
            x.copy_(out)


register_part("position", "rope", RotaryEncoding)
register_part("position", "none", lambda **kw: None)


class PairRotary(PositionEncoding):
    """Rotation of NEIGHBOURING dimensions: the pair (2i, 2i + 1) of the first `dims` dimensions of a head turns by
    position * f_i, f_i = base^(-2i / dims); the rest of the head passes.

    `scaling` = {factor s, original L, fast, slow} stretches the slow pairs (YaRN: Peng, Quesnelle, Fan, Shippole,
    "YaRN: Efficient Context Window Extension of Large Language Models"): with n(t) = dims ln(L / (2 pi t)) / (2 ln base),
    the index of the pair that makes t turns within L positions, lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)),
    dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency becomes f_i (1 - ramp_i) + f_i / s
    ramp_i, and cosine and sine are multiplied by `magnitude` = 0.1 ln s + 1.

    Frequencies are tabulated once in double precision and rounded to float32; the angle, its cosine and sine are
    float32 on the device.  The kernels that rotate (`ops.rotary_heads_append`, `ops.latent_prep`, `ops.rotate_pairs`) take
    `freq`, `dims` and `magnitude` from here; mixers call them, so `apply` serves the generic [T, heads, d] form only."""

    def __init__(self, dims: int, base: float, scaling: Optional[dict] = None):
        self.dims, self.base = int(dims), float(base)
        if self.dims < 0 or self.dims % 2 or self.base <= 0:
            raise ValueError(f"pair rotation over {self.dims} dimensions with base {self.base}")
        self.scaling = None
        if scaling:
            self.scaling = {k: float(scaling[k]) for k in ("factor", "original", "fast", "slow")}
            if self.scaling["factor"] <= 0 or self.scaling["original"] <= 0 or self.scaling["fast"] <= 0 or self.scaling["slow"] <= 0:
                raise ValueError(f"pair rotation: scaling {scaling}")
        self.freq = None

    @property
    def magnitude(self) -> float:
        return 0.1 * math.log(self.scaling["factor"]) + 1.0 if self.scaling else 1.0

    def table(self) -> torch.Tensor:
        half = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        sc = self.scaling
        if sc:
            def index_of(turns: float) -> float:
                return self.dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
            lo = max(math.floor(index_of(sc["fast"])), 0)
            hi = min(math.ceil(index_of(sc["slow"])), self.dims - 1)
            for i in range(half):
                ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
                f[i] = f[i] / sc["factor"] * ramp + f[i] * (1.0 - ramp)
        return torch.tensor(f, dtype=torch.float64).to(torch.float32)

    def prepare(self, device) -> None:
        self.freq = self.table().to(device)

    def table_key(self):
        sc = tuple(sorted(self.scaling.items())) if self.scaling else None
        return ("pair_rope", self.base, self.dims, sc)

    def apply(self, ctx, q, k, positions) -> None:
        for x in (q, k):
            ops.rotate_pairs(x, x, positions, self.freq, self.dims, self.magnitude)


register_part("position", "rope_pairs", PairRotary)

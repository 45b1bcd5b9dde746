"""A plain, slow statement of the Zegorax forward pass: one whole sequence at a time, no cache,
no batch, one function per mechanism, torch on the CPU only (float64 unless told otherwise).
It shares no code with `reinfer_b200`; the tests compare the engine with it.

Notation.  x is the residual stream [T, width]; `lin(x, W, b) = x W^T + b` with W stored [out, in];
rms(v) = v / sqrt(mean(v^2) + eps).  Every norm is Dynamic Tanh, `dyt(v) = tanh(alpha v) * w + b`.
A layer reads ONE norm of the stream and adds both sublayers' results at once:

    h = dyt(x);   x += mixer(h) + ff(h)                 (ff may be missing)

Layers `loop.start .. loop.stop - 1` run `loop.times` times in a row with the same weights (each pass
is a layer of its own as far as memories go).  Embedding: token row + learned position row; output:
`lin(dyt(x), embed)`.  Three mixers:

* `delta`             a matrix memory per head written by the delta rule with one decay per head and token;
                      q, k, v through a short causal convolution and silu; q, k unit vectors
* `attention`         differential attention: two softmax maps per head over the same values, the second
                      subtracted with a learned weight; half-split rotation with stretched slow frequencies;
                      a sigmoid gate per head
* `latent_attention`  keys and values rebuilt per head from one normalised latent per token plus one rotated key
                      part shared by the heads; sliding window; neighbouring-pair rotation; an elementwise gate

Feed-forwards: dense gated with tanh-gelu and biases, or a mixture of gated silu experts whose chosen
logits are softmaxed among themselves.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch


# ---------------------------------------------------------------- file reading
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        buf = data[b:en]
        dt = e["dtype"]
        if dt == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f4").copy()).double()
        elif dt == "BF16":
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy()).double()
        elif dt in ("I32", "I64"):
            t = torch.from_numpy(np.frombuffer(buf, dtype="<i4" if dt == "I32" else "<i8").copy()).long()
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = t.reshape(e["shape"])
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ---------------------------------------------------------------- small pieces
def lin(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ w.t()
    return y if b is None else y + b


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def dyt(v: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    return torch.tanh(alpha * v) * w + b


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ---------------------------------------------------------------- rotations
def stretched_frequencies(dims: int, base: float, scaling: Optional[dict]) -> List[float]:
    """f_i = base^(-2i/dims); with `scaling` (factor, low, high, original) a frequency whose wavelength
    l = 2 pi / f is shorter than original/high stays, one longer than original/low is divided by the factor,
    and between the two it is blended with s = (original/l - low) / (high - low)."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            fac, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                pass
            elif wave > orig / low:
                f = f / fac
            else:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / fac + s * f
        out.append(f)
    return out


def rotate_half_split(x: torch.Tensor, positions: torch.Tensor, freqs: List[float]) -> torch.Tensor:
    """x [T, ..., d]: dimension i of the first 2 * len(freqs) turns together with dimension i + len(freqs)."""
    n = len(freqs)
    if n == 0:
        return x
    ang = positions.to(x.dtype)[:, None] * torch.tensor(freqs, dtype=x.dtype)[None, :]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :n], x[..., n:2 * n]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * n:]], dim=-1)


def rotate_neighbours(x: torch.Tensor, positions: torch.Tensor, freqs: List[float]) -> torch.Tensor:
    """x [T, ..., d]: dimensions (2i, 2i + 1) of the first 2 * len(freqs) turn together."""
    n = len(freqs)
    if n == 0:
        return x
    ang = positions.to(x.dtype)[:, None] * torch.tensor(freqs, dtype=x.dtype)[None, :]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., 2 * n:]], dim=-1)


# ---------------------------------------------------------------- softmax attention of one head
def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int] = None) -> torch.Tensor:
    """q [T, d], k [T, d], v [T, dv]: position i sees j <= i, and with a window only i - j < window."""
    T = q.shape[0]
    s = (q @ k.t()) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    s = s.masked_fill(~seen, float("-inf"))
    return torch.softmax(s, dim=-1) @ v


# ---------------------------------------------------------------- mixers
def differential_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = lin(h, w[p + "q"]).view(T, H, 2, d)
    k = lin(h, w[p + "k"]).view(T, G, 2, d)
    v = lin(h, w[p + "v"]).view(T, G, dv)
    rot = m["rot"]
    fr = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    q, k = rotate_half_split(q, pos, fr), rotate_half_split(k, pos, fr)
    lam = torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum()) + m["diff"]
    gate = torch.sigmoid(lin(h, w[p + "g"]))                            # [T, H]
    heads = []
    for hd in range(H):
        g = hd // (H // G)
        a1 = softmax_attention(q[:, hd, 0], k[:, g, 0], v[:, g], m["scale"])
        a2 = softmax_attention(q[:, hd, 1], k[:, g, 1], v[:, g], m["scale"])
        o = rms(a1 - lam * a2, eps) * (1.0 - m["diff"])
        heads.append(o * gate[:, hd:hd + 1])
    return lin(torch.cat(heads, dim=-1), w[p + "o"])


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dn, dr, dv, rkv = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    fr = stretched_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    cq = rms(lin(h, w[p + "dq"]), eps) * w[p + "dq.norm"]
    q = lin(cq, w[p + "uq"]).view(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_neighbours(q[..., dn:], pos, fr)
    down = lin(h, w[p + "dkv"])
    c = rms(down[:, :rkv], eps) * w[p + "dkv.norm"]
    k_rot = rotate_neighbours(down[:, rkv:], pos, fr)                   # one rotated key part for all heads
    k_plain = lin(c, w[p + "uk"]).view(T, H, dn)
    v = lin(c, w[p + "uv"]).view(T, H, dv)
    window = m.get("mask", {}).get("size") if m.get("mask") else None
    heads = []
    for hd in range(H):
        qq = torch.cat([q_plain[:, hd], q_rot[:, hd]], dim=-1)
        kk = torch.cat([k_plain[:, hd], k_rot], dim=-1)
        heads.append(softmax_attention(qq, kk, v[:, hd], m["scale"], window))
    o = torch.cat(heads, dim=-1) * torch.sigmoid(lin(h, w[p + "g"]))
    return lin(o, w[p + "o"])


def short_convolution(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K]: y[t, c] = sum_j taps[c, K - 1 - j] u[t - j, c], zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + padded[K - 1 - j:K - 1 - j + T] * taps[:, K - 1 - j][None, :]
    return y


def unit(v: torch.Tensor) -> torch.Tensor:
    return v / torch.sqrt((v * v).sum(dim=-1, keepdim=True) + 1e-6)


def gated_delta_rule(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(lin(h, w[p + "q"]), w[p + "q.conv"])).view(T, G, dk)
    k = silu(short_convolution(lin(h, w[p + "k"]), w[p + "k.conv"])).view(T, G, dk)
    v = silu(short_convolution(lin(h, w[p + "v"]), w[p + "v.conv"])).view(T, H, dv)
    q, k = unit(q) * dk ** -0.5, unit(k)
    beta = torch.sigmoid(lin(h, w[p + "b"]))                            # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(lin(h, w[p + "a"]) + w[p + "dt_bias"]))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.t() @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.t() @ q[t, g]
    o = rms(out, eps) * w[p + "norm"] * silu(lin(h, w[p + "g"])).view(T, H, dv)
    return lin(o.reshape(T, H * dv), w[p + "o"])


MIXERS = {"attention": differential_attention, "latent_attention": latent_attention, "delta": gated_delta_rule}


# ---------------------------------------------------------------- feed-forwards
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    a = gelu_tanh(lin(h, w[p + "gate"], w[p + "gate.b"])) * lin(h, w[p + "up"], w[p + "up.b"])
    return lin(a, w[p + "down"], w[p + "down.b"])


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, top: int):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmaxed among themselves."""
    z = lin(h, w[p + "router"], w[p + "router.b"])
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def expert_mixture(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    idx, wt = route(h, w, p, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            ht = h[t:t + 1]
            y = lin(silu(lin(ht, w[f"{p}e{e}.gate"])) * lin(ht, w[f"{p}e{e}.up"]), w[f"{p}e{e}.down"])
            out[t] = out[t] + a * y[0]
    return out


def feed_forward(h, w, p, mlp):
    return dense_ff(h, w, p) if mlp["kind"] == "dense" else expert_mixture(h, w, p, mlp)


# ---------------------------------------------------------------- the model
def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, dtype=torch.float64, trace: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  `trace`, if a list, gets the stream after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    T = ids.shape[0]
    eps = cfg["norm"]["eps"]
    x = w["embed"][ids] + w["pos"][:T]
    for i in run_order(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        h = dyt(x, w[p + "norm1"], w[p + "norm1.b"], w[p + "norm1.alpha"])
        y = MIXERS[L["type"]](h, w, p + "mix.", L["mixer"], eps)
        if L.get("mlp") is not None:
            y = y + feed_forward(h, w, p + "mlp.", L["mlp"])
        x = x + y
        if trace is not None:
            trace.append(x.clone())
    return lin(dyt(x, w["final.norm"], w["final.norm.b"], w["final.norm.alpha"]), w["embed"])

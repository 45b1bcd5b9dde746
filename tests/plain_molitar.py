"""A plain, slow statement of the Molitar forward pass: one whole sequence at a time, no cache,
no batch, one function per mechanism, torch on the CPU only (float64 unless told otherwise).
It shares no code with `reinfer_b200`; the tests compare the engine with it.

Notation.  x is the residual stream [T, width]; `lin(x, W) = x W^T` with W stored [out, in];
rms(v) = v / sqrt(mean(v^2) + eps).  Norm weights are stored around zero: norm(v) = rms(v) * (1 + w).
Every sublayer is wrapped by two norms,

    x += m * norm_b(mixer(norm_a(x)));     x += m * norm_d(ff(norm_c(x)))      (the second only with a feed-forward)

and the output is `lin(norm(x), embed) * logit_scale` with the token table as output matrix.  Two mixers:

* `latent_attention`  queries through a low-rank bottleneck with an RMS norm inside; keys and values rebuilt per head
                      from ONE normalised latent vector per token, plus one rotated key part that all heads share;
                      rotation with stretched frequencies (YaRN)
* `attention`         grouped heads, projections with biases, partial rotation, scores squashed by tanh, a softmax
                      whose denominator holds one more learned term per head, values mixed with those of the first
                      such layer, and a sigmoid gate on the heads' outputs

Rotations pair neighbouring dimensions (2i, 2i + 1).  The feed-forward is the gated one with silu.
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


def norm_offset(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: the weight is stored as its distance from one."""
    return rms(v, eps) * (1.0 + w)


def norm_plain(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The norm inside the latent bottlenecks: the weight as stored."""
    return rms(v, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def dense_ff(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return lin(silu(lin(h, gate)) * lin(h, up), down)


# ---------------------------------------------------------------- rotation
def rotary_frequencies(rot: dict) -> (torch.Tensor, float):
    """(frequency of every pair, factor on cosine and sine).  Plain: f_i = base^(-2i / dims).  With `scaling`
    (factor s, original length L, fast and slow turn counts): a pair that turns more than `fast` times within L
    keeps its frequency, one that turns less than `slow` times gets f_i / s, those between are blended linearly by
    their index; cosine and sine grow by 0.1 ln s + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=torch.float64), 1.0
    s, L = float(sc["factor"]), float(sc["original"])

    def index_of(turns: float) -> float:
        return dims * math.log(L / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(f[i] / s * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(s) + 1.0


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """v [T, heads, d]: the first rot['dims'] dimensions of every head are rotated, (2i, 2i+1) together, by
    position * f_i; the rest passes."""
    f, mag = rotary_frequencies(rot)
    dims = int(rot["dims"])
    ang = positions.to(v.dtype)[:, None] * f.to(v.dtype)[None, :]                 # [T, dims/2]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = v.clone()
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---------------------------------------------------------------- softmax attention, one head at a time
def causal_softmax_head(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, softcap: Optional[float] = None,
                        sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q, k [T, d], v [T, dv].  Scores q.k * scale, optionally squashed to cap * tanh(score / cap); position i sees
    j <= i; `sink`: a number that joins the denominator as exp(sink) and brings no value."""
    T = q.shape[0]
    s = (q @ k.t()) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    top = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.reshape(1, 1).to(s.dtype))
    e = torch.exp(s - top)
    den = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(s.dtype) - top)
    return (e / den) @ v


def latent_attention(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    H, dn, dr, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    T = h.shape[0]
    cq = norm_plain(lin(h, w[p + "dq"]), w[p + "dq.norm"], eps)
    q = lin(cq, w[p + "uq"]).view(T, H, dn + dr)
    dkv = lin(h, w[p + "dkv"])
    c = norm_plain(dkv[:, :r], w[p + "dkv.norm"], eps)
    k_shared = rotate_pairs(dkv[:, r:].reshape(T, 1, dr), positions, m["rot"])[:, 0]
    q_rot = rotate_pairs(q[..., dn:].contiguous(), positions, m["rot"])
    k_plain = lin(c, w[p + "uk"]).view(T, H, dn)
    val = lin(c, w[p + "uv"]).view(T, H, dv)
    heads = []
    for i in range(H):
        qi = torch.cat([q[:, i, :dn], q_rot[:, i]], dim=-1)
        ki = torch.cat([k_plain[:, i], k_shared], dim=-1)
        heads.append(causal_softmax_head(qi, ki, val[:, i], float(m["scale"])))
    return lin(torch.cat(heads, dim=-1), w[p + "o"])


def gated_attention(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str,
                    v_first: Optional[torch.Tensor]):
    """Returns (output, the values this layer would hand on as the first ones).  v_first: the first value-mixing
    layer's values [T, G, dv], or None where this layer is that first one or mixes nothing."""
    H, G, d, dv = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = lin(h, w[p + "q"], w[p + "q.b"]).view(T, H, d)
    k = lin(h, w[p + "k"], w[p + "k.b"]).view(T, G, d)
    v = lin(h, w[p + "v"], w[p + "v.b"]).view(T, G, dv)
    own_v = v
    if m.get("v_mix") and v_first is not None:
        lam = w[p + "vmix"].reshape(())
        v = (1.0 - lam) * v + lam * v_first
    q, k = rotate_pairs(q, positions, m["rot"]), rotate_pairs(k, positions, m["rot"])
    heads = []
    for i in range(H):
        g = i // (H // G)
        heads.append(causal_softmax_head(q[:, i], k[:, g], v[:, g], float(m["scale"]), m.get("softcap"), w[p + "sink"][i]))
    out = torch.cat(heads, dim=-1) * torch.sigmoid(lin(h, w[p + "g"]))
    return lin(out, w[p + "o"]), own_v


# ---------------------------------------------------------------- the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; `layers_out` collects the residual stream after every layer."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    T = x.shape[0]
    positions = torch.arange(T)
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm_offset(x, w[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            y = latent_attention(h, positions, layer["mixer"], w, p + "mix.", eps)
        elif layer["type"] == "attention":
            mixes = bool(layer["mixer"].get("v_mix"))
            y, own = gated_attention(h, positions, layer["mixer"], w, p + "mix.", v_first if mixes else None)
            if mixes and v_first is None:
                v_first = own
        else:
            raise ValueError(layer["type"])
        x = x + mult * norm_offset(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = norm_offset(x, w[p + "norm2"], eps)
            y = dense_ff(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"])
            x = x + mult * norm_offset(y, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(norm_offset(x, w["final.norm"], eps), w["embed"]) * float(cfg["logit_scale"])

"""Typed configuration of the Zegorax architecture: a decoder whose layers are listed one by one in config.json, each
with one of three mixers and a dense or expert-mixture feed-forward (or none), and with a stretch of layers that may run
several times in a row.

    {"architecture": "Zegorax", "vocab": V, "width": h, "max_positions": P, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "diff",
                           "rot": {"base", "dims", "scaling": {"factor", "low", "high", "original"}}},
                 "mlp": null | {"kind": "dense", "ff": F}
                             | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k}}},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "mask": {"size": W},
                           "rot": {"base", "dims"}}, "mlp": ...},
                {"type": "delta",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": ...}, ...]}

`loop`, `rot.scaling`, `mask` and `kv_heads` may be absent (every layer once, plain frequencies, every earlier position
visible, one key head per head).  Every size and constant comes from the file; nothing is read off tensor shapes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import InvalidValue, MissingKey

MIXER_TYPES = ("attention", "latent_attention", "delta")


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key)
    if v is None:
        raise MissingKey(f"{where}.{key}")
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise InvalidValue(f"{where}.{key}", f"expected a positive integer, got {v!r}")
    return int(v)


def _number(d: Mapping[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if v is None:
        raise MissingKey(f"{where}.{key}")
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise InvalidValue(f"{where}.{key}", f"expected a finite number, got {v!r}")
    return float(v)


def _section(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise MissingKey(f"{where}.{key}")
    return v


def _parse_rot(rot: Mapping[str, Any], limit: int, where: str) -> dict:
    dims = rot.get("dims")
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > limit:
        raise InvalidValue(where + ".dims", f"expected an even count of at most {limit} rotated dimensions, got {dims!r}")
    base = _number(rot, "base", where)
    if base <= 0:
        raise InvalidValue(where + ".base", "must be positive")
    out: Dict[str, Any] = {"base": base, "dims": int(dims), "scaling": None}
    sc = rot.get("scaling")
    if sc is not None:
        if not isinstance(sc, Mapping):
            raise InvalidValue(where + ".scaling", f"expected an object, got {sc!r}")
        out["scaling"] = {k: _number(sc, k, where + ".scaling") for k in ("factor", "low", "high", "original")}
        if min(out["scaling"].values()) <= 0 or out["scaling"]["high"] == out["scaling"]["low"]:
            raise InvalidValue(where + ".scaling", "factor, low, high and original must be positive, and high differ from low")
    return out


def _heads(m: Mapping[str, Any], where: str) -> Tuple[int, int]:
    heads = _pos_int(m, "heads", where)
    kv = _pos_int(m, "kv_heads", where) if m.get("kv_heads") is not None else heads
    if heads % kv:
        raise InvalidValue(where + ".kv_heads", f"{heads} heads are no multiple of {kv} key heads")
    return heads, kv


def _parse_mixer(kind: str, m: Mapping[str, Any], where: str) -> dict:
    out: Dict[str, Any] = {"dim": _pos_int(m, "dim", where), "vdim": _pos_int(m, "vdim", where)}
    if kind == "delta":
        out["heads"], out["kv_heads"] = _heads(m, where)
        out["conv"] = _pos_int(m, "conv", where)
        return out
    out["scale"] = _number(m, "scale", where)
    if kind == "attention":
        out["heads"], out["kv_heads"] = _heads(m, where)
        out["diff"] = _number(m, "diff", where)
        out["rot"] = _parse_rot(_section(m, "rot", where), out["dim"], where + ".rot")
        return out
    out["heads"] = _pos_int(m, "heads", where)
    out["q_rank"], out["kv_rank"] = _pos_int(m, "q_rank", where), _pos_int(m, "kv_rank", where)
    out["rot_dim"] = _pos_int(m, "rot_dim", where)
    out["rot"] = _parse_rot(_section(m, "rot", where), out["rot_dim"], where + ".rot")
    mask = m.get("mask")
    out["window"] = None
    if mask is not None:
        if not isinstance(mask, Mapping):
            raise InvalidValue(where + ".mask", f"expected an object, got {mask!r}")
        out["window"] = _pos_int(mask, "size", where + ".mask")
    return out


def _parse_mlp(mlp, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
        raise InvalidValue(where + ".kind", f"expected 'dense' or 'moe', got {mlp!r}")
    if mlp["kind"] == "dense":
        return {"kind": "dense", "ff": _pos_int(mlp, "ff", where)}
    router = _section(mlp, "router", where)
    out = {"kind": "moe", "ff": _pos_int(_section(mlp, "expert", where), "ff", where + ".expert"),
           "experts": _pos_int(router, "experts", where + ".router"), "top": _pos_int(router, "top", where + ".router")}
    if out["top"] > out["experts"]:
        raise InvalidValue(where + ".router.top", f"{out['top']} of {out['experts']} experts")
    return out


@dataclass(frozen=True)
class ZegoraxLayer:
    type: str
    mixer: Any                       # a plain dict of validated sizes and constants
    mlp: Any                         # None, {"kind": "dense", "ff"} or {"kind": "moe", "ff", "experts", "top"}


@dataclass(frozen=True)
class ZegoraxConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: Tuple[ZegoraxLayer, ...]
    loop: Optional[Tuple[int, int, int]] = None         # (start, stop, times)
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Zegorax"

    default_eos_ids = ()

    # names the serving code asks of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def run_order(self) -> Tuple[int, ...]:
        """Layer indices in the order they run: the looped stretch `times` times in a row, the rest once."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        a, b, times = self.loop
        return tuple(range(a)) + tuple(range(a, b)) * times + tuple(range(b, n))

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ZegoraxConfig":
        vocab, width = _pos_int(d, "vocab", "config"), _pos_int(d, "width", "config")
        max_positions = _pos_int(d, "max_positions", "config")
        eps = _number(_section(d, "norm", "config"), "eps", "norm")
        if eps < 0:
            raise InvalidValue("norm.eps", "must be >= 0")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise MissingKey("layers")
        layers = []
        for i, rl in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(rl, Mapping) or rl.get("type") not in MIXER_TYPES:
                raise InvalidValue(where + ".type", f"expected one of {MIXER_TYPES}, got {rl.get('type') if isinstance(rl, Mapping) else rl!r}")
            mixer = _parse_mixer(rl["type"], _section(rl, "mixer", where), where + ".mixer")
            layers.append(ZegoraxLayer(rl["type"], mixer, _parse_mlp(rl.get("mlp"), where + ".mlp")))
        loop = None
        raw_loop = d.get("loop")
        if raw_loop is not None:
            if not isinstance(raw_loop, Mapping):
                raise InvalidValue("loop", f"expected an object, got {raw_loop!r}")
            for k in ("start", "stop"):
                v = raw_loop.get(k)
                if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                    raise InvalidValue(f"loop.{k}", f"expected a layer index, got {v!r}")
            a, b, times = int(raw_loop["start"]), int(raw_loop["stop"]), _pos_int(raw_loop, "times", "loop")
            if not a <= b <= len(layers):
                raise InvalidValue("loop", f"layers {a}..{b - 1} of {len(layers)}")
            loop = (a, b, times)
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos))
        return cls(vocab=vocab, width=width, max_positions=max_positions, norm_eps=eps, layers=tuple(layers), loop=loop,
                   eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "delta":
                mixer = {k: m[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
            else:
                rot: Dict[str, Any] = {"base": m["rot"]["base"], "dims": m["rot"]["dims"]}
                if m["rot"]["scaling"] is not None:
                    rot["scaling"] = dict(m["rot"]["scaling"])
                if l.type == "attention":
                    mixer = {k: m[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale", "diff")}
                else:
                    mixer = {k: m[k] for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale")}
                    if m["window"] is not None:
                        mixer["mask"] = {"size": m["window"]}
                mixer["rot"] = rot
            mlp = None
            if l.mlp is not None and l.mlp["kind"] == "dense":
                mlp = {"kind": "dense", "ff": l.mlp["ff"]}
            elif l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp["ff"]}, "router": {"experts": l.mlp["experts"], "top": l.mlp["top"]}}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "max_positions": self.max_positions, "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

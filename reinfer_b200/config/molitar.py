"""Typed configuration of the Molitar architecture: a decoder whose layers are listed one by one in config.json,
each with one of two attention mixers and a dense gated feed-forward (or none).

    {"architecture": "Molitar", "vocab": V, "width": h, "norm": {"eps": e}, "residual_mult": m, "logit_scale": s,
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale",
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                 "mlp": null | {"kind": "dense", "ff": F}},
                {"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "v_mix",
                           "rot": {"base", "dims"}},
                 "mlp": ...}, ...]}

`rot.scaling`, `softcap`, `v_mix` and `kv_heads` may be absent (no stretching, no cap, no mixing, one key/value head per
query head).  Every size and constant comes from the file; nothing is read off tensor shapes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import InvalidValue, MissingKey

MIXER_TYPES = ("latent_attention", "attention")


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
        out["scaling"] = {k: _number(sc, k, where + ".scaling") for k in ("factor", "original", "fast", "slow")}
        if min(out["scaling"].values()) <= 0:
            raise InvalidValue(where + ".scaling", "factor, original, fast and slow must be positive")
    return out


def _parse_mixer(kind: str, m: Mapping[str, Any], where: str) -> dict:
    out: Dict[str, Any] = {"heads": _pos_int(m, "heads", where), "dim": _pos_int(m, "dim", where),
                           "vdim": _pos_int(m, "vdim", where), "scale": _number(m, "scale", where)}
    if kind == "latent_attention":
        out["q_rank"], out["kv_rank"] = _pos_int(m, "q_rank", where), _pos_int(m, "kv_rank", where)
        out["rot_dim"] = _pos_int(m, "rot_dim", where)
        out["rot"] = _parse_rot(_section(m, "rot", where), out["rot_dim"], where + ".rot")
        return out
    out["kv_heads"] = _pos_int(m, "kv_heads", where) if m.get("kv_heads") is not None else out["heads"]
    if out["heads"] % out["kv_heads"]:
        raise InvalidValue(where + ".kv_heads", f"{out['heads']} query heads are no multiple of {out['kv_heads']} key/value heads")
    out["rot"] = _parse_rot(_section(m, "rot", where), out["dim"], where + ".rot")
    cap = m.get("softcap")
    out["softcap"] = None
    if cap is not None:
        out["softcap"] = _number(m, "softcap", where)
        if out["softcap"] <= 0:
            raise InvalidValue(where + ".softcap", "must be positive (leave it out for no cap)")
    vm = m.get("v_mix", False)
    if not isinstance(vm, bool):
        raise InvalidValue(where + ".v_mix", f"expected true or false, got {vm!r}")
    out["v_mix"] = vm
    return out


def _parse_mlp(mlp, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
        raise InvalidValue(where + ".kind", f"expected 'dense', got {mlp!r}")
    return {"kind": "dense", "ff": _pos_int(mlp, "ff", where)}


@dataclass(frozen=True)
class MolitarLayer:
    type: str
    mixer: Any                       # a plain dict of validated sizes and constants
    mlp: Any                         # None or {"kind": "dense", "ff"}


@dataclass(frozen=True)
class MolitarConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_scale: float
    layers: Tuple[MolitarLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Molitar"

    default_eos_ids = ()

    # names the serving code asks of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def first_value_layer(self) -> Optional[int]:
        """The first layer that mixes values: its own values are what the later such layers mix in."""
        for i, l in enumerate(self.layers):
            if l.type == "attention" and l.mixer["v_mix"]:
                return i
        return None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MolitarConfig":
        vocab, width = _pos_int(d, "vocab", "config"), _pos_int(d, "width", "config")
        eps = _number(_section(d, "norm", "config"), "eps", "norm")
        if eps < 0:
            raise InvalidValue("norm.eps", "must be >= 0")
        mult = _number(d, "residual_mult", "config")
        logit_scale = _number(d, "logit_scale", "config") if d.get("logit_scale") is not None else 1.0
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise MissingKey("layers")
        layers = []
        for i, rl in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(rl, Mapping) or rl.get("type") not in MIXER_TYPES:
                raise InvalidValue(where + ".type", f"expected one of {MIXER_TYPES}, got {rl.get('type') if isinstance(rl, Mapping) else rl!r}")
            mixer = _parse_mixer(rl["type"], _section(rl, "mixer", where), where + ".mixer")
            layers.append(MolitarLayer(rl["type"], mixer, _parse_mlp(rl.get("mlp"), where + ".mlp")))
        first = None
        for i, l in enumerate(layers):
            if l.type == "attention" and l.mixer["v_mix"]:
                size = (l.mixer["kv_heads"], l.mixer["vdim"])
                if first is None:
                    first = (i, size)
                elif size != first[1]:
                    raise InvalidValue(f"layers[{i}].mixer.v_mix", f"layer {i} mixes in the values of layer {first[0]}, whose key/value "
                                                                   f"heads and value size {first[1]} differ from its own {size}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos))
        return cls(vocab=vocab, width=width, norm_eps=eps, residual_mult=mult, logit_scale=logit_scale, layers=tuple(layers),
                   eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            m = l.mixer
            rot: Dict[str, Any] = {"base": m["rot"]["base"], "dims": m["rot"]["dims"]}
            if m["rot"]["scaling"] is not None:
                rot["scaling"] = dict(m["rot"]["scaling"])
            if l.type == "latent_attention":
                mixer = {k: m[k] for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale")}
            else:
                mixer = {k: m[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale")}
                if m["softcap"] is not None:
                    mixer["softcap"] = m["softcap"]
                mixer["v_mix"] = m["v_mix"]
            mixer["rot"] = rot
            layers.append({"type": l.type, "mixer": mixer, "mlp": None if l.mlp is None else dict(l.mlp)})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                               "logit_scale": self.logit_scale, "layers": layers}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

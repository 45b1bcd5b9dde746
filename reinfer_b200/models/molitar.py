"""Molitar as a ModelSpec.  Layers are sandwiches (block `sandwich`): an RMS norm before every sublayer and a second one on
what the sublayer puts out (`rms_out`, which carries the residual multiplier), all with weights stored as their distance from
one.  Per layer one of two mixers - `latent_attention` (keys and values rebuilt from one cached latent vector per token,
stretched pair rotation) or `gated_attention` (biases, partial pair rotation, soft cap, sink, value mixing across layers,
output gate) - and a dense gated feed-forward or none.  The output matrix is the token table; the scale on the logits is
folded into the last norm's weight.  Layer i's tensors start with `l<i>.`.
"""
from __future__ import annotations

from ..config.molitar import MolitarConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def _position(rot: dict) -> dict:
    return {"kind": "rope_pairs", "dims": rot["dims"], "base": rot["base"], "scaling": rot["scaling"]}


def _mixer(cfg: MolitarConfig, index: int, kind: str, m, prefix: str) -> PartSpec:
    if kind == "latent_attention":
        return PartSpec("latent_attention", {"hidden": cfg.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
                                             "vdim": m["vdim"], "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"],
                                             "eps": cfg.norm_eps, "position": _position(m["rot"])}, prefix)
    v_mix = None
    if m["v_mix"]:
        v_mix = "first" if cfg.first_value_layer() == index else "mix"
    return PartSpec("gated_attention", {"hidden": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
                                        "vdim": m["vdim"], "scale": m["scale"], "position": _position(m["rot"]), "bias": True,
                                        "softcap": m["softcap"], "sink": True, "v_mix": v_mix, "gate": True}, prefix)


def build_spec(cfg: MolitarConfig) -> ModelSpec:
    h = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"width": h, "eps": cfg.norm_eps, "weight_name": "", "unit_offset": True}, name)

    def out_norm(name: str) -> PartSpec:
        return PartSpec("rms_out", {"width": h, "eps": cfg.norm_eps, "mult": cfg.residual_mult, "weight_name": "",
                                    "unit_offset": True}, name)

    layers, ignorable = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        roles = dict(mixer_norm=norm(p + "norm1"), mixer=_mixer(cfg, i, l.type, l.mixer, p + "mix."), mixer_out_norm=out_norm(p + "norm1b"))
        if l.mlp is not None:
            roles.update(ffn_norm=norm(p + "norm2"),
                         ffn=PartSpec("swiglu", {"hidden": h, "intermediate": l.mlp["ff"], "names": ("gate", "up", "down")}, p + "mlp."),
                         ffn_out_norm=out_norm(p + "norm2b"))
        else:
            ignorable += [p + "norm2", p + "norm2b"]            # norms nobody reads
        if l.type == "attention" and not l.mixer["v_mix"]:
            ignorable.append(p + "mix.vmix")                    # a mixing weight nobody reads
        layers.append(LayerSpec(f"l{i}", block="sandwich", **roles))
    return ModelSpec(
        hidden_size=h, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": h, "table_name": "embed"}, ""),
        layers=tuple(layers),
        final_norm=PartSpec("rmsnorm", {"width": h, "eps": cfg.norm_eps, "weight_name": "", "unit_offset": True,
                                        "gain": cfg.logit_scale}, "final.norm"),
        lm_head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": h, "tied": True}, ""),
        ignorable_tensors=tuple(ignorable))


def register() -> None:
    register_architecture("Molitar", MolitarConfig, build_spec, aliases=("molitar",))

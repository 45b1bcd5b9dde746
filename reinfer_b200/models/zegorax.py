"""Zegorax as a ModelSpec.  Token table plus a table of learned position vectors; every norm is Dynamic Tanh (tensors
`<name>`, `<name>.b`, `<name>.alpha`); a layer reads ONE norm of the stream and adds mixer and feed-forward at once (block
`parallel`).  Per layer one of three mixers - `diff_attention` (two softmax maps per head, half-split rotation with stretched
slow frequencies, a gate per head), `latent_attention` (one cached latent per token, sliding window, neighbouring-pair
rotation, an elementwise gate) or `head_delta` (the gated delta rule with one decay per head, short convolutions) - and a
feed-forward: dense gated with tanh-gelu and biases, a mixture of gated silu experts routed by their logits, or none.  A
stretch of layers may run several times in a row with the same weights; every run has a cache of its own (the run order
repeats the layers' indices).  The token table is the output matrix.  Layer i's tensors start with `l<i>.`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zegorax import ZegoraxConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def _norm(width: int, name: str) -> PartSpec:
    return PartSpec("dyt", {"width": width, "weight_name": "", "bias_name": ".b", "alpha_name": ".alpha"}, name)


def _mixer(cfg: ZegoraxConfig, kind: str, m, prefix: str) -> PartSpec:
    h, eps = cfg.width, cfg.norm_eps
    if kind == "delta":
        return PartSpec("head_delta", {"hidden": h, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                                       "conv": m["conv"], "eps": eps}, prefix)
    rot = m["rot"]
    if kind == "attention":
        position = {"kind": "rope", "head_dim": m["dim"], "theta": rot["base"], "rotary_dim": rot["dims"], "scaling": rot["scaling"]} \
            if rot["dims"] else None
        return PartSpec("diff_attention", {"hidden": h, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                                           "scale": m["scale"], "diff": m["diff"], "eps": eps, "position": position, "gate": True}, prefix)
    if rot["scaling"] is not None:
        raise ValueError("Zegorax: the latent attention's rotation takes no frequency scaling")
    position = {"kind": "rope_pairs", "dims": rot["dims"], "base": rot["base"], "scaling": None}
    return PartSpec("latent_attention", {"hidden": h, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                                         "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps,
                                         "position": position, "window": m["window"], "gate": True}, prefix)


def _ffn(cfg: ZegoraxConfig, mlp, prefix: str) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("gated_ffn", {"hidden": cfg.width, "intermediate": mlp["ff"], "activation": "gelu_tanh", "bias": True,
                                      "names": ("gate", "up", "down")}, prefix)
    return PartSpec("expert_mixture", {"hidden": cfg.width, "experts": mlp["experts"], "top": mlp["top"], "inner": mlp["ff"],
                                       "expert_names": ("e{}.gate", "e{}.up", "e{}.down"), "router_name": "router",
                                       "correction_name": "router.b", "gated": True, "activation": "silu",
                                       "route": "chosen_logits"}, prefix)


def build_spec(cfg: ZegoraxConfig) -> ModelSpec:
    h = cfg.width
    layers = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        roles = dict(mixer_norm=_norm(h, p + "norm1"), mixer=_mixer(cfg, l.type, l.mixer, p + "mix."))
        if l.mlp is not None:
            roles["ffn"] = _ffn(cfg, l.mlp, p + "mlp.")
        layers.append(LayerSpec(f"l{i}", block="parallel", **roles))
    return ModelSpec(
        hidden_size=h, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": h, "positions": cfg.max_positions,
                                         "table_name": "embed", "positions_name": "pos"}, ""),
        layers=tuple(layers),
        final_norm=_norm(h, "final.norm"),
        lm_head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": h, "tied": True}, "head."),
        order=cfg.run_order())


def register() -> None:
    register_architecture("Zegorax", ZegoraxConfig, build_spec, aliases=("zegorax",))

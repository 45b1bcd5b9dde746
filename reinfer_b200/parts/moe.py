"""A mixture of small feed-forward experts.  Each token uses `top` of `experts + identity` choices:

    s      = softmax(router(x))                  over all choices, 32-bit
    chosen = the `top` largest of s + correction (the correction steers the choice only)
    out    = sum over the chosen e of s[e] * expert_e(x)       (the weights are not renormalised)

An expert is down(act(up(x))) with act = relu(.)^2 and no biases; the last `identity` choices are experts that
hand their input back unchanged and have no tensors.

Two options make the other common form.  `gated=True`: an expert is down(f(gate(x)) * up(x)) with f = `activation`
(silu or the tanh form of gelu), three tensors an expert.  `route="chosen_logits"`: the vector beside the router's matrix
(`correction_name`) is a bias of the logits, the `top` largest logits are chosen and the weights are the softmax over the
chosen logits alone.

Over many tokens (a prompt portion) the stacked products compute every expert for every token where a token uses `top`
of them.  A gated mixture in bfloat16 whose tokens use at most half of the experts then takes the grouped form
(`ops.moe_grouped_experts`): rows sorted by expert on the device, two grouped tensor-core products over the chosen
pairs alone, the weighted sum per token in the order of the experts.  A decode step's few tokens touch most experts
anyway and keep the stacked form.

The experts' up matrices are stacked by rows at load and their down matrices side by side, and the router's choice
is kept dense (gates [T, experts], zero where an expert was not chosen): one product makes every expert's inner
activations, the activation kernel multiplies each by its token's gate, and one product with the stacked down
matrices is then the weighted sum over the chosen experts, an expert that was not chosen adding exact zeros.  A
token's result never depends on what else is in the batch.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import FeedForward, register_part
from .linear import matmul, matmul_into_residual


GROUPED = os.environ.get("REINFER_B200_MOE_GROUPED", "1") != "0"    # 0: the stacked products at every token count
GROUPED_FROM = 256                                                  # tokens of a step from which the grouped form is taken


class ExpertMixture(FeedForward):
    def __init__(self, hidden: int, experts: int, top: int, inner: int, identity: int = 0,
                 expert_names=("e{}.up", "e{}.down"), router_name: str = "router", correction_name: str = "correction",
                 gated: bool = False, activation: str = "silu", route: str = "scores"):
        """expert_names: (up, down), or with `gated` (gate, up, down) - patterns that take the expert's index."""
        self.hidden, self.E, self.I, self.top, self.ff = int(hidden), int(experts), int(identity), int(top), int(inner)
        if self.E < 1 or self.I < 0 or not 1 <= self.top <= self.E + self.I:
            raise ValueError(f"expert mixture: {self.E} experts, {self.I} identity experts, top {self.top}")
        self.gated, self.activation, self.route = bool(gated), activation, route
        if route not in ops.MOE_MODES or (self.gated and activation not in ops.GLU_ACTS):
            raise ValueError(f"expert mixture: route {route!r}, activation {activation!r}")
        if len(expert_names) != (3 if self.gated else 2):
            raise ValueError("expert mixture: tensor names for (gate,) up and down")
        self.gate_name = expert_names[0] if self.gated else None
        self.up_name, self.down_name = expert_names[-2:]
        self.router_name, self.correction_name = router_name, correction_name
        self.w_up = self.w_down = self.w_router = self.correction = None

    def param_specs(self):
        h, n = self.hidden, self.E + self.I
        out = {self.router_name: ParamSpec((n, h), std=0.1), self.correction_name: ParamSpec((n,), std=0.02)}
        for e in range(self.E):
            if self.gated:
                out[self.gate_name.format(e)] = ParamSpec((self.ff, h))
            out[self.up_name.format(e)] = ParamSpec((self.ff, h))
            out[self.down_name.format(e)] = ParamSpec((h, self.ff))
        return out

    def bind(self, t):
        ups = [t[self.up_name.format(e)] for e in range(self.E)]
        if self.gated:
            ups = [t[self.gate_name.format(e)] for e in range(self.E)] + ups     # [all gates; all ups]: one gated pair over E * ff columns
        downs = [t[self.down_name.format(e)] for e in range(self.E)]
        if len({m.dtype for m in ups + downs}) > 1:
            ups, downs = [m.float() for m in ups], [m.float() for m in downs]
        self.w_up = torch.cat(ups, dim=0).contiguous()                  # [E * ff, h]  (gated: [2 * E * ff, h])
        self.w_down = torch.cat(downs, dim=1).contiguous()              # [h, E * ff]
        self.w_router = t[self.router_name]
        self.correction = t[self.correction_name].float().contiguous()

    def forward(self, ctx, xn, residual):
        T = xn.shape[0]
        gates, ident = ops.moe_router(xn, self.w_router, self.correction, self.E, self.top, mode=self.route)     # 32-bit, product and choice
        if self.gated and ident is None and T >= GROUPED_FROM and 2 * self.top <= self.E and GROUPED:
            # (a step of this many tokens is beyond the products that do the next norm's work: nothing is lost by not asking)
            fresh = bool(getattr(ctx, "fresh_residual", False))
            if ops.moe_grouped_experts(xn, gates, self.top, self.w_up, self.w_down, self.ff, self.activation, residual, store=fresh):
                ctx.fresh_residual = False
                return None
        if self.gated:
            act = torch.empty((T, self.E * self.ff), dtype=xn.dtype, device=xn.device)
            # bfloat16: the activation and the expert's weight in the product's epilogue; else 32-bit sums and a kernel behind them
            fused = T and xn.dtype == torch.bfloat16 and self.w_up.dtype == torch.bfloat16 and \
                ops.gemm_bf16_swiglu(xn, self.w_up, act, act=self.activation, gates=gates, ff=self.ff)
            if T and not fused:
                ops.glu_act(matmul(ctx, xn, self.w_up, out_dtype=torch.float32), act, self.activation, None, gates, self.ff)
        else:
            act = ops.relu2_gate(matmul(ctx, xn, self.w_up), gates, self.ff)
        if ident is not None:
            ctx.norm_ahead = None           # the stream is not complete behind the down product: nobody's rows can be made there
        left = matmul_into_residual(ctx, act, self.w_down, residual)
        if ident is not None and T:
            # the identity experts' share: the token's own row times the sum of their chosen scores - left to the
            # block where it adds such a term on its way, else added here
            if getattr(ctx, "takes_row_multiple", False) and getattr(ctx, "row_multiple", None) is None:
                ctx.row_multiple = (ident, xn)
            else:
                ops.rows_axpy(residual if left is None else left[0], ident, xn)
        return left


register_part("ffn", "expert_mixture", ExpertMixture)

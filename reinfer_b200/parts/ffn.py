"""SwiGLU feed-forward: down( silu(x Wg^T) * (x Wu^T) ), no bias
(crates/cuda/src/engine.rs:4288-4314; crates/cuda/kernels/dense_kernels.cu:236-248).
Gate and up rows are concatenated once at load into one `[2F, h]` matrix so that one
product serves both (the reference runs two); in bfloat16 that product keeps two
accumulators and applies the activation in its epilogue."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import FeedForward, RowScaled, register_part
from .linear import matmul, matmul_into_residual, takes_row_scaled


class SwiGLU(FeedForward):
    def __init__(self, hidden: int, intermediate: int, names=("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        """names: the local tensor names of the gate, up and down matrices."""
        self.hidden, self.inter = int(hidden), int(intermediate)
        self.names = tuple(names)
        self.w_gate_up = None
        self.w_down = None

    def param_specs(self):
        g, u, d = self.names
        return {g: ParamSpec((self.inter, self.hidden)),
                u: ParamSpec((self.inter, self.hidden)),
                d: ParamSpec((self.hidden, self.inter))}

    def bind(self, tensors):
        g, u = tensors[self.names[0]], tensors[self.names[1]]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors[self.names[2]]

    @property
    def takes_row_scaled(self) -> bool:
        """The first product (gate and up) can apply the factor of rows that the norm left without it."""
        return takes_row_scaled(self.w_gate_up)

    def forward(self, ctx, xn, residual):
        act = torch.empty((xn.shape[0], self.inter), dtype=xn.dtype, device=xn.device)
        if isinstance(xn, RowScaled):
            if not ops.gemm_bf16_swiglu(xn.rows, self.w_gate_up, act, row_scale=xn.scale()):
                raise ValueError("swiglu: rows without their factor need the tensor-core product")
            return matmul_into_residual(ctx, act, self.w_down, residual)
        fused = xn.dtype == torch.bfloat16 and self.w_gate_up.dtype == torch.bfloat16 and \
            ops.gemm_bf16_swiglu(xn, self.w_gate_up, act)          # activation in the product's epilogue
        if not fused:
            gu = matmul(ctx, xn, self.w_gate_up)
            ops.swiglu(gu, act)
        return matmul_into_residual(ctx, act, self.w_down, residual)


class GatedFFN(FeedForward):
    """down( f(x Wg^T + bg) * (x Wu^T + bu) ) + bd with f = silu or the tanh form of gelu and optional biases on all three
    projections (tensors `<name>.b`).  Gate and up are one product; in bfloat16 its epilogue adds the biases to the 32-bit
    sums, applies f and rounds once (`ops.gemm_bf16_swiglu`), else the product leaves 32-bit sums and `ops.glu_act` does the
    same.  The last bias goes into the stream before the last product, so that the product may
    still do the work of the norm that reads the stream next."""

    def __init__(self, hidden: int, intermediate: int, activation: str = "silu", bias: bool = False,
                 names=("gate_proj.weight", "up_proj.weight", "down_proj.weight"), bias_suffix: str = ".b"):
        self.hidden, self.inter = int(hidden), int(intermediate)
        if activation not in ops.GLU_ACTS:
            raise ValueError(f"gated feed-forward: activation {activation!r} (known: {sorted(ops.GLU_ACTS)})")
        self.activation, self.bias = activation, bool(bias)
        self.names = tuple(names)
        self.bias_names = tuple(n + bias_suffix for n in self.names)
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None

    def param_specs(self):
        g, u, d = self.names
        out = {g: ParamSpec((self.inter, self.hidden)), u: ParamSpec((self.inter, self.hidden)), d: ParamSpec((self.hidden, self.inter))}
        if self.bias:
            bg, bu, bd = self.bias_names
            out.update({bg: ParamSpec((self.inter,), std=0.1), bu: ParamSpec((self.inter,), std=0.1), bd: ParamSpec((self.hidden,), std=0.1)})
        return out

    def bind(self, tensors):
        g, u = tensors[self.names[0]], tensors[self.names[1]]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors[self.names[2]]
        if self.bias:
            self.b_gate_up = torch.cat([tensors[self.bias_names[0]].float(), tensors[self.bias_names[1]].float()]).contiguous()
            self.b_down = tensors[self.bias_names[2]].float().contiguous()

    def forward(self, ctx, xn, residual):
        T = xn.shape[0]
        act = torch.empty((T, self.inter), dtype=xn.dtype, device=xn.device)
        fused = T and xn.dtype == torch.bfloat16 and self.w_gate_up.dtype == torch.bfloat16 and \
            ops.gemm_bf16_swiglu(xn, self.w_gate_up, act, act=self.activation, bias=self.b_gate_up)
        if T and not fused:
            ops.glu_act(matmul(ctx, xn, self.w_gate_up, out_dtype=torch.float32), act, self.activation, self.b_gate_up)
        if self.b_down is None or T == 0:
            return matmul_into_residual(ctx, act, self.w_down, residual)
        if getattr(ctx, "fresh_residual", False):
            # the tensor holds nothing yet: the product stores, the bias follows
            ctx.fresh_residual = False
            matmul(ctx, act, self.w_down, out=residual, accumulate=False)
            ops.add_row_vector(residual, self.b_down)
            return None
        ops.add_row_vector(residual, self.b_down)
        return matmul_into_residual(ctx, act, self.w_down, residual)


register_part("ffn", "swiglu", SwiGLU)
register_part("ffn", "gated_ffn", GatedFFN)

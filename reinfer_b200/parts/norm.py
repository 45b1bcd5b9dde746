"""RMSNorm: x * (1/sqrt(mean(x^2) + eps)) * w, eps inside the root, plain weight,
32-bit arithmetic (crates/cuda/kernels/dense_kernels.cu:59-88; the residual-fused
form :257-296).  Two options serve checkpoints of another convention: `unit_offset` (the tensor
holds the weight's distance from one: the factor is 1 + w) and `gain` (a constant on the output, for
instance a scale on the logits folded into the last norm); either makes the bound weight float32,
formed once at load, so that 1 + w keeps the digits a 16-bit sum would drop."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Norm, PreparedRows, RowScaled, register_part


def effective_weight(w: torch.Tensor, unit_offset: bool, gain: float) -> torch.Tensor:
    """The factor a norm multiplies with: the stored tensor, or (1 + w) * gain as float32."""
    if not unit_offset and gain == 1.0:
        return w
    f = w.float()
    if unit_offset:
        f = f + 1.0
    if gain != 1.0:
        f = f * gain
    return f.contiguous()


class RMSNorm(Norm):
    adds_partial_sums = True            # delta may be a stack [S, rows, width] of partial sums
    leaves_row_scale = True             # forward(..., scaled_ok=True) may return a RowScaled

    def __init__(self, width: int, eps: float, weight_name: str = "weight", unit_offset: bool = False, gain: float = 1.0):
        """weight_name: the local name of the weight ("" where the part's prefix is the tensor's whole name)."""
        self.width, self.eps, self.weight_name = int(width), float(eps), str(weight_name)
        self.unit_offset, self.gain = bool(unit_offset), float(gain)
        self.weight = None

    def param_specs(self):
        return {self.weight_name: ParamSpec((self.width,), init="norm_offset" if self.unit_offset else "norm")}

    def bind(self, tensors):
        self.weight = effective_weight(tensors[self.weight_name], self.unit_offset, self.gain)

    def prepared_by(self, ctx, a, w, residual):
        """residual += a w^T by a product that also makes this norm's rows of the new residual (a decode step's few
        rows, bfloat16): PreparedRows for forward(..., delta=that, scaled_ok=True), or None where that form does not
        apply and nothing was done."""
        if self.weight is None or ctx.dtype != torch.bfloat16 or not ops.DEFER_SUMS or residual.shape[1] != self.width:
            return None
        made = ops.gemm_bf16_residual_norm(a, w, residual, self.weight)
        return None if made is None else PreparedRows(self, made[0], made[1])

    def forward(self, ctx, x, out=None, delta=None, row_idx=None, scaled_ok=False):
        if isinstance(delta, PreparedRows):
            if delta.norm is not self or not scaled_ok or out is not None or row_idx is not None:
                raise ValueError("rmsnorm: rows prepared by a product are for the norm and the reader they were made for")
            return RowScaled(delta.rows, delta.sumsq, self.width, self.eps)
        if scaled_ok and out is None and row_idx is None and ctx.dtype == torch.bfloat16 and ops.DEFER_SUMS and \
                0 < x.shape[0] <= ops.STREAMING_TOKENS and self.width % 4 == 0 and \
                (delta is None or delta.dtype == torch.float32):
            # a decode step's few rows: the division is left to the product that reads them, so that no CTA
            # of this kernel has to wait for a row's whole sum
            y, sumsq = ops.residual_rowscale(x, delta, self.weight)
            return RowScaled(y, sumsq, self.width, self.eps)
        rows = x.shape[0] if row_idx is None else row_idx.numel()
        if out is None:
            out = torch.empty((rows, self.width), dtype=ctx.dtype, device=x.device)
        ops.add_rmsnorm(x, delta, self.weight, out, self.eps, row_idx)
        return out


class ResidualOutNorm(Norm):
    """The norm of a layer that normalises what a sublayer puts OUT, not what it reads:
        x += mult * y / sqrt(mean(y^2) + eps) * w
    in one kernel, 32-bit.  y is the sublayer's output as float32 rows, or the stack of partial sums its last
    product left.  `add` can leave the new x once more, rounded to bfloat16, for the sublayer that reads it next."""
    adds_partial_sums = True

    def __init__(self, width: int, eps: float, mult: float = 1.0, weight_name: str = "weight", unit_offset: bool = False):
        self.width, self.eps, self.mult, self.weight_name = int(width), float(eps), float(mult), str(weight_name)
        self.unit_offset = bool(unit_offset)
        self.weight = None

    def param_specs(self):
        return {self.weight_name: ParamSpec((self.width,), init="norm_offset" if self.unit_offset else "norm")}

    def bind(self, tensors):
        self.weight = effective_weight(tensors[self.weight_name], self.unit_offset, 1.0)

    def add(self, ctx, x, y, rounded=None, extra=None, ahead=None):
        """extra = (a [rows], src [rows, width]): a[r] * src[r] joins y[r] before the norm.  ahead: the norm that reads
        the stream next, for a reader that takes rows without their factor; where its form applies (a decode step's
        few rows, bfloat16) the same kernel leaves that norm's rows and PreparedRows comes back, else None."""
        next_w = None
        if ahead is not None and getattr(ahead, "leaves_row_scale", False) and getattr(ahead, "width", None) == self.width and \
                ahead.weight is not None and ahead.weight.dtype == torch.float32 and ctx.dtype == torch.bfloat16 and ops.DEFER_SUMS and \
                0 < x.shape[0] <= ops.STREAMING_TOKENS and self.width % 4 == 0:
            next_w = ahead.weight
        made = ops.residual_outnorm(x, y, self.weight, self.eps, self.mult, rounded=rounded, extra=extra, next_w=next_w)
        return None if made is None else PreparedRows(ahead, made[0], made[1])

    def forward(self, ctx, x, out=None, delta=None, row_idx=None):
        raise TypeError("an output norm has no rows to hand on: the block calls add(ctx, x, y)")


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "rms_out", ResidualOutNorm)

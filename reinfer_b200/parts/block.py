"""Arrangements of a layer's parts.  A block class is constructed with the layer's parts by
role (`Block(parts: dict role -> part)`), says with `roles` which ones it needs, and runs the
layer on the residual stream in `forward(ctx, x, cache)`.  'prenorm':
    x += mixer(mixer_norm(x));  x += ffn(ffn_norm(x))       (crates/cuda/src/engine.rs:4071-4333)
Mixer and feed-forward add into the residual stream themselves (their last product
accumulates into it), so no separate residual kernel runs.  Either may instead return
what is still to be added (a tensor of x's shape, or a stack [S, T, h] of partial sums):
the block hands it to the norm that reads x next, which adds it on the way; what the
feed-forward leaves is the block's own result, for the norm of the next block."""
from __future__ import annotations

import torch

from .. import ops
from .base import PreparedRows, register_part


def need_roles(block_name: str, parts, roles) -> None:
    missing = [r for r in roles if r not in parts]
    if missing:
        raise ValueError(f"block '{block_name}' needs the roles {list(roles)}; the layer lacks {missing} "
                         f"(it has {list(parts)})")


class PreNormBlock:
    roles = ("mixer_norm", "mixer", "ffn_norm", "ffn")
    hands_on_sums = True                # forward takes and returns what is still to be added to x

    def __init__(self, parts):
        need_roles("prenorm", parts, self.roles)
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = (parts[r] for r in self.roles)

    def forward(self, ctx, x, cache, delta=None):
        """Runs the layer on the residual stream x (in place).  delta: what the block before left to be
        added to x first.  Returns what this block leaves to be added (None: nothing)."""
        xn = _norm(self.mixer_norm, self.mixer, ctx, x, delta)
        after = getattr(ctx, "norm_after_block", None)
        ctx.norm_ahead = self.ffn_norm if _prepares(self.ffn_norm, self.ffn) else None
        try:
            delta = self.mixer.forward(ctx, xn, x, cache)
            xn = _norm(self.ffn_norm, self.ffn, ctx, x, delta)
            ctx.norm_ahead = after
            return self.ffn.forward(ctx, xn, x)
        finally:
            ctx.norm_ahead = None

    def entry_norm(self):
        """The norm that reads the residual stream first in this block, if the part before this block may do that
        norm's work in its last product (else None)."""
        return self.mixer_norm if _prepares(self.mixer_norm, self.mixer) else None


def _prepares(norm, reader) -> bool:
    """Whether a product before `norm` may make the norm's rows itself: the norm knows how and hands rows without
    their factor to a reader that takes them."""
    if not hasattr(norm, "prepared_by"):
        return False
    if getattr(norm, "prepares_complete_rows", False):        # rows that lack nothing: every reader takes them
        return True
    return getattr(norm, "leaves_row_scale", False) and getattr(reader, "takes_row_scaled", False)


def _hands_row_scaled(norm, reader) -> bool:
    """Whether `norm` may hand rows without their factor to `reader`."""
    return bool(getattr(norm, "leaves_row_scale", False) and getattr(reader, "takes_row_scaled", False))


def _norm(norm, reader, ctx, x, delta):
    """The norm before `reader`; rows without their factor only where both sides know of them."""
    if getattr(norm, "leaves_row_scale", False) and getattr(reader, "takes_row_scaled", False):
        return norm.forward(ctx, x, delta=delta, scaled_ok=True)
    return norm.forward(ctx, x, delta=delta)


class PreNormMixerBlock:
    """x += mixer(mixer_norm(x)) and nothing else: a layer without a feed-forward."""
    roles = ("mixer_norm", "mixer")
    hands_on_sums = True

    def __init__(self, parts):
        need_roles("prenorm_mixer", parts, self.roles)
        self.mixer_norm, self.mixer = (parts[r] for r in self.roles)

    def forward(self, ctx, x, cache, delta=None):
        xn = _norm(self.mixer_norm, self.mixer, ctx, x, delta)
        ctx.norm_ahead = getattr(ctx, "norm_after_block", None)
        try:
            return self.mixer.forward(ctx, xn, x, cache)
        finally:
            ctx.norm_ahead = None

    def entry_norm(self):
        return self.mixer_norm if _prepares(self.mixer_norm, self.mixer) else None


class OutNormBlock:
    """x += m * norm1(mixer(x));  x += m * norm2(ffn(x)): the sublayers read the stream itself and the norm (kind
    `rms_out`, which also holds m) sits on what they put out.  A sublayer gets a fresh float32 tensor in the place of
    the residual (`ctx.fresh_residual`: its last product stores there, or leaves partial sums) and the norm's
    kernel adds the normalised rows to x.  In bfloat16 the products read the stream's rounding, which the kernel
    that last wrote the stream leaves beside it (`ctx.rounded_stream`).  The feed-forward is optional."""
    roles = ("mixer", "mixer_norm")
    hands_on_sums = True
    reads_rounded_stream = True

    def __init__(self, parts):
        need_roles("out_norm", parts, self.roles)
        self.mixer, self.mixer_norm = parts["mixer"], parts["mixer_norm"]
        self.ffn, self.ffn_norm = parts.get("ffn"), parts.get("ffn_norm")
        if (self.ffn is None) != (self.ffn_norm is None):
            raise ValueError("block 'out_norm': a feed-forward and its norm come together")
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not hasattr(n, "add"):
                raise ValueError("block 'out_norm' needs norms that add a sublayer's normalised output to the stream (kind 'rms_out')")

    @staticmethod
    def _settle(ctx, x, delta) -> None:
        """What the block before left to be added to x is added now (this block's sublayers read x itself)."""
        if delta is None:
            return
        if isinstance(delta, PreparedRows):
            return                                  # the product that made them has completed x already
        for part in (delta if delta.dim() == 3 else delta.unsqueeze(0)):
            ops.residual_add(x, part.contiguous())
        ctx.rounded_stream = None

    @staticmethod
    def _reads(ctx, x):
        """What a sublayer reads: x in 32-bit, its rounding in bfloat16 (made here if nobody left one)."""
        if ctx.dtype == torch.float32:
            return x
        r = ctx.rounded_stream
        if r is None or r.shape != x.shape:
            r = ops.round_rows(x)
        return r

    def _sublayer(self, ctx, x, norm, run) -> None:
        h = self._reads(ctx, x)
        y = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        ctx.fresh_residual, ctx.norm_ahead = True, None
        ctx.takes_row_multiple, ctx.row_multiple = True, None
        try:
            left = run(h, y)
            if left is None and ctx.fresh_residual and x.shape[0]:
                raise RuntimeError("block 'out_norm': the sublayer did not hand over its output (parts.linear.matmul_into_residual)")
            extra = ctx.row_multiple
        finally:
            ctx.fresh_residual = ctx.takes_row_multiple = False
            ctx.row_multiple = None
        rounded = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if ctx.dtype == torch.bfloat16 else None
        norm.add(ctx, x, y if left is None else left, rounded, extra=extra)
        ctx.rounded_stream = rounded

    def forward(self, ctx, x, cache, delta=None):
        self._settle(ctx, x, delta)
        self._sublayer(ctx, x, self.mixer_norm, lambda h, y: self.mixer.forward(ctx, h, y, cache))
        if self.ffn is not None:
            self._sublayer(ctx, x, self.ffn_norm, lambda h, y: self.ffn.forward(ctx, h, y))
        return None


class SandwichBlock:
    """x += m * out_norm(mixer(norm(x)));  x += m * out_norm'(ffn(norm'(x))): a norm before every sublayer (it reads the
    stream, as in 'prenorm') and another on what the sublayer puts out (kind `rms_out`, which also holds m and adds the
    normalised rows to x, as in 'out_norm').  The sublayer gets a fresh float32 tensor in the place of the residual
    (`ctx.fresh_residual`: its last product stores there, or leaves its partial sums).  Roles: mixer_norm, mixer,
    mixer_out_norm and - together or not at all - ffn_norm, ffn, ffn_out_norm."""
    roles = ("mixer_norm", "mixer", "mixer_out_norm")
    hands_on_sums = True

    def __init__(self, parts):
        need_roles("sandwich", parts, self.roles)
        self.mixer_norm, self.mixer, self.mixer_out_norm = (parts[r] for r in self.roles)
        self.ffn_norm, self.ffn, self.ffn_out_norm = parts.get("ffn_norm"), parts.get("ffn"), parts.get("ffn_out_norm")
        have = [x is not None for x in (self.ffn_norm, self.ffn, self.ffn_out_norm)]
        if any(have) and not all(have):
            raise ValueError("block 'sandwich': a feed-forward comes with the norm before it and the norm behind it")
        for n in (self.mixer_out_norm, self.ffn_out_norm):
            if n is not None and not hasattr(n, "add"):
                raise ValueError("block 'sandwich' needs output norms that add a sublayer's normalised output to the stream (kind 'rms_out')")

    @staticmethod
    def _sublayer(ctx, x, pre, part, post, run, delta=None, ahead=None):
        """ahead: the norm that reads the stream after this sublayer, if its reader takes rows without their factor;
        the output norm's kernel then leaves that norm's rows too (returned, for `delta` of the next sublayer)."""
        xn = _norm(pre, part, ctx, x, delta)
        y = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        ctx.fresh_residual, ctx.norm_ahead = True, None
        try:
            left = run(xn, y)
            if left is None and ctx.fresh_residual and x.shape[0]:
                raise RuntimeError("block 'sandwich': the sublayer did not hand over its output (parts.linear.matmul_into_residual)")
        finally:
            ctx.fresh_residual = False
        return post.add(ctx, x, y if left is None else left, None, ahead=ahead)

    def entry_norm(self):
        """The norm a block before this one may prepare (rows without their factor, which the mixer takes)."""
        return self.mixer_norm if _hands_row_scaled(self.mixer_norm, self.mixer) else None

    def forward(self, ctx, x, cache, delta=None):
        if isinstance(delta, PreparedRows) and delta.norm is not self.mixer_norm:
            delta = None                            # rows made for another norm; the product that made them has completed x already
        after = getattr(ctx, "norm_after_block", None)
        if self.ffn is None:
            return self._sublayer(ctx, x, self.mixer_norm, self.mixer, self.mixer_out_norm,
                                  lambda h, y: self.mixer.forward(ctx, h, y, cache), delta, ahead=after)
        ahead = self.ffn_norm if _hands_row_scaled(self.ffn_norm, self.ffn) else None
        made = self._sublayer(ctx, x, self.mixer_norm, self.mixer, self.mixer_out_norm,
                              lambda h, y: self.mixer.forward(ctx, h, y, cache), delta, ahead=ahead)
        return self._sublayer(ctx, x, self.ffn_norm, self.ffn, self.ffn_out_norm, lambda h, y: self.ffn.forward(ctx, h, y), made, ahead=after)


class ParallelBlock:
    """h = norm(x);  x += mixer(h) + ffn(h): ONE norm, and both sublayers read its rows.  The feed-forward is optional.
    The mixer adds into the stream itself (nothing of it may be left to a later norm: the feed-forward's last product
    has to see the stream with the mixer's share in it, where it does the next norm's work); what the feed-forward
    leaves is the block's own result."""
    roles = ("mixer_norm", "mixer")
    hands_on_sums = True

    def __init__(self, parts):
        need_roles("parallel", parts, self.roles)
        self.norm, self.mixer, self.ffn = parts["mixer_norm"], parts["mixer"], parts.get("ffn")

    def forward(self, ctx, x, cache, delta=None):
        h = self.norm.forward(ctx, x, delta=delta)
        after = getattr(ctx, "norm_after_block", None)
        if self.ffn is None:
            ctx.norm_ahead = after
            try:
                return self.mixer.forward(ctx, h, x, cache)
            finally:
                ctx.norm_ahead = None
        defer = ctx.defer_residual
        ctx.defer_residual, ctx.norm_ahead = False, None
        try:
            left = self.mixer.forward(ctx, h, x, cache)
        finally:
            ctx.defer_residual = defer
        if left is not None:                        # a mixer that hands its sum on all the same
            for part in (left if left.dim() == 3 else left.unsqueeze(0)):
                ops.residual_add(x, part.contiguous())
        ctx.norm_ahead = after
        try:
            return self.ffn.forward(ctx, h, x)
        finally:
            ctx.norm_ahead = None

    def entry_norm(self):
        return self.norm if getattr(self.norm, "prepares_complete_rows", False) and hasattr(self.norm, "prepared_by") else None


register_part("block", "parallel", ParallelBlock)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "prenorm", PreNormBlock)
register_part("block", "out_norm", OutNormBlock)
register_part("block", "prenorm_mixer", PreNormMixerBlock)

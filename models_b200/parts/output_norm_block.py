"""A layer whose norms sit on the sublayers' results, with a learned scale per channel:

    x += mixer_scale * mixer_norm(mixer(x));      x += feed_forward_scale * feed_forward_norm(feed_forward(x))

The sublayers read x itself (in the compute type: one kernel stores the stream's rows that way, and from then on the kernel
that adds a sublayer's result also leaves the new rows in that type for the next reader).  A sublayer hands over float32
rows of the model's width -- the float32 sums of its last product -- or, as a pair of mixers with an RMS norm each
(`forward_pair`), two of them; norm, scale, the pair's mean and the addition into the float32 stream are ONE kernel.  The
norm is a layer norm with a gain and no bias.

A sublayer is a part with `forward_wide` (float32 rows), a split part (a first product, something in between, a last
product), or a pair with `forward_pair`.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part, RunContext, StreamRows, as_delta
from .linear import linear
from .registry import build_part, register_part


class OutputNormBlock(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = build_part("norm", spec.feed_forward_norm, runtime)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime)
        self.parts = [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]
        for part in (self.mixer, self.feed_forward):
            if part is not None and not any(hasattr(part, name) for name in ("forward_pair", "forward_wide")) \
                    and not all(hasattr(part, name) for name in ("input_matrix", "output_matrix", "inner")):
                raise ValueError(f"{type(part).__name__} is neither a split part nor one with float32 results: this block cannot run it")
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and (getattr(norm.spec, "kind", None) != "layernorm" or getattr(norm.spec, "bias", True)):
                raise ValueError("this block's norms are layer norms with a gain and no bias")
        self.width = spec.mixer_norm.size

    def _scales(self):
        return ["mixer_scale"] + (["feed_forward_scale"] if self.feed_forward is not None else [])

    def parameters(self):
        out = [p for part in self.parts for p in part.parameters()]
        return out + [ParamRequest(self.spec.weights[name], (self.width,), "gain") for name in self._scales()]

    def load(self, tensors):
        for part in self.parts:
            part.load(tensors)
        self.scales = {name: self.runtime.vector(tensors[self.spec.weights[name]]) for name in self._scales()}

    def _sublayer(self, x, xn, part, norm, scale, batch, run, copy):
        """x += scale * norm(part(xn)); returns the new rows of x in the compute type if `copy`."""
        copy_dtype = self.runtime.compute_dtype if copy else None
        if hasattr(part, "forward_pair"):
            a, b, gain_a, gain_b = part.forward_pair(xn, batch, run)
            return ops.outnorm_add(x, a, norm.weight, scale, norm.spec.eps, b=b, gain_a=gain_a, gain_b=gain_b, copy_dtype=copy_dtype)
        if hasattr(part, "forward_wide"):
            y = part.forward_wide(xn, batch, run)
        else:
            dtype = self.runtime.compute_dtype
            w_out = part.output_matrix()
            proj = linear(xn, part.input_matrix(), dtype)
            mid = torch.empty((xn.shape[0], w_out.shape[1]), dtype=dtype, device=xn.device)
            part.inner(proj[:, :part.input_matrix().shape[0]], mid, batch, run, 1.0)
            y = linear(mid, w_out, torch.float32)
        return ops.outnorm_add(x, y, norm.weight, scale, norm.spec.eps, copy_dtype=copy_dtype)

    def forward(self, x: torch.Tensor, pending, batch, run: RunContext, following=None):
        """`pending`: None, a delta still to be added, or the stream's rows in the compute type that the block before left for
        this one (a StreamRows).  `following`: the block that runs next; if it is one of these, it is handed the rows."""
        rows = None
        if isinstance(pending, StreamRows):
            rows = pending.rows if pending.reader is self else None
        elif as_delta(pending) is not None:
            ops.residual_add(x, as_delta(pending))
        float_mode = self.runtime.compute_dtype == torch.float32
        if rows is None:
            rows = x if float_mode else ops.store_rows(x, self.runtime.compute_dtype)
        # (in the 32-bit mode the sublayers read the stream itself: nothing is copied; a sublayer is done reading before the add)
        hand_on = isinstance(following, OutputNormBlock) and not float_mode
        has_ff = self.feed_forward is not None
        rows = self._sublayer(x, rows, self.mixer, self.mixer_norm, self.scales["mixer_scale"], batch, run,
                              copy=not float_mode and (has_ff or hand_on))
        if has_ff:
            rows = self._sublayer(x, x if float_mode else rows, self.feed_forward, self.feed_forward_norm,
                                  self.scales["feed_forward_scale"], batch, run, copy=hand_on)
        return StreamRows(rows, following) if hand_on else None


OutputNormBlock.takes_next_block = True  # `forward` is told which block runs next
register_part("block", "output_norm", OutputNormBlock)

"""A pre-norm layer over several copies of the residual stream (hyper-connections).

The stream is x [tokens, streams * width] float32, copy s in columns s * width .. (s + 1) * width.  For the mixer and
then, if the layer has one, the feed-forward, with that sublayer's learned numbers in [streams], out [streams] and
mix [streams, streams] (indexed [from, to]):

    u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y   (all t at once, from the old copies)

Reading (the weighted sum and the RMS norm) is one kernel, writing (the mixing and the addition) another, and a writing
with the reading that follows it (the feed-forward's, or the next block's) a third that passes over the copies once; y reaches the writing kernel as the
float32 sums of the sublayer's last product, in both modes.  With `streams` 0 there is one stream
and no such numbers: x += sublayer(norm(x)), the addition riding in the last product where its kernel takes it.

A sublayer is a split part (a first product, something in between, a last product) or a part that offers
`forward_wide` (float32 rows of the model's width).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part, RunContext, StreamsRead, as_delta
from .linear import add_linear, linear
from .registry import build_part, register_part


class HyperBlock(Part):
    takes_next_block = True  # `forward` is told which block runs next

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
            if part is not None and not hasattr(part, "forward_wide") \
                    and not all(hasattr(part, name) for name in ("input_matrix", "output_matrix", "inner")):
                raise ValueError(f"{type(part).__name__} is neither a split part nor one with float32 results: this block cannot run it")
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and spec.streams and not getattr(norm, "foldable", False):
                raise ValueError(f"{type(norm).__name__} cannot ride in the kernel that reads the streams")
        self.width = spec.mixer_norm.size
        self.streams = spec.streams

    def _sublayers(self):
        return ("mixer", "feed_forward") if self.feed_forward is not None else ("mixer",)

    def parameters(self):
        out = [p for part in self.parts for p in part.parameters()]
        n, S = self.spec.weights, self.streams
        if S:
            for which in self._sublayers():
                out += [ParamRequest(n[which + "_in"], (S,), "gain"), ParamRequest(n[which + "_out"], (S,), "gain"),
                        ParamRequest(n[which + "_mix"], (S, S), "gain")]
        return out

    def load(self, tensors):
        for part in self.parts:
            part.load(tensors)
        n, rt = self.spec.weights, self.runtime
        self.connections = {}
        if self.streams:
            if self.streams > ops.hyper_max_streams() and rt.device.type == "cuda":
                raise ValueError(f"{self.streams} streams exceed the kernels' {ops.hyper_max_streams()}")
            for which in self._sublayers():
                self.connections[which] = tuple(rt.vector(tensors[n[f"{which}_{r}"]]) for r in ("in", "out", "mix"))

    def _result(self, part, xn, batch, run) -> torch.Tensor:
        """The sublayer's result as float32 rows."""
        if hasattr(part, "forward_wide"):
            return part.forward_wide(xn, batch, run)
        mid = self._middle(part, xn, batch, run)
        return linear(mid, part.output_matrix(), torch.float32)

    def _middle(self, part, xn, batch, run) -> torch.Tensor:
        dtype = self.runtime.compute_dtype
        w_out = part.output_matrix()
        proj = linear(xn, part.input_matrix(), dtype)
        mid = torch.empty((xn.shape[0], w_out.shape[1]), dtype=dtype, device=xn.device)
        part.inner(proj, mid, batch, run, 1.0)
        return mid

    def _sublayer(self, x, which, norm, part, batch, run):
        if self.streams:
            read, out, mix = self.connections[which]
            xn = ops.hyper_read_norm(x, read, norm.weight, norm.spec.eps, self.runtime.compute_dtype)
            ops.hyper_write(x, self._result(part, xn, batch, run), out, mix)
            return
        xn = norm.forward(x, None)
        if hasattr(part, "forward_wide"):
            ops.residual_add(x, part.forward_wide(xn, batch, run))
        else:
            add_linear(x, self._middle(part, xn, batch, run), part.output_matrix())

    def forward(self, x: torch.Tensor, pending, batch, run: RunContext, following=None):
        """`pending`: None, or a StreamsRead that the block before took for this one.  `following`: the block that runs next."""
        if isinstance(pending, StreamsRead) and pending.reader is not self:
            pending = None  # (somebody else's reading: the copies are up to date all the same)
        if as_delta(pending) is not None:
            raise RuntimeError("a block over several streams takes no pending delta: the block before it must have added its own")
        if not self.streams:
            self._sublayer(x, "mixer", self.mixer_norm, self.mixer, batch, run)
            if self.feed_forward is not None:
                self._sublayer(x, "feed_forward", self.feed_forward_norm, self.feed_forward, batch, run)
            return None
        # Every writing but the model's last passes over the copies together with the reading that follows it (the
        # feed-forward's, or the next block's mixer's): one kernel, the same bits as the two.
        dtype = self.runtime.compute_dtype
        read, out, mix = self.connections["mixer"]
        if isinstance(pending, StreamsRead):
            xn = pending.rows
        else:
            xn = ops.hyper_read_norm(x, read, self.mixer_norm.weight, self.mixer_norm.spec.eps, dtype)
        y = self._result(self.mixer, xn, batch, run)
        if self.feed_forward is not None:
            norm = self.feed_forward_norm
            read, out_ff, mix_ff = self.connections["feed_forward"]
            xn = ops.hyper_write_read_norm(x, y, out, mix, read, norm.weight, norm.spec.eps, dtype)
            y, out, mix = self._result(self.feed_forward, xn, batch, run), out_ff, mix_ff
        if isinstance(following, HyperBlock) and following.streams == self.streams:
            norm = following.mixer_norm
            rows = ops.hyper_write_read_norm(x, y, out, mix, following.connections["mixer"][0], norm.weight, norm.spec.eps, dtype)
            return StreamsRead(rows, following)
        ops.hyper_write(x, y, out, mix)
        return None


register_part("block", "prenorm_hyper", HyperBlock)

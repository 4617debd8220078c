"""Two mixers on the same rows whose results are RMS-normed over the model's width and averaged:

    1/2 (left(xn) / rms(left(xn)) * gain_left + right(xn) / rms(right(xn)) * gain_right),   rms(v) = sqrt(mean(v^2) + eps)

Both are split parts (parts/split.py): their first matrices are stacked into ONE product; each then turns its columns of that
result into the input of its own last product, whose float32 sums are what the norms read.  `forward_pair` hands the two
float32 results and the gains to a block that folds norms and mean into its own kernel; `forward_wide` does them here.  At most
one of the two may ask for keys and values, and at most one for per-sequence state: a run of the schedule owns one of each.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Mixer, RunContext
from .linear import linear, stack_rows
from .registry import build_part, register_part


class NormedPairMixer(Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.left = build_part("mixer", spec.left, runtime)
        self.right = build_part("mixer", spec.right, runtime)
        for side in (self.left, self.right):
            if not all(hasattr(side, name) for name in ("input_matrix", "output_matrix", "inner")):
                raise ValueError(f"{type(side).__name__} is no split part: it cannot stand beside another mixer")
        if self.left.kv_request() is not None and self.right.kv_request() is not None:
            raise ValueError("both mixers ask for keys and values; a run owns one cache")
        if self.left.state_request() is not None and self.right.state_request() is not None:
            raise ValueError("both mixers ask for per-sequence state; a run owns one state")

    def parameters(self):
        n, W = self.spec.weights, self.spec.hidden_size
        return self.left.parameters() + self.right.parameters() + [ParamRequest(n["left"], (W,), "gain"), ParamRequest(n["right"], (W,), "gain")]

    def load(self, tensors):
        self.left.load(tensors)
        self.right.load(tensors)
        first = [self.left.input_matrix(), self.right.input_matrix()]
        if first[0].dtype != first[1].dtype:
            first = [m.float() for m in first]
        self.w_in, self.in_starts = stack_rows(first)
        self.in_widths = [m.shape[0] for m in first]
        n = self.spec.weights
        self.gains = (self.runtime.vector(tensors[n["left"]]), self.runtime.vector(tensors[n["right"]]))

    def kv_request(self):
        return self.left.kv_request() or self.right.kv_request()

    def state_request(self):
        return self.left.state_request() or self.right.state_request()

    def decode_class(self, sequences: int, max_kv_len: int):
        return tuple(side.decode_class(sequences, max_kv_len) if hasattr(side, "decode_class") else 0
                     for side in (self.left, self.right))

    def forward_pair(self, xn: torch.Tensor, batch, run: RunContext):
        """(left result, right result, left gain, right gain): float32 [T, width] each, before norms and mean."""
        dtype = self.runtime.compute_dtype
        proj = linear(xn, self.w_in, dtype)
        results = []
        for side, at, n in zip((self.left, self.right), self.in_starts, self.in_widths):
            w_out = side.output_matrix()
            mid = torch.empty((xn.shape[0], w_out.shape[1]), dtype=dtype, device=xn.device)
            side.inner(proj[:, at:at + n], mid, batch, run, 1.0)
            results.append(linear(mid, w_out, torch.float32))
        return results[0], results[1], self.gains[0], self.gains[1]

    def forward_wide(self, xn: torch.Tensor, batch, run: RunContext) -> torch.Tensor:
        a, b, gain_a, gain_b = self.forward_pair(xn, batch, run)
        return ops.pair_norm_mean(a, b, gain_a, gain_b, self.spec.eps)

    def forward(self, xn: torch.Tensor, batch, run: RunContext) -> torch.Tensor:
        out = self.forward_wide(xn, batch, run)
        return out if self.runtime.compute_dtype == torch.float32 else out.to(self.runtime.compute_dtype)


register_part("mixer", "normed_pair", NormedPairMixer)

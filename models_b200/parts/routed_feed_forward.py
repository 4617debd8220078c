"""A mixture of experts: every token uses the `top` experts with the largest router logits.

Router logits z = R.xn are float32 sums; the chosen experts' weights are the softmax over the chosen logits only.  An expert
is a gated feed-forward with clamped branches, g = min(Wg.xn, limit), u = clamp(Wu.xn, -limit, limit),
Wd.(g * sigmoid(slope * g) * (u + 1)).  A shared expert of the same form (sizes and limit of its own) runs for every token
and is added multiplied by sigmoid(w.xn), one number per token.

The step's (token, choice) entries are sorted by expert on the device; the experts' two products are then grouped products
over the sorted rows (a block a tile of one expert's rows), whose grids depend on the number of tokens only -- nothing comes
back to the host, so a step can be captured.  A prompt with enough rows per expert pads every expert's rows to whole tiles
of 128 and runs both products as grouped tcgen05 products (bfloat16 weights).  A step of few entries (decoding) skips the sorting: every entry streams its
expert's matrices through a kernel of dot products, which is what the memory allows at that size.  The shared expert's gate, up and score rows are one dense product.  The result
is float32 [tokens, width]: the weighted sum of the chosen experts' float32 results plus the shared expert's.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Part
from .linear import linear, stack_rows
from .registry import register_part


class RoutedFeedForward(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if not 1 <= spec.top <= spec.num_experts:
            raise ValueError(f"top {spec.top} of {spec.num_experts} experts")

    def _expert_names(self, role: str):
        return [self.spec.weights["expert_" + role].format(expert=e) for e in range(self.spec.num_experts)]

    def parameters(self):
        s, n = self.spec, self.spec.weights
        ff, W = s.expert.intermediate_size, s.hidden_size
        out = [ParamRequest(n["router"], (s.num_experts, W))]
        for role, shape in (("gate", (ff, W)), ("up", (ff, W)), ("down", (W, ff))):
            out += [ParamRequest(name, shape) for name in self._expert_names(role)]
        if s.shared is not None:
            f = s.shared.intermediate_size
            out += [ParamRequest(n["shared_gate"], (f, W)), ParamRequest(n["shared_up"], (f, W)),
                    ParamRequest(n["shared_down"], (W, f)), ParamRequest(n["shared_gate_score"], (1, W))]
        return out

    def load(self, tensors):
        s, n, rt = self.spec, self.spec.weights, self.runtime
        self.router = rt.matrix(tensors[n["router"]])
        stacked = {}
        for role in ("gate", "up", "down"):
            parts = [rt.matrix(tensors[name]) for name in self._expert_names(role)]
            if len({m.dtype for m in parts}) > 1:
                parts = [m.float() for m in parts]
            stacked[role] = torch.stack(parts, dim=0).contiguous()
        if len({m.dtype for m in stacked.values()} | {self.router.dtype}) > 1:
            stacked = {r: m.float() for r, m in stacked.items()}
            self.router = self.router.float()
        # gate and up matrices in one buffer (all experts' gate rows, then all up rows): the grouped tensor-core product
        # reads both through one map
        self.w_gate_up = torch.stack([stacked["gate"], stacked["up"]], dim=0).contiguous()
        self.w_gate, self.w_up, self.w_down = self.w_gate_up[0], self.w_gate_up[1], stacked["down"]
        self.grouped = self.w_gate_up.is_cuda and ops.grouped_product_takes(self.w_gate_up, self.w_down)
        self.shared_in = None
        if s.shared is not None:
            first = [rt.matrix(tensors[n[r]]) for r in ("shared_gate", "shared_up", "shared_gate_score")]
            if len({m.dtype for m in first}) > 1:
                first = [m.float() for m in first]
            self.shared_in, self.shared_starts = stack_rows(first)
            self.shared_down = rt.matrix(tensors[n["shared_down"]])

    def forward_wide(self, xn: torch.Tensor, batch=None, run=None) -> torch.Tensor:
        """float32 [tokens, width]."""
        s = self.spec
        x = xn if xn.dtype == self.router.dtype else xn.to(self.router.dtype)
        chosen, weights = ops.router_topk(x, self.router, s.top)
        position = None
        if chosen.numel() <= ops.EXPERT_ROWS_ENTRIES:
            # a decode step: every entry streams its expert's matrices; no sorting, no tiles of mostly empty rows
            mid = ops.expert_rows_first(x, self.w_gate, self.w_up, chosen, s.expert.limit, s.expert.swish_slope)
            slot_out = ops.expert_rows_second(mid, self.w_down, chosen)
        elif self.grouped and chosen.numel() >= ops.GROUPED_ROWS_PER_EXPERT * s.num_experts:
            # a prompt: every expert's rows fill tiles of their own, and both products run on the tcgen05 tensor cores
            plan = ops.route_pad(chosen, s.num_experts)
            mid = ops.grouped_first_product(ops.gather_rows(x, plan), self.w_gate_up, plan, s.expert.limit, s.expert.swish_slope)
            slot_out, position = ops.grouped_second_product(mid, self.w_down, plan), plan.position
        else:
            plan = ops.route_sort(chosen, s.num_experts)
            mid = ops.expert_first_product(x, self.w_gate, self.w_up, plan, s.expert.limit, s.expert.swish_slope)
            slot_out = ops.expert_second_product(mid, self.w_down, plan)
        if self.shared_in is None:
            return ops.expert_combine(slot_out, weights, position=position)
        dtype = self.runtime.compute_dtype
        proj = linear(xn, self.shared_in, dtype)
        f, at = s.shared.intermediate_size, self.shared_starts
        shared_mid = torch.empty((xn.shape[0], f), dtype=dtype, device=xn.device)
        ops.clamped_swish(proj[:, at[0]:at[0] + f], proj[:, at[1]:at[1] + f], shared_mid, s.shared.limit, s.shared.swish_slope)
        shared = linear(shared_mid, self.shared_down, torch.float32)
        return ops.expert_combine(slot_out, weights, shared, proj[:, at[2]:at[2] + 1], position)

    def forward(self, xn: torch.Tensor, batch=None, run=None) -> torch.Tensor:
        out = self.forward_wide(xn, batch, run)
        return out if self.runtime.compute_dtype == torch.float32 else out.to(self.runtime.compute_dtype)


register_part("feed_forward", "routed", RoutedFeedForward)

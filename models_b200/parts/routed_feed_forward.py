"""A mixture of experts: every token uses the `top` experts with the largest router logits.

Router logits z = R.xn are float32 sums; the chosen experts' weights are the softmax over the chosen logits only.  An expert
is a gated feed-forward with clamped branches, g = min(Wg.xn, limit), u = clamp(Wu.xn, -limit, limit),
Wd.(g * sigmoid(slope * g) * (u + 1)).  A shared expert of the same form (sizes and limit of its own) runs for every token
and is added multiplied by sigmoid(w.xn), one number per token.

Variations the spec may ask for.  A "scored" rule: the scores s = softmax(z) run over ALL router outputs, the choice runs on
s + correction (a tensor), restricted to the outputs of the `keep_groups` best of `groups` equal groups of neighbouring outputs
(a group counts by its largest choice score), and the weights are weight_scale * s of the chosen, not renormalised.  Identity
experts: the router's last outputs stand for experts without tensors whose result is their input; their entries skip both
products and enter the weighted sum as the token's own row.  An expert without clamps and without the one added to the up
branch (limit +inf, slope 1, up_offset 0: silu(g) * u).  A shared expert that is added as it is, without a gate.

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
        self.outputs = spec.num_experts + spec.identity_experts  # what the router has: experts, then identity experts
        if not 1 <= spec.top <= self.outputs:
            raise ValueError(f"top {spec.top} of {self.outputs} router outputs")
        if spec.rule not in ("top_logits", "scored"):
            raise ValueError(f"router rule {spec.rule!r} is not built (known: top_logits, scored)")
        if spec.rule != "scored" and (spec.correction or spec.groups != 1 or spec.weight_scale != 1.0):
            raise ValueError("a correction, groups and a weight scale belong to the scored rule")
        if self.outputs % spec.groups or not 1 <= spec.keep_groups <= spec.groups:
            raise ValueError(f"{spec.groups} groups (keeping {spec.keep_groups}) do not cut {self.outputs} router outputs evenly")

    def _expert_names(self, role: str):
        return [self.spec.weights["expert_" + role].format(expert=e) for e in range(self.spec.num_experts)]

    def parameters(self):
        s, n = self.spec, self.spec.weights
        ff, W = s.expert.intermediate_size, s.hidden_size
        out = [ParamRequest(n["router"], (self.outputs, W))]
        if s.correction:
            out.append(ParamRequest(n["correction"], (self.outputs,), "bias"))
        for role, shape in (("gate", (ff, W)), ("up", (ff, W)), ("down", (W, ff))):
            out += [ParamRequest(name, shape) for name in self._expert_names(role)]
        if s.shared is not None:
            f = s.shared.intermediate_size
            out += [ParamRequest(n["shared_gate"], (f, W)), ParamRequest(n["shared_up"], (f, W)),
                    ParamRequest(n["shared_down"], (W, f))]
            if s.shared_gated:
                out.append(ParamRequest(n["shared_gate_score"], (1, W)))
        return out

    def load(self, tensors):
        s, n, rt = self.spec, self.spec.weights, self.runtime
        self.router = rt.matrix(tensors[n["router"]])
        self.correction = rt.vector(tensors[n["correction"]]) if s.correction else None
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
            first = [rt.matrix(tensors[n[r]]) for r in ("shared_gate", "shared_up") + (("shared_gate_score",) if s.shared_gated else ())]
            if len({m.dtype for m in first}) > 1:
                first = [m.float() for m in first]
            self.shared_in, self.shared_starts = stack_rows(first)
            self.shared_down = rt.matrix(tensors[n["shared_down"]])

    def forward_wide(self, xn: torch.Tensor, batch=None, run=None) -> torch.Tensor:
        """float32 [tokens, width]."""
        s = self.spec
        e = s.expert
        x = xn if xn.dtype == self.router.dtype else xn.to(self.router.dtype)
        chosen, weights = ops.router_topk(x, self.router, s.top, scored=s.rule == "scored", correction=self.correction,
                                          groups=s.groups, keep=s.keep_groups, weight_scale=s.weight_scale)
        position = None
        # (an identity expert's id lies beyond the experts': the sorting and the products leave its entries out, and the
        # weighted sum takes the token's own row for them)
        if chosen.numel() <= ops.EXPERT_ROWS_ENTRIES:
            # a decode step: every entry streams its expert's matrices; no sorting, no tiles of mostly empty rows
            mid = ops.expert_rows_first(x, self.w_gate, self.w_up, chosen, e.limit, e.swish_slope, e.up_offset)
            slot_out = ops.expert_rows_second(mid, self.w_down, chosen)
        elif self.grouped and chosen.numel() >= ops.GROUPED_ROWS_PER_EXPERT * s.num_experts:
            # a prompt: every expert's rows fill tiles of their own, and both products run on the tcgen05 tensor cores
            plan = ops.route_pad(chosen, s.num_experts)
            mid = ops.grouped_first_product(ops.gather_rows(x, plan), self.w_gate_up, plan, e.limit, e.swish_slope, e.up_offset)
            slot_out, position = ops.grouped_second_product(mid, self.w_down, plan), plan.position
        else:
            plan = ops.route_sort(chosen, s.num_experts)
            mid = ops.expert_first_product(x, self.w_gate, self.w_up, plan, e.limit, e.swish_slope, up_offset=e.up_offset)
            slot_out = ops.expert_second_product(mid, self.w_down, plan)
        identity = dict(chosen=chosen, experts=s.num_experts, rows=x) if s.identity_experts else {}
        if self.shared_in is None:
            return ops.expert_combine(slot_out, weights, position=position, **identity)
        dtype = self.runtime.compute_dtype
        proj = linear(xn, self.shared_in, dtype)
        f, at = s.shared.intermediate_size, self.shared_starts
        shared_mid = torch.empty((xn.shape[0], f), dtype=dtype, device=xn.device)
        ops.clamped_swish(proj[:, at[0]:at[0] + f], proj[:, at[1]:at[1] + f], shared_mid, s.shared.limit, s.shared.swish_slope,
                          s.shared.up_offset)
        shared = linear(shared_mid, self.shared_down, torch.float32)
        score = proj[:, at[2]:at[2] + 1] if s.shared_gated else None
        return ops.expert_combine(slot_out, weights, shared, score, position, **identity)

    def forward(self, xn: torch.Tensor, batch=None, run=None) -> torch.Tensor:
        out = self.forward_wide(xn, batch, run)
        return out if self.runtime.compute_dtype == torch.float32 else out.to(self.runtime.compute_dtype)


register_part("feed_forward", "routed", RoutedFeedForward)

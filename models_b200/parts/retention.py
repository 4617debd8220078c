"""Retention: linear attention with a fixed decay per head, no softmax and no denominator.

q = Wq.xn, k = Wk.xn (heads of `head_dim`), v = Wv.xn (heads of `value_dim`); q and k are rotated over the first
coordinates of every head (the spec's `position`), k is then multiplied by `key_scale`; per head
S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t; every head's o_t is divided by its root mean square, the heads
side by side are multiplied by silu(Wg.xn), then Wo.  The state S is float32 [heads, head_dim, value_dim] per sequence in
the engine's state area (zero when a sequence starts); the mixer keeps no keys or values.  Everything between the first
products and the last one is float32 arithmetic in both modes.

Variations the spec may ask for: q, k and v pass an activation as they leave their products (`input_activation`); instead
of every head's own root mean square, the heads side by side pass ONE RMS norm with a gain tensor (`norm` "all"); the
gate's activation is a sigmoid instead of a silu (`gate_activation`).  With these and no rotation the mixer is lightning
attention: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t over silu'd projections, normed together, sigmoid-gated.
"""

from __future__ import annotations

import torch

from ..cache.state import StateRequest
from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Mixer, RunContext
from .linear import stack_rows
from .registry import build_part, register_part
from .split import SplitPart


class RetentionMixer(SplitPart, Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if len(spec.decay) != spec.num_heads:
            raise ValueError(f"{len(spec.decay)} decays for {spec.num_heads} heads")
        self.qk_width = spec.num_heads * spec.head_dim
        self.v_width = spec.num_heads * spec.value_dim
        self.position = None
        if spec.position is not None:
            if spec.position.rotary_dim > spec.head_dim:
                raise ValueError(f"rotary_dim {spec.position.rotary_dim} exceeds head_dim {spec.head_dim}")
            if spec.position.pairing != "half":
                raise ValueError("this mixer rotates split-half pairs only")
            key = ("position", spec.position, runtime.max_positions)
            if key not in runtime.shared:
                runtime.shared[key] = build_part("position", spec.position, runtime)
            self.position = runtime.shared[key]
        self.decay = torch.tensor(list(spec.decay), dtype=torch.float32, device=runtime.device)
        if spec.norm not in ("head", "all"):
            raise ValueError(f"the retention's norm is 'head' or 'all', got {spec.norm!r}")
        if spec.gate_activation not in ("silu", "sigmoid"):
            raise ValueError(f"the retention's gate is 'silu' or 'sigmoid', got {spec.gate_activation!r}")
        if spec.input_activation is not None and spec.input_activation not in ops.ACTIVATIONS:
            raise ValueError(f"input activation {spec.input_activation!r} is not built (known: {', '.join(sorted(ops.ACTIVATIONS))})")
        if spec.norm == "head" and spec.gate_activation != "silu":
            raise ValueError("a sigmoid gate comes with the norm over all heads")
        self.whole_norm = spec.norm == "all"

    def parameters(self):
        s, n = self.spec, self.spec.weights
        return [ParamRequest(n["q"], (self.qk_width, s.hidden_size)), ParamRequest(n["k"], (self.qk_width, s.hidden_size)),
                ParamRequest(n["v"], (self.v_width, s.hidden_size)), ParamRequest(n["gate"], (self.v_width, s.hidden_size)),
                ParamRequest(n["o"], (s.hidden_size, self.v_width))] + \
               ([ParamRequest(n["norm"], (self.v_width,), "gain")] if self.whole_norm else [])

    def load(self, tensors):
        n, rt = self.spec.weights, self.runtime
        first = [rt.matrix(tensors[n[r]]) for r in ("q", "k", "v", "gate")]
        if len({m.dtype for m in first}) > 1:
            first = [m.float() for m in first]
        self.w_in, self.starts = stack_rows(first)
        self.w_o = rt.matrix(tensors[n["o"]])
        self.norm_gain = rt.vector(tensors[n["norm"]]) if self.whole_norm else None

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_o

    def state_request(self):
        s = self.spec
        return StateRequest((s.num_heads, s.head_dim, s.value_dim), torch.float32)

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        s, pos = self.spec, self.position
        if run.state is None:
            raise RuntimeError("the retention mixer needs its per-sequence state; its run has none")
        at = self.starts
        q = proj[:, at[0]:at[0] + self.qk_width]
        k = proj[:, at[1]:at[1] + self.qk_width]
        v = proj[:, at[2]:at[2] + self.v_width]
        g = proj[:, at[3]:at[3] + self.v_width]
        tables = (pos.cos if pos else None, pos.sin if pos else None, pos.rotary_dim if pos else 0)
        if self.whole_norm:
            # the walk leaves o as floats; one norm over all heads, the gate and the storage type follow in a kernel of their own
            raw = torch.empty((proj.shape[0], self.v_width), dtype=torch.float32, device=proj.device)
            ops.retention_scan(q, k, v, None, batch.positions, *tables, self.decay, s.key_scale, s.eps, run.state, batch.slots,
                               batch.cu_q, s.num_heads, s.head_dim, s.value_dim, None, scale, batch.max_q_len,
                               input_activation=s.input_activation, raw_out=raw)
            ops.group_norm_gate(raw, self.norm_gain, g, mid, s.eps, s.gate_activation)
            return
        ops.retention_scan(q, k, v, g, batch.positions, *tables, self.decay, s.key_scale, s.eps, run.state, batch.slots, batch.cu_q,
                           s.num_heads, s.head_dim, s.value_dim, mid, scale, batch.max_q_len, input_activation=s.input_activation)


register_part("mixer", "retention", RetentionMixer)

"""The gated delta rule: a matrix of state per head that forgets by a gate and writes by the error of what it would read.

q = Wq.xn, k = Wk.xn (`num_kv_heads` heads of `head_dim`), v = Wv.xn (`num_heads` heads of `value_dim`), no biases; each
passes a short causal convolution over time per channel (the last of its `conv_taps` weights meets the current token, zeros
before the sequence's start) and a silu; q and k become unit vectors x / sqrt(sum x^2 + unit_eps), q times head_dim^-1/2;
beta = sigmoid(Wb.xn) and g = exp(-exp(A_log) * softplus(Wa.xn + dt_bias)), one number per head and token.  Per head (which
uses q/k head h / (heads / kv_heads)):

    S <- g S;    u = beta (v - S^T k);    S <- S + k u^T;    o = S^T q          (the read-out sees the token's own write)

Every head's o is divided by its root mean square, multiplied by a gain of value_dim numbers that the heads share and by
silu(Wg.xn); then Wo.  The per-sequence state is float32 and lives in the engine's state area: S [heads, head_dim, value_dim],
then the convolutions' last conv_taps - 1 inputs [conv_taps - 1, channels].  Everything between the first products and the
last one is float32 arithmetic in both modes.
"""

from __future__ import annotations

import torch

from ..cache.state import StateRequest
from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Mixer, RunContext
from .linear import stack_rows
from .registry import register_part
from .split import SplitPart


class GatedDeltaMixer(SplitPart, Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are no multiple of {spec.num_kv_heads} query/key heads")
        if spec.conv_taps < 1:
            raise ValueError(f"a convolution has at least one weight per channel, got {spec.conv_taps}")
        self.qk_width = spec.num_kv_heads * spec.head_dim
        self.v_width = spec.num_heads * spec.value_dim
        self.channels = 2 * self.qk_width + self.v_width  # q | k | v, the convolved columns
        self.state_floats = spec.num_heads * spec.head_dim * spec.value_dim  # S; the convolutions' tail follows

    def parameters(self):
        s, n = self.spec, self.spec.weights
        W, H = s.hidden_size, s.num_heads
        return [ParamRequest(n["q"], (self.qk_width, W)), ParamRequest(n["k"], (self.qk_width, W)), ParamRequest(n["v"], (self.v_width, W)),
                ParamRequest(n["q_conv"], (self.qk_width, s.conv_taps), "bias"), ParamRequest(n["k_conv"], (self.qk_width, s.conv_taps), "bias"),
                ParamRequest(n["v_conv"], (self.v_width, s.conv_taps), "bias"), ParamRequest(n["b"], (H, W)), ParamRequest(n["a"], (H, W)),
                ParamRequest(n["A_log"], (H,), "bias"), ParamRequest(n["dt_bias"], (H,), "bias"), ParamRequest(n["norm"], (s.value_dim,), "gain"),
                ParamRequest(n["gate"], (self.v_width, W)), ParamRequest(n["o"], (W, self.v_width))]

    def load(self, tensors):
        n, rt = self.spec.weights, self.runtime
        qkv = [rt.matrix(tensors[n[r]]) for r in ("q", "k", "v")]
        rest = [rt.matrix(tensors[n[r]]) for r in ("a", "b", "gate")]
        if len({m.dtype for m in qkv + rest}) > 1:
            qkv, rest = [m.float() for m in qkv], [m.float() for m in rest]
        # q, k and v in one piece (the convolution walks their columns as one row), then a, b and the gate
        self.w_in, self.starts = stack_rows([torch.cat(qkv, dim=0)] + rest)
        self.w_o = rt.matrix(tensors[n["o"]])
        self.conv = torch.cat([rt.vector(tensors[n[r]]) for r in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.decay = (-torch.exp(rt.vector(tensors[n["A_log"]]))).contiguous()  # g = exp(decay * softplus(.))
        self.dt_bias = rt.vector(tensors[n["dt_bias"]])
        self.gain = rt.vector(tensors[n["norm"]])

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_o

    def state_request(self):
        return StateRequest((self.state_floats + (self.spec.conv_taps - 1) * self.channels,), torch.float32)

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        s = self.spec
        if run.state is None:
            raise RuntimeError("the gated delta rule needs its per-sequence state; its run has none")
        at, H = self.starts, s.num_heads
        qkv = proj[:, at[0]:at[0] + self.channels]
        a_in, b_in = proj[:, at[1]:at[1] + H], proj[:, at[2]:at[2] + H]
        gate = proj[:, at[3]:at[3] + self.v_width]
        conv = ops.short_conv(qkv, self.conv, run.state, self.state_floats, batch.slots, batch.cu_q, batch.max_q_len, activation="silu",
                              store_tail=True)
        ops.gated_delta_scan(conv, 0, self.qk_width, 2 * self.qk_width, a_in, b_in, gate, self.decay, self.dt_bias, self.gain,
                             s.unit_eps, s.eps, run.state, 0, batch.slots, batch.cu_q, H, s.num_kv_heads, s.head_dim, s.value_dim,
                             mid, scale)


register_part("mixer", "gated_delta", GatedDeltaMixer)

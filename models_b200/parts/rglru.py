"""A recurrent block around a real-gated linear recurrent unit.

Two branches of `width` channels: y = gelu_tanh(Wy.xn + by) and u = conv(Wx.xn + bx), a short causal convolution per channel
with a bias (the last of its `conv_taps` weights meets the current token; zeros before the sequence's start; no activation).
The channels form `blocks` equal blocks; in block b, r = sigmoid(Ra[b].u_b + ra_b) and i = sigmoid(Ri[b].u_b + ri_b) with square
matrices.  log a = -rate * r * softplus(lambda), a = exp(log a);

    S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t         from S = 0, the first token like every other;

result Wo.(S * y).  The per-sequence state is float32 in the engine's state area: S [width], then the convolution's last
conv_taps - 1 inputs [conv_taps - 1, width].  The convolution's result, both gates (their small products included) and the
recurrence are float32 arithmetic in both modes.
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


class RglruMixer(SplitPart, Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.width % spec.blocks:
            raise ValueError(f"{spec.width} channels are no whole blocks of {spec.blocks}")
        self.per = spec.width // spec.blocks

    def parameters(self):
        s, n = self.spec, self.spec.weights
        R, W, B, per = s.width, s.hidden_size, s.blocks, self.per
        return [ParamRequest(n["y"], (R, W)), ParamRequest(n["y_bias"], (R,), "bias"), ParamRequest(n["x"], (R, W)),
                ParamRequest(n["x_bias"], (R,), "bias"), ParamRequest(n["conv"], (R, s.conv_taps), "bias"),
                ParamRequest(n["conv_bias"], (R,), "bias"), ParamRequest(n["gate_a"], (B, per, per)),
                ParamRequest(n["gate_a_bias"], (B, per), "bias"), ParamRequest(n["gate_i"], (B, per, per)),
                ParamRequest(n["gate_i_bias"], (B, per), "bias"), ParamRequest(n["lam"], (R,), "bias"), ParamRequest(n["o"], (W, R))]

    def load(self, tensors):
        s, n, rt = self.spec, self.spec.weights, self.runtime
        first = [rt.matrix(tensors[n[r]]) for r in ("y", "x")]
        if first[0].dtype != first[1].dtype:
            first = [m.float() for m in first]
        self.w_in, self.starts = stack_rows(first)
        self.w_o = rt.matrix(tensors[n["o"]])
        self.y_bias, self.x_bias = rt.vector(tensors[n["y_bias"]]), rt.vector(tensors[n["x_bias"]])
        self.conv, self.conv_bias = rt.vector(tensors[n["conv"]]), rt.vector(tensors[n["conv_bias"]])
        # both gates' matrices of a block one below the other: one small product per block gives [r sums | i sums]
        self.gates = torch.cat([rt.vector(tensors[n["gate_a"]]), rt.vector(tensors[n["gate_i"]])], dim=1).contiguous()
        # for prompts in the bfloat16 mode: every block's matrices twice side by side, [2 per, 2 per] bfloat16 (see `inner`)
        self.gates_twice = None
        if rt.mode == "bfloat16" and tensors[n["gate_a"]].dtype == torch.bfloat16 and tensors[n["gate_i"]].dtype == torch.bfloat16:
            twice = torch.cat([self.gates, self.gates], dim=2).to(torch.bfloat16).contiguous()
            if twice.is_cuda and ops.gemm_tcgen05_takes(twice[0], ops.EPI_F32) and (2 * self.per) % 8 == 0:
                self.gates_twice = twice
        self.r_bias = rt.vector(tensors[n["gate_a_bias"]]).reshape(-1).contiguous()
        self.i_bias = rt.vector(tensors[n["gate_i_bias"]]).reshape(-1).contiguous()
        self.rate = (-float(s.rate) * torch.nn.functional.softplus(rt.vector(tensors[n["lam"]]))).contiguous()  # log a = rate * r

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_o

    def state_request(self):
        return StateRequest((self.spec.width * self.spec.conv_taps,), torch.float32)  # S, then conv_taps - 1 rows of inputs

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        s = self.spec
        if run.state is None:
            raise RuntimeError("the recurrent block needs its per-sequence state; its run has none")
        R, at = s.width, self.starts
        y_in, x_in = proj[:, at[0]:at[0] + R], proj[:, at[1]:at[1] + R]
        rows = proj.shape[0]
        sums = torch.empty((rows, 2 * R), dtype=torch.float32, device=proj.device)
        if self.gates_twice is not None and rows > ops.WIDE_ROWS:
            # a prompt: the gates' small products on the tensor cores.  u goes in as two bfloat16 numbers (its rounding and the
            # rest, side by side along K, against the block's matrices repeated), so the sums keep float accuracy
            u, split = ops.short_conv(x_in, self.conv, run.state, R, batch.slots, batch.cu_q, batch.max_q_len, in_bias=self.x_bias,
                                      out_bias=self.conv_bias, store_tail=True, split_per=self.per)
            for b in range(s.blocks):
                at = b * 2 * self.per
                ops.gemm_tcgen05(split[:, at:at + 2 * self.per], self.gates_twice[b], ops.EPI_F32, out=sums[:, at:at + 2 * self.per])
        else:
            u = ops.short_conv(x_in, self.conv, run.state, R, batch.slots, batch.cu_q, batch.max_q_len, in_bias=self.x_bias,
                               out_bias=self.conv_bias, store_tail=True)
            ops.head_linear(u, self.gates, sums, s.blocks, tensor_cores=False)
        ops.rglru_scan(sums, self.per, u, y_in, self.r_bias, self.i_bias, self.y_bias, self.rate, run.state, 0, batch.slots, batch.cu_q,
                       batch.max_q_len, mid, scale)


register_part("mixer", "rglru", RglruMixer)

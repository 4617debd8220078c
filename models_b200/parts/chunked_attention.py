"""Grouped-query softmax attention whose projections are normalised as a whole and whose visibility is cut into chunks.

q = Wq.xn + bq, k = Wk.xn + bk, v = Wv.xn + bv; with `projection_norm` the whole row q (all heads side by side) passes ONE RMS
norm with a gain of that size, and so does k, before the heads are split; every head's first coordinates are then rotated by the
token's position (the spec's `position`); score(i, j) = scale * q_i.k_j; with `chunk` n, query i sees key j <= i only if
floor(i / n) = floor(j / n), chunks counted from position 0 of the sequence whatever the step's cut; softmax over the visible
keys; head h reads the keys and values of head h / (heads / kv_heads); then Wo.  Biases, norms, rotation, scores and weights
are float32 arithmetic in both modes.
"""

from __future__ import annotations

import torch

from ..cache.kv_cache import KvRequest
from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Mixer, RunContext
from .linear import stack_rows
from .registry import build_part, register_part
from .split import SplitPart


class ChunkedAttentionMixer(SplitPart, Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are no multiple of {spec.num_kv_heads} kv heads")
        if spec.chunk is not None and spec.chunk < 1:
            raise ValueError(f"a chunk holds at least one position, got {spec.chunk}")
        self.q_width = spec.num_heads * spec.head_dim
        self.k_width = spec.num_kv_heads * spec.head_dim
        self.v_width = spec.num_kv_heads * spec.value_dim
        self.mid_width = spec.num_heads * spec.value_dim
        self.position = None
        if spec.position is not None:
            if spec.position.rotary_dim > spec.head_dim:
                raise ValueError(f"rotary_dim {spec.position.rotary_dim} exceeds head_dim {spec.head_dim}")
            key = ("position", spec.position, runtime.max_positions)
            if key not in runtime.shared:
                runtime.shared[key] = build_part("position", spec.position, runtime)
            self.position = runtime.shared[key]

    def parameters(self):
        s, n = self.spec, self.spec.weights
        out = [ParamRequest(n["q"], (self.q_width, s.hidden_size)), ParamRequest(n["k"], (self.k_width, s.hidden_size)),
               ParamRequest(n["v"], (self.v_width, s.hidden_size)), ParamRequest(n["o"], (s.hidden_size, self.mid_width))]
        if s.bias:
            out += [ParamRequest(n["q_bias"], (self.q_width,), "bias"), ParamRequest(n["k_bias"], (self.k_width,), "bias"),
                    ParamRequest(n["v_bias"], (self.v_width,), "bias")]
        if s.projection_norm:
            out += [ParamRequest(n["q_norm"], (self.q_width,), "gain"), ParamRequest(n["k_norm"], (self.k_width,), "gain")]
        return out

    def load(self, tensors):
        s, n, rt = self.spec, self.spec.weights, self.runtime
        first = [rt.matrix(tensors[n[r]]) for r in ("q", "k", "v")]
        if len({m.dtype for m in first}) > 1:
            first = [m.float() for m in first]
        self.w_in, self.starts = stack_rows(first)
        self.w_o = rt.matrix(tensors[n["o"]])
        self.biases = tuple(rt.vector(tensors[n[r]]) for r in ("q_bias", "k_bias", "v_bias")) if s.bias else (None, None, None)
        self.gains = tuple(rt.vector(tensors[n[r]]) for r in ("q_norm", "k_norm")) if s.projection_norm else (None, None)

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_o

    def kv_request(self):
        s = self.spec
        return KvRequest(s.num_kv_heads, s.head_dim, None, s.value_dim)

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        s, pos = self.spec, self.position
        if run.k_pool is None:
            raise RuntimeError("the attention mixer needs cache pools; its run has none")
        if not run.writes_cache:
            raise RuntimeError("this mixer writes the cache it reads; a run that reads another run's cache is not built for it")
        if scale != 1.0:
            raise ValueError("this mixer's result cannot be scaled on its way out")
        group = batch.groups[run.group]
        at = self.starts
        q = proj[:, at[0]:at[0] + self.q_width]
        k = proj[:, at[1]:at[1] + self.k_width]
        v = proj[:, at[2]:at[2] + self.v_width]
        ops.project_norm_rotate_store(q, k, v, *self.biases, *self.gains, s.eps, batch.positions, pos.cos if pos else None,
                                      pos.sin if pos else None, pos.rotary_dim if pos else 0, pos.interleaved if pos else False,
                                      run.k_pool, run.v_pool, group.slot_mapping, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim)
        ops.gated_attention(q, mid, run.k_pool, run.v_pool, group.block_table, batch.cu_q, batch.kv_lens, batch.max_q_len,
                            s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, "softmax", s.scale, block=s.chunk or 0)


register_part("mixer", "chunked_attention", ChunkedAttentionMixer)

"""Grouped-query softmax attention with bounded scores, a temperature per head and a sink.

q = Wq.xn, k = Wk.xn (heads of `head_dim`), v = Wv.xn (heads of `value_dim`); q and k are rotated by their position over
the first coordinates of every head (the spec's `position`) and then, with `unit_norm`, divided by their root mean square
over the head (no gain); with `value_position` the value of position j is rotated by j before it is cached and every head's
sum over the keys is turned back by the query's position i, so that what comes out depends on i - j only;
score(i, j) = scale * temperature_h * q_i.k_j, then softcap * tanh(score / softcap); key j <= i gets the weight
exp(s_j) / (sink + sum_j' exp(s_j')) where `sink` adds 1 to the denominator, a key of score 0 that has no value;
head h reads the keys and values of head h / (heads / kv_heads); then Wo.  Rotation, norms, scores and weights are float32
arithmetic in both modes.
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


class CappedAttentionMixer(SplitPart, Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are no multiple of {spec.num_kv_heads} kv heads")
        if spec.head_dim > 256:
            raise ValueError(f"this mixer takes heads of up to 256 coordinates, got {spec.head_dim}")
        self.q_width = spec.num_heads * spec.head_dim
        self.k_width = spec.num_kv_heads * spec.head_dim
        self.v_width = spec.num_kv_heads * spec.value_dim
        self.mid_width = spec.num_heads * spec.value_dim
        self.position = self._tables(spec.position, spec.head_dim, "rotary_dim")
        self.value_position = self._tables(spec.value_position, spec.value_dim, "the values' rotary_dim")
        if self.value_position is not None:
            if not self.value_position.interleaved or self.value_position.rotary_dim != spec.value_dim:
                raise ValueError("values are rotated over all their coordinates in pairs (2m, 2m + 1)")
            if self.position is not None and not self.position.interleaved:
                raise ValueError("keys and values are rotated in one layout of pairs; the keys' is not (2i, 2i + 1)")

    def _tables(self, spec, limit, what):
        if spec is None:
            return None
        if spec.rotary_dim > limit:
            raise ValueError(f"{what} {spec.rotary_dim} exceeds {limit}")
        key = ("position", spec, self.runtime.max_positions)
        if key not in self.runtime.shared:
            self.runtime.shared[key] = build_part("position", spec, self.runtime)
        return self.runtime.shared[key]

    def parameters(self):
        s, n = self.spec, self.spec.weights
        out = [ParamRequest(n["q"], (self.q_width, s.hidden_size)), ParamRequest(n["k"], (self.k_width, s.hidden_size)),
               ParamRequest(n["v"], (self.v_width, s.hidden_size)), ParamRequest(n["o"], (s.hidden_size, self.mid_width))]
        if s.head_temperature:
            out.append(ParamRequest(n["temperature"], (s.num_heads,), "bias"))
        return out

    def load(self, tensors):
        s, n, rt = self.spec, self.spec.weights, self.runtime
        first = [rt.matrix(tensors[n[r]]) for r in ("q", "k", "v")]
        if len({m.dtype for m in first}) > 1:
            first = [m.float() for m in first]
        self.w_in, self.starts = stack_rows(first)
        self.w_o = rt.matrix(tensors[n["o"]])
        self.temperature = rt.vector(tensors[n["temperature"]]) if s.head_temperature else None

    def input_matrix(self):
        return self.w_in

    def output_matrix(self):
        return self.w_o

    def kv_request(self):
        s = self.spec
        return KvRequest(s.num_kv_heads, s.head_dim, None, s.value_dim)

    def inner(self, proj: torch.Tensor, mid: torch.Tensor, batch, run: RunContext, scale: float = 1.0) -> None:
        s, pos, vpos = self.spec, self.position, self.value_position
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
        ops.rotate_norm_store(q, k, v, batch.positions, pos.cos if pos else None, pos.sin if pos else None,
                              pos.rotary_dim if pos else 0, pos.interleaved if pos else True, s.unit_norm, s.eps,
                              vpos.cos if vpos else None, vpos.sin if vpos else None, vpos.rotary_dim if vpos else 0,
                              run.k_pool, run.v_pool, group.slot_mapping, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim)
        ops.gated_attention(q, mid, run.k_pool, run.v_pool, group.block_table, batch.cu_q, batch.kv_lens, batch.max_q_len,
                            s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, "softmax", s.scale,
                            head_scale=self.temperature, softcap=s.softcap, sink=s.sink,
                            turn_cos=vpos.cos if vpos else None, turn_sin=vpos.sin if vpos else None)


register_part("mixer", "capped_attention", CappedAttentionMixer)

"""Typed configuration of the Kivezen decoder, read from the keys of its own config.json.

A Kivezen model keeps `streams` copies of the residual stream (hyper-connections): a sublayer reads a learned mix
of the copies through an RMS norm, and its result goes back into all copies at once together with a learned mixing
of the copies among themselves (without the key `streams` there is one stream and a plain residual sum).  Every layer
names its mixer and carries its own sizes and constants; a span of layers may run several times in a row with the
same weights, each pass with a cache and state of its own (`loop`):

  "attention"  grouped-query softmax attention: rotary positions on the first part of a head (pairs 2i, 2i + 1;
               optionally stretched, "scaling"), queries and keys then divided by their root mean square, values
               rotated by their own position and the result turned back by the query's, a learned temperature per
               head, scores bounded by softcap * tanh(. / softcap), and one more term of score 0 in the softmax's
               denominator;
  "lightning"  linear attention with a fixed decay per head over silu'd projections, a float32 state per sequence
               instead of a cache, one RMS norm over all heads, a sigmoid gate.

The feed-forward is dense, down(gelu_tanh(up(h))), or a mixture of experts: the `top` experts by router logit, weighted
by the softmax over the chosen logits, plus a shared expert behind a sigmoid gate; an expert is
down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate(h), limit) and u = clamp(up(h), -limit, limit).
The logits pass logit_softcap * tanh(. / logit_softcap).

config.json (every size and constant of a model is here or is a tensor's shape):

    {"architecture": "Kivezen", "vocab": V, "width": W, "norm": {"eps": e}, "streams": S, "logit_softcap": c,
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": s, "softcap": c,
                           "rot": {"dims": r, "base": b, "scaling": {"factor": f, "original": n, "fast": x, "slow": y}}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "lightning", "mixer": {"heads": H, "dim": D, "vdim": Dv, "decay": [d_0, ...]},
                 "mlp": {"kind": "moe", "router": {"experts": E, "top": k}, "expert": {"ff": F, "limit": l},
                         "shared": {"ff": F, "limit": l}} | null}, ...]}

Tensors: `embed`, `head`, `final.norm`, and per layer i under `l<i>.`: `norm1`, `norm2`, with hyper-connections
`hc1.{in,out,mix}`, `hc2.{in,out,mix}`; `mix.{q,k,v,temp,o}` (attention), `mix.{q,k,v,g,norm,o}` (lightning);
`mlp.{up,down}` (dense), `mlp.router`, `mlp.e<j>.{gate,up,down}`, `mlp.shared.{gate,up,down,sg}` (experts).
Linear weights are [out, in].
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .kabanex import UNLIMITED_POSITIONS, _float, _get, _int
from .llama import ConfigError
from .specs import (
    CappedAttentionSpec,
    ClampedExpertSpec,
    DenseFeedForwardSpec,
    EmbeddingSpec,
    HeadSpec,
    HyperBlockSpec,
    ModelSpec,
    NormSpec,
    RetentionSpec,
    RopeScalingSpec,
    RopeSpec,
    RoutedFeedForwardSpec,
    ScheduleEntry,
)

ARCHITECTURE = "Kivezen"
MIXERS = ("attention", "lightning")
# Constants the design fixes.
SWISH_SLOPE = 1.702  # an expert's gate branch is g * sigmoid(1.702 g)
MAGNITUDE_SLOPE = 0.1  # stretched rotary tables are multiplied by 0.1 * ln(factor) + 1


@dataclass(frozen=True)
class KivezenScaling:
    factor: float
    original: float  # positions the unstretched frequencies were made for
    fast: float
    slow: float


@dataclass(frozen=True)
class KivezenAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float  # 0: scores are not bounded
    rot_dims: int  # 0 with rot_base 0: the layer has no "rot" at all (no rotation of values either)
    rot_base: float
    scaling: Optional[KivezenScaling]


@dataclass(frozen=True)
class KivezenLightning:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class KivezenExpert:
    ff: int
    limit: float


@dataclass(frozen=True)
class KivezenFeedForward:
    kind: str  # "dense" or "moe"
    ff: int = 0  # dense
    experts: int = 0
    top: int = 0
    expert: Optional[KivezenExpert] = None
    shared: Optional[KivezenExpert] = None


@dataclass(frozen=True)
class KivezenLayer:
    type: str
    mixer: object
    mlp: Optional[KivezenFeedForward]


def _expert(raw, where: str) -> KivezenExpert:
    return KivezenExpert(_int(raw, "ff", where), _float(raw, "limit", where, positive=True))


def _attention(mixer, where: str) -> KivezenAttention:
    heads, kv_heads = _int(mixer, "heads", where), _int(mixer, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    dim, vdim = _int(mixer, "dim", where), _int(mixer, "vdim", where)
    softcap = _float(mixer, "softcap", where, positive=True) if mixer.get("softcap") is not None else 0.0
    rot = mixer.get("rot")
    dims, base, scaling = 0, 0.0, None
    if rot is not None:
        dims = _int(rot, "dims", where + ".rot", least=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim ({dim}), got {dims}")
        if vdim % 2:
            raise ConfigError(f"config.json: {where}.vdim must be even (values are rotated in pairs), got {vdim}")
        base = _float(rot, "base", where + ".rot", positive=True)
        if base == 1.0:
            raise ConfigError(f"config.json: {where}.rot.base must differ from 1")
        s = rot.get("scaling")
        if s is not None:
            sw = where + ".rot.scaling"
            scaling = KivezenScaling(_float(s, "factor", sw, positive=True), _float(s, "original", sw, positive=True),
                                     _float(s, "fast", sw, positive=True), _float(s, "slow", sw, positive=True))
    return KivezenAttention(heads, kv_heads, dim, vdim, _float(mixer, "scale", where), softcap, dims, base, scaling)


def _lightning(mixer, where: str) -> KivezenLightning:
    heads = _int(mixer, "heads", where)
    decay = _get(mixer, "decay", where)
    if not isinstance(decay, (list, tuple)) or len(decay) != heads:
        raise ConfigError(f"config.json: {where}.decay must list one number per head ({heads})")
    values = []
    for n, d in enumerate(decay):
        if isinstance(d, bool) or not isinstance(d, (int, float)) or not 0.0 <= d <= 1.0:
            raise ConfigError(f"config.json: {where}.decay[{n}] must be a number in [0, 1], got {d!r}")
        values.append(float(d))
    return KivezenLightning(heads, _int(mixer, "dim", where), _int(mixer, "vdim", where), tuple(values))


def _feed_forward(mlp, where: str) -> Optional[KivezenFeedForward]:
    if mlp is None:
        return None
    kind = _get(mlp, "kind", where)
    if kind == "dense":
        return KivezenFeedForward("dense", ff=_int(mlp, "ff", where))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not built (known: dense, moe)")
    router = _get(mlp, "router", where)
    experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router.top ({top}) exceeds the {experts} experts")
    shared = mlp.get("shared")
    return KivezenFeedForward("moe", experts=experts, top=top, expert=_expert(_get(mlp, "expert", where), where + ".expert"),
                              shared=None if shared is None else _expert(shared, where + ".shared"))


@dataclass(frozen=True)
class KivezenConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    streams: int  # 0: no hyper-connections (one stream, plain residual sums)
    logit_softcap: float  # 0: none
    loop: Optional[Tuple[int, int, int]]  # (start, stop, times)
    layers: Tuple[KivezenLayer, ...]

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "KivezenConfig":
        vocab = _int(raw, "vocab", "the model")
        width = _int(raw, "width", "the model")
        eps = _float(_get(raw, "norm", "the model"), "eps", "norm", positive=True)
        streams = _int(raw, "streams", "the model") if raw.get("streams") is not None else 0
        cap = _float(raw, "logit_softcap", "the model", positive=True) if raw.get("logit_softcap") is not None else 0.0
        listed = _get(raw, "layers", "the model")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not built (known: {', '.join(MIXERS)})")
            mixer = _get(entry, "mixer", where)
            parsed = _attention(mixer, where + ".mixer") if kind == "attention" else _lightning(mixer, where + ".mixer")
            layers.append(KivezenLayer(kind, parsed, _feed_forward(entry.get("mlp"), where + ".mlp")))
        loop = None
        if raw.get("loop") is not None:
            lp = raw["loop"]
            start, stop, times = _int(lp, "start", "loop", least=0), _int(lp, "stop", "loop", least=0), _int(lp, "times", "loop")
            if not start <= stop <= len(layers):
                raise ConfigError(f"config.json: loop must satisfy start <= stop <= {len(layers)} layers, got {start}, {stop}")
            loop = (start, stop, times)
        return KivezenConfig(str(raw.get("architecture", ARCHITECTURE)), vocab, width, eps, streams, cap, loop, tuple(layers))

    def to_dict(self) -> dict:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.softcap:
                    mixer["softcap"] = m.softcap
                if m.rot_base:
                    mixer["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
                    if m.scaling is not None:
                        s = m.scaling
                        mixer["rot"]["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            f = layer.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "router": {"experts": f.experts, "top": f.top},
                       "expert": {"ff": f.expert.ff, "limit": f.expert.limit}}
                if f.shared is not None:
                    mlp["shared"] = {"ff": f.shared.ff, "limit": f.shared.limit}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": layers}
        if self.streams:
            out["streams"] = self.streams
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    def run_order(self):
        """Which layer each run of the schedule is: the looped span `times` times in a row, then the rest."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def model_spec(self) -> ModelSpec:
        blocks = []
        W, eps = self.width, self.norm_eps
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            m = layer.mixer
            names = {r: p + "mix." + r for r in ("q", "k", "v", "o")}
            if layer.type == "attention":
                position = value_position = None
                if m.rot_base:
                    scaling = None
                    if m.scaling is not None:
                        s = m.scaling
                        scaling = RopeScalingSpec("yarn", s.factor, low_freq_factor=s.slow, high_freq_factor=s.fast,
                                                  original_max_position=s.original,
                                                  magnitude=MAGNITUDE_SLOPE * math.log(s.factor) + 1.0)
                    if m.rot_dims:
                        position = RopeSpec(rotary_dim=m.rot_dims, theta=m.rot_base, pairing="interleaved", scaling=scaling)
                    value_position = RopeSpec(rotary_dim=m.vdim, theta=m.rot_base, pairing="interleaved")
                names["temperature"] = p + "mix.temp"
                mixer = CappedAttentionSpec(
                    hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                    scale=m.scale, eps=eps, position=position, unit_norm=True, value_position=value_position,
                    head_temperature=True, softcap=m.softcap, sink=True, weights=names)
            else:
                names.update(gate=p + "mix.g", norm=p + "mix.norm")
                mixer = RetentionSpec(hidden_size=W, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, decay=m.decay,
                                      key_scale=1.0, eps=eps, position=None, weights=names, input_activation="silu",
                                      norm="all", gate_activation="sigmoid")
            f = layer.mlp
            feed_forward = feed_forward_norm = None
            if f is not None:
                feed_forward_norm = NormSpec(W, eps, {"weight": p + "norm2"})
                if f.kind == "dense":
                    feed_forward = DenseFeedForwardSpec(W, f.ff, "gelu_tanh", {"up": p + "mlp.up", "down": p + "mlp.down"})
                else:
                    ff_names = {"router": p + "mlp.router"}
                    for r in ("gate", "up", "down"):
                        ff_names["expert_" + r] = p + "mlp.e{expert}." + r
                        ff_names["shared_" + r] = p + "mlp.shared." + r
                    ff_names["shared_gate_score"] = p + "mlp.shared.sg"
                    feed_forward = RoutedFeedForwardSpec(
                        hidden_size=W, num_experts=f.experts, top=f.top,
                        expert=ClampedExpertSpec(f.expert.ff, f.expert.limit, SWISH_SLOPE),
                        shared=None if f.shared is None else ClampedExpertSpec(f.shared.ff, f.shared.limit, SWISH_SLOPE),
                        weights=ff_names)
            hc = {}
            if self.streams:
                for which, q in (("mixer", "hc1"), ("feed_forward", "hc2")):
                    for r in ("in", "out", "mix"):
                        hc[f"{which}_{r}"] = f"{p}{q}.{r}"
            blocks.append(HyperBlockSpec(mixer=mixer, feed_forward=feed_forward, mixer_norm=NormSpec(W, eps, {"weight": p + "norm1"}),
                                         feed_forward_norm=feed_forward_norm, streams=self.streams, weights=hc))
        # a layer without a feed-forward reads no second norm and no second set of connections; a file that holds them all
        # the same is taken
        unused = tuple(pattern for i, layer in enumerate(self.layers) if layer.mlp is None
                       for pattern in (f"l{i}.norm2", f"l{i}.hc2.*"))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=W,
            max_positions=UNLIMITED_POSITIONS,
            embedding=EmbeddingSpec(self.vocab, W, 1.0, {"weight": "embed"}),
            layers=tuple(blocks),
            schedule=tuple(ScheduleEntry(i) for i in self.run_order()),
            final_norm=NormSpec(W, eps, {"weight": "final.norm"}),
            head=HeadSpec(self.vocab, W, False, {"weight": "head"}, softcap=self.logit_softcap),
            residual_streams=max(1, self.streams),
            ignored_tensors=unused,
        )

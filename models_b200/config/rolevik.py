"""Typed configuration of the Rolevik decoder, read from the keys of its own config.json.

A Rolevik layer puts its norms on the sublayers' RESULTS: x += ls1 * LN(mixer(x)), then x += ls2 * LN(ff(x)), where the
sublayers read x itself, LN is a layer norm with a gain and no bias, and ls1, ls2 are learned scales per channel.  Every
layer names its mixer and carries its own sizes and constants:

  "parallel"  two mixers on the same rows, each with an output matrix of its own, whose results are RMS-normed over the
              width and averaged.  Left: grouped-query softmax attention with biased projections, ONE RMS norm over the whole
              query projection and one over the whole key projection (before the heads are split), rotary positions on the
              first part of a head (pairs i, i + dims/2), and visibility in chunks: query i sees key j <= i only if both lie
              in the same chunk of mask.size positions counted from position 0.  Right: the gated delta rule over q, k, v
              that pass a short causal convolution and a silu, unit-length q and k, a write strength and a decay per head and
              token, a float32 state per head, an RMS norm per head and a silu gate.
  "rglru"     a gated linear recurrence: a gelu branch times the state of a real-gated linear recurrent unit whose input
              passes a short causal convolution and whose two gates come from block-diagonal matrices.

The feed-forward is dense and gated, down(gelu_tanh(gate(h)) * up(h)), or a mixture of experts down(silu(gate(h)) * up(h)):
scores are the softmax of the router's outputs over experts and identity experts together; the choice runs on the scores
plus a correction, inside the best `groups.keep` of `groups.count` groups of neighbouring outputs; the weights are the
chosen scores times router.scale; the last router.identity outputs stand for experts that return their input; a shared
expert runs for every token.  A layer may have no feed-forward.  The logits reuse the embedding table, times logit_scale.

config.json (every size and constant of a model is here or is a tensor's shape):

    {"architecture": "Rolevik", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s}, "logit_scale": c,
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": s, "mask": {"size": n},
                                    "rot": {"dims": r, "base": b}},
                           "right": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "conv": taps}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "rglru", "mixer": {"width": R, "blocks": B, "conv": taps},
                 "mlp": {"kind": "moe", "router": {"experts": E, "identity": I, "top": k, "scale": s,
                                                   "groups": {"count": g, "keep": m}},
                         "expert": {"ff": F}, "shared": {"ff": F}} | null}, ...]}

Tensors: `embed`, `final.norm`, and per layer i under `l<i>.`: `norm1`, `norm2`, `ls1`, `ls2`;
`mix.left.{q,k,v}` with `.b`, `mix.left.{q,k}.norm`, `mix.left.o`, `mix.left.out`; `mix.right.{q,k,v}` with `.conv`,
`mix.right.{a,b,g,A_log,dt_bias,norm,o}`, `mix.right.out`; `mix.{y,x}` with `.b`, `mix.conv` with `.b`, `mix.{ra,ri}` with
`.b`, `mix.lam`, `mix.o` (rglru); `mlp.{gate,up,down}` (dense); `mlp.router`, `mlp.correction`, `mlp.e<j>.{gate,up,down}`,
`mlp.shared.{gate,up,down}` (experts).  Linear weights are [out, in].
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .kabanex import UNLIMITED_POSITIONS, _float, _get, _int
from .llama import ConfigError
from .specs import (
    ChunkedAttentionSpec,
    ClampedExpertSpec,
    EmbeddingSpec,
    GatedDeltaSpec,
    GatedFeedForwardSpec,
    HeadSpec,
    LayerNormSpec,
    ModelSpec,
    NormedPairSpec,
    OutputNormBlockSpec,
    RglruSpec,
    RopeSpec,
    RoutedFeedForwardSpec,
    ScheduleEntry,
)

ARCHITECTURE = "Rolevik"
MIXERS = ("parallel", "rglru")
# Constants the design fixes.
DELTA_UNIT_EPS = 1e-6  # unit vectors of the delta rule: x / sqrt(sum x^2 + 1e-6)
RGLRU_RATE = 8.0       # log a = -8 * r * softplus(lambda)


@dataclass(frozen=True)
class RolevikAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int  # 0: no "mask", every earlier key is visible
    rot_dims: int  # 0: no rotation
    rot_base: float  # 0: the layer has no "rot" at all


@dataclass(frozen=True)
class RolevikDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class RolevikParallel:
    left: RolevikAttention
    right: RolevikDelta


@dataclass(frozen=True)
class RolevikRglru:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class RolevikFeedForward:
    kind: str  # "dense" or "moe"
    ff: int = 0  # dense
    experts: int = 0
    identity: int = 0
    top: int = 0
    scale: float = 1.0
    groups: int = 1
    keep: int = 1
    expert_ff: int = 0
    shared_ff: int = 0  # 0: no shared expert


@dataclass(frozen=True)
class RolevikLayer:
    type: str
    mixer: object
    mlp: Optional[RolevikFeedForward]


def _heads(mixer, where):
    heads, kv_heads = _int(mixer, "heads", where), _int(mixer, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    return heads, kv_heads, _int(mixer, "dim", where), _int(mixer, "vdim", where)


def _attention(mixer, where: str) -> RolevikAttention:
    heads, kv_heads, dim, vdim = _heads(mixer, where)
    chunk = _int(mixer["mask"], "size", where + ".mask") if mixer.get("mask") is not None else 0
    dims, base = 0, 0.0
    if mixer.get("rot") is not None:
        rot = mixer["rot"]
        dims = _int(rot, "dims", where + ".rot", least=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim ({dim}), got {dims}")
        base = _float(rot, "base", where + ".rot", positive=True)
    return RolevikAttention(heads, kv_heads, dim, vdim, _float(mixer, "scale", where), chunk, dims, base)


def _feed_forward(mlp, where: str) -> Optional[RolevikFeedForward]:
    if mlp is None:
        return None
    kind = _get(mlp, "kind", where)
    if kind == "dense":
        return RolevikFeedForward("dense", ff=_int(mlp, "ff", where))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not built (known: dense, moe)")
    router = _get(mlp, "router", where)
    rw = where + ".router"
    experts, top = _int(router, "experts", rw), _int(router, "top", rw)
    identity = _int(router, "identity", rw, least=0) if router.get("identity") is not None else 0
    scale = _float(router, "scale", rw) if router.get("scale") is not None else 1.0
    groups = keep = 1
    if router.get("groups") is not None:
        groups, keep = _int(router["groups"], "count", rw + ".groups"), _int(router["groups"], "keep", rw + ".groups")
    total = experts + identity
    if total % groups or keep > groups:
        raise ConfigError(f"config.json: {rw}.groups must cut the {total} router outputs into equal groups and keep at most all of "
                          f"them, got count {groups}, keep {keep}")
    if top > total // groups * keep:
        raise ConfigError(f"config.json: {rw}.top ({top}) exceeds the {total // groups * keep} outputs of the kept groups")
    shared = mlp.get("shared")
    return RolevikFeedForward("moe", experts=experts, identity=identity, top=top, scale=scale, groups=groups, keep=keep,
                              expert_ff=_int(_get(mlp, "expert", where), "ff", where + ".expert"),
                              shared_ff=0 if shared is None else _int(shared, "ff", where + ".shared"))


@dataclass(frozen=True)
class RolevikConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: Tuple[RolevikLayer, ...]

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "RolevikConfig":
        vocab = _int(raw, "vocab", "the model")
        width = _int(raw, "width", "the model")
        eps = _float(_get(raw, "norm", "the model"), "eps", "norm", positive=True)
        embedding_scale = _float(raw["embedding"], "scale", "embedding") if raw.get("embedding") is not None else 1.0
        logit_scale = _float(raw, "logit_scale", "the model") if raw.get("logit_scale") is not None else 1.0
        listed = _get(raw, "layers", "the model")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            mixer = _get(entry, "mixer", where)
            mw = where + ".mixer"
            if kind == "parallel":
                right = _get(mixer, "right", mw)
                parsed = RolevikParallel(_attention(_get(mixer, "left", mw), mw + ".left"),
                                         RolevikDelta(*_heads(right, mw + ".right"), _int(right, "conv", mw + ".right")))
            elif kind == "rglru":
                parsed = RolevikRglru(_int(mixer, "width", mw), _int(mixer, "blocks", mw), _int(mixer, "conv", mw))
                if parsed.width % parsed.blocks:
                    raise ConfigError(f"config.json: {mw}.width ({parsed.width}) must be a multiple of blocks ({parsed.blocks})")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not built (known: {', '.join(MIXERS)})")
            layers.append(RolevikLayer(kind, parsed, _feed_forward(entry.get("mlp"), where + ".mlp")))
        return RolevikConfig(str(raw.get("architecture", ARCHITECTURE)), vocab, width, eps, embedding_scale, logit_scale, tuple(layers))

    def to_dict(self) -> dict:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "parallel":
                a, d = m.left, m.right
                left = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
                if a.chunk:
                    left["mask"] = {"size": a.chunk}
                if a.rot_base:
                    left["rot"] = {"dims": a.rot_dims, "base": a.rot_base}
                mixer = {"left": left,
                         "right": {"heads": d.heads, "kv_heads": d.kv_heads, "dim": d.dim, "vdim": d.vdim, "conv": d.conv}}
            else:
                mixer = {"width": m.width, "blocks": m.blocks, "conv": m.conv}
            f = layer.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.expert_ff},
                       "router": {"experts": f.experts, "identity": f.identity, "top": f.top, "scale": f.scale,
                                  "groups": {"count": f.groups, "keep": f.keep}}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale, "layers": layers}

    def model_spec(self) -> ModelSpec:
        blocks = []
        W, eps = self.width, self.norm_eps
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            m = layer.mixer
            if layer.type == "parallel":
                a, d = m.left, m.right
                lp, rp = p + "mix.left.", p + "mix.right."
                names = {r: lp + r for r in ("q", "k", "v", "o")}
                names.update(q_bias=lp + "q.b", k_bias=lp + "k.b", v_bias=lp + "v.b", q_norm=lp + "q.norm", k_norm=lp + "k.norm")
                position = RopeSpec(rotary_dim=a.rot_dims, theta=a.rot_base, pairing="half") if a.rot_dims else None
                left = ChunkedAttentionSpec(hidden_size=W, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, value_dim=a.vdim,
                                            scale=a.scale, eps=eps, position=position, chunk=a.chunk or None, bias=True,
                                            projection_norm=True, weights=names)
                names = {r: rp + r for r in ("q", "k", "v", "o", "a", "b", "A_log", "dt_bias", "norm")}
                names.update(gate=rp + "g", q_conv=rp + "q.conv", k_conv=rp + "k.conv", v_conv=rp + "v.conv")
                right = GatedDeltaSpec(hidden_size=W, num_heads=d.heads, num_kv_heads=d.kv_heads, head_dim=d.dim, value_dim=d.vdim,
                                       conv_taps=d.conv, unit_eps=DELTA_UNIT_EPS, eps=eps, weights=names)
                mixer = NormedPairSpec(left, right, W, eps, {"left": lp + "out", "right": rp + "out"})
            else:
                mp = p + "mix."
                names = {r: mp + r for r in ("y", "x", "conv", "o")}
                names.update(y_bias=mp + "y.b", x_bias=mp + "x.b", conv_bias=mp + "conv.b", gate_a=mp + "ra", gate_a_bias=mp + "ra.b",
                             gate_i=mp + "ri", gate_i_bias=mp + "ri.b", lam=mp + "lam")
                mixer = RglruSpec(hidden_size=W, width=m.width, blocks=m.blocks, conv_taps=m.conv, rate=RGLRU_RATE, weights=names)
            f = layer.mlp
            feed_forward = feed_forward_norm = None
            scales = {"mixer_scale": p + "ls1"}
            if f is not None:
                feed_forward_norm = LayerNormSpec(W, eps, {"weight": p + "norm2"}, bias=False)
                scales["feed_forward_scale"] = p + "ls2"
                if f.kind == "dense":
                    feed_forward = GatedFeedForwardSpec(W, f.ff, "gelu_tanh", False,
                                                        {r: p + "mlp." + r for r in ("gate", "up", "down")})
                else:
                    ff_names = {"router": p + "mlp.router", "correction": p + "mlp.correction"}
                    for r in ("gate", "up", "down"):
                        ff_names["expert_" + r] = p + "mlp.e{expert}." + r
                        ff_names["shared_" + r] = p + "mlp.shared." + r
                    plain = lambda ff: ClampedExpertSpec(ff, math.inf, 1.0, up_offset=0.0)  # noqa: E731  silu(gate) * up
                    feed_forward = RoutedFeedForwardSpec(
                        hidden_size=W, num_experts=f.experts, top=f.top, expert=plain(f.expert_ff),
                        shared=plain(f.shared_ff) if f.shared_ff else None, weights=ff_names, rule="scored", correction=True,
                        groups=f.groups, keep_groups=f.keep, weight_scale=f.scale, identity_experts=f.identity, shared_gated=False)
            blocks.append(OutputNormBlockSpec(mixer=mixer, feed_forward=feed_forward,
                                              mixer_norm=LayerNormSpec(W, eps, {"weight": p + "norm1"}, bias=False),
                                              feed_forward_norm=feed_forward_norm, weights=scales))
        # a layer without a feed-forward reads no second norm and no second scale; a file that holds them all the same is taken
        unused = tuple(pattern for i, layer in enumerate(self.layers) if layer.mlp is None for pattern in (f"l{i}.norm2", f"l{i}.ls2"))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=W,
            max_positions=UNLIMITED_POSITIONS,
            embedding=EmbeddingSpec(self.vocab, W, self.embedding_scale, {"weight": "embed"}),
            layers=tuple(blocks),
            schedule=tuple(ScheduleEntry(i) for i in range(len(blocks))),
            final_norm=LayerNormSpec(W, eps, {"weight": "final.norm"}, bias=False),
            head=HeadSpec(self.vocab, W, True, {}, logit_scale=self.logit_scale),
            ignored_tensors=unused,
        )

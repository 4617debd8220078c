"""Architecture-neutral descriptions of a decoder: what each part is and which sizes it has.

An architecture's typed configuration (for instance `LlamaConfig`) is translated once into a
`ModelSpec`.  Everything below the configuration layer -- parts, cache, step function -- reads
only these records, so no part knows which model it is in.  Every size and constant is a field;
nothing here has a default that stands for a particular model.

The per-layer questions integrallis/models answers with predicates on its config
(`usesRope(layer)`, `usesSlidingWindow(layer)`, `ropeTheta(layer)`;
backend-java/.../llama/LlamaConfig.java:129-173) become per-layer records here: each
`BlockSpec` carries its own mixer, feed-forward and norms, so one model may mix kinds.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


@dataclass(frozen=True)
class RopeScalingSpec:
    """How pair frequencies are stretched.  kind: "linear" (angle * 1/factor), "llama3", or "yarn": with
    pair(t) = dims * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(pair(high_freq_factor)), 0) and
    hi = min(ceil(pair(low_freq_factor)), dims - 1), pair i has ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) and
    the frequency f_i / factor * ramp_i + f_i * (1 - ramp_i): pairs that turn often within `original` positions keep
    their frequency, slow ones are divided by `factor`."""

    kind: str
    factor: float
    low_freq_factor: float = 0.0
    high_freq_factor: float = 0.0
    original_max_position: int = 0
    magnitude: float = 1.0  # multiplies every cosine and sine of the table


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding over the first `rotary_dim` coordinates of a head.

    pairing "half": pair i is (x[i], x[i + rotary_dim/2]); "interleaved": (x[2i], x[2i+1]).
    Mirrors RotaryTable(rotaryDim, theta, frequencyScale, frequencyFactors) plus its neox flag
    (backend-java/.../ops/RotaryTable.java:48-75,91-100).
    """

    rotary_dim: int
    theta: float
    pairing: str
    scaling: Optional[RopeScalingSpec] = None
    kind: str = "rope"


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a cache.  `window` None: all earlier keys; n: the n
    positions that end at the query.  `scale` multiplies each dot product."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: Optional[RopeSpec]
    window: Optional[int]
    bias: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "attention"


@dataclass(frozen=True)
class LayerNormSpec:
    """(x - mean) / sqrt(variance + eps) * weight + bias over the last axis; the variance is the mean of
    the squared deviations from the mean.  `bias` False: there is no bias tensor."""

    size: int
    eps: float
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "layernorm"
    bias: bool = True


@dataclass(frozen=True)
class TalkingAttentionSpec:
    """Causal grouped-query attention whose softmax weights are mixed ACROSS heads before they meet the
    values: w'_h(i, j) = sum_g talk[h, g] w_g(i, j); head h applies w'_h to the values of its own
    key/value head.  Keys have `head_dim` coordinates and values `value_dim`.  Query i sees key j <= i
    if i - j < `window` (None: no limit) or j < `keep_first` (the first positions of a sequence stay
    visible to every later query, at their true positions).  `gated`: head h's result is multiplied by
    sigmoid(gate_h . xn), one number per head and token, before the output matrix."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    position: Optional[RopeSpec]
    window: Optional[int]
    keep_first: int
    gated: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "talking_attention"


@dataclass(frozen=True)
class MinGruSpec:
    """A gated recurrence whose gates read the current token only: z = sigmoid(Wz.xn + bz),
    u = Wx.xn + bx, candidate c = u + 1/2 where u >= 0 and sigmoid(u) elsewhere,
    S_t = (1 - z) S_(t-1) + z c element by element, result Wo.(S_t * silu(Wg.xn)).  The state is
    `state_size` float32 numbers per sequence and starts at zero."""

    hidden_size: int
    state_size: int
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "mingru"


@dataclass(frozen=True)
class SideBySideSpec:
    """Two mixers that read the same rows; the result is left_scale * left + right_scale * right."""

    left: object
    right: object
    left_scale: float
    right_scale: float
    kind: str = "side_by_side"


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    """down(act(up(x))), no gate.  activation: a name of the activation table ("relu2": relu squared; "xielu": a
    quadratic above zero and an exponential below it whose two shape numbers are a tensor, `weights["act"]`)."""

    hidden_size: int
    intermediate_size: int
    activation: str
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "dense"


@dataclass(frozen=True)
class ParallelBlockSpec:
    """One layer with ONE norm whose rows both sublayers read: h = norm(x); x += mixer(h) + feed_forward(h).
    `feed_forward` None: the layer has only the mixer."""

    mixer: object
    feed_forward: Optional[object]
    norm: object
    kind: str = "parallel"


@dataclass(frozen=True)
class GatedFeedForwardSpec:
    """down(act(gate(x)) * up(x)), dense."""

    hidden_size: int
    intermediate_size: int
    activation: str
    bias: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "gated"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which mixer, which feed-forward, which norms, and how they are arranged.

    kind "prenorm": x += mixer(norm(x)); x += feed_forward(norm(x))
    (backend-java/.../llama/LlamaForwardPass.java:1028-1182).
    """

    mixer: object
    feed_forward: object
    mixer_norm: object
    feed_forward_norm: object
    kind: str = "prenorm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  The order in which layers run is a list of these: a layer may be
    named twice (its weights are shared, each run has a cache of its own) and a run may read the
    cache that an earlier run wrote (`cache_from` is that run's index in the schedule) instead of
    writing one."""

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int
    scale: float
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "embedding"


@dataclass(frozen=True)
class HeadSpec:
    """Output projection to the vocabulary.  `tied`: it uses the embedding table and owns no
    tensor (backend-java/.../llama/LlamaWeights.java:83-89).  The logits are multiplied by
    `logit_scale`, then with `softcap` c != 0 become c * tanh(logits / c)
    (backend-java/.../llama/LlamaForwardPass.java:1751-1764)."""

    vocab_size: int
    hidden_size: int
    tied: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    logit_scale: float = 1.0
    softcap: float = 0.0
    kind: str = "linear_head"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object
    head: HeadSpec
    stop_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    # Copies of the residual stream that the blocks keep side by side ([tokens, streams * width]); they all start as
    # the embedding's rows and are added up before the final norm.  1: the usual single stream.
    residual_streams: int = 1
    # Tensors a checkpoint of this architecture may hold that the model does not read: name patterns
    # (fnmatch) of buffers that are recomputed, and names that must repeat another tensor exactly (a
    # tied model's stored output matrix).  Anything else that is not asked for is an error.
    ignored_tensors: Tuple[str, ...] = ()
    duplicate_tensors: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)

    def __post_init__(self):
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule[{index}] names layer {entry.layer}, the model has {len(self.layers)}")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < index:
                    raise ValueError(
                        f"schedule[{index}] reads the cache of run {entry.cache_from}, which is not an earlier run")
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(
                        f"schedule[{index}] reads the cache of run {entry.cache_from}, which owns none")


@dataclass(frozen=True)
class SigmoidAttentionSpec:
    """Causal grouped-query attention whose weights are sigmoids, not a softmax: key j <= i gets
    sigmoid(scale * q_i.k_j - slope_h * (i - j) + bias_h) and the weights are not normalised over keys.
    slope_h = 2^(-slope_exponent * (h + 1) / heads) (`slope_exponent` 0: no distance term).  `qk_norm`: queries and
    keys pass an RMS norm per head (eps `eps`, one gain shared by the heads) before anything else.
    `temperature_coef` c != 0: the query at position p is multiplied by 1 + c * ln(floor((p + 1) / temperature_every) + 1).
    `head_bias`: bias_h is a tensor of one number per head (else 0).  `gated`: the heads side by side are multiplied
    element by element by sigmoid(gate . xn) before the output matrix.  There is no rotation."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    eps: float
    qk_norm: bool
    temperature_coef: float
    temperature_every: int
    slope_exponent: float
    head_bias: bool
    gated: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "sigmoid_attention"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal softmax attention whose keys and values are expanded from ONE cached row per position:
    c = rmsnorm(down . xn) of `latent_dim` numbers (gain, eps `eps`); head h has k = up_k[h] . c (`head_dim`) and
    v = up_v[h] . c (`value_dim`); score = scale * q.k; no positions enter.  `gated`: head h's result is multiplied
    by sigmoid(gate_h . xn), one number per head and token."""

    hidden_size: int
    num_heads: int
    head_dim: int
    value_dim: int
    latent_dim: int
    scale: float
    eps: float
    gated: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "latent_attention"


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with a fixed decay per head and no normalisation over keys: per head a float32 state
    S [head_dim, value_dim] that starts at zero, S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  Queries and keys
    are rotated (`position`, or None), keys then multiplied by `key_scale`; every head's o_t is divided by its root
    mean square (eps `eps`, no gain), the heads side by side are multiplied by silu(gate . xn), then the output matrix."""

    hidden_size: int
    num_heads: int
    head_dim: int
    value_dim: int
    decay: Tuple[float, ...]
    key_scale: float
    eps: float
    position: Optional[RopeSpec]
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "retention"
    # Variations.  `input_activation` (a name of the activation table, or None) is applied to q, k and v as they leave
    # their products.  `norm` "head": every head's o_t is divided by its own root mean square, no gain; "all": the heads
    # side by side pass ONE RMS norm with a gain tensor (`weights["norm"]`).  `gate_activation`: "silu" or "sigmoid".
    input_activation: Optional[str] = None
    norm: str = "head"
    gate_activation: str = "silu"


@dataclass(frozen=True)
class GatedResidualBlockSpec:
    """A pre-norm layer whose sublayer results pass a gate on their way into the stream:
    h = mixer_norm(x); x += sigmoid(Gm . h + bm) * mixer(h); then, if the layer has a feed-forward,
    h = feed_forward_norm(x); x += sigmoid(Gf . h + bf) * feed_forward(h).  The gates are [width, width] matrices
    with a bias, named in `weights` (mixer_gate, mixer_gate_bias, feed_forward_gate, feed_forward_gate_bias)."""

    mixer: object
    feed_forward: Optional[object]
    mixer_norm: object
    feed_forward_norm: Optional[object]
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "prenorm_gated"


@dataclass(frozen=True)
class CappedAttentionSpec:
    """Causal grouped-query softmax attention with a bounded score and an optional sink.
    q and k are rotated (`position`, or None) and then, with `unit_norm`, divided by their root mean square per head
    (eps `eps`, no gain).  score = scale * temperature_h * q.k with one learned number per head (`head_temperature`,
    `weights["temperature"]`; else 1), then with `softcap` c != 0: c * tanh(score / c).  `sink`: the softmax has one more
    term of score 0 in its denominator that has no value, p_j = exp(s_j) / (1 + sum exp(s_j)).
    `value_position`: the value of position j is rotated by j over its first `rotary_dim` coordinates before it is
    cached, and every head's result at position i is rotated back by -i after the sum over the keys."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    eps: float
    position: Optional[RopeSpec]
    unit_norm: bool
    value_position: Optional[RopeSpec]
    head_temperature: bool
    softcap: float
    sink: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "capped_attention"


@dataclass(frozen=True)
class ClampedExpertSpec:
    """One gated feed-forward with clamped branches: g = min(gate . x, limit), u = clamp(up . x, -limit, limit),
    down . (g * sigmoid(swish_slope * g) * (u + up_offset)); no biases.  limit = +inf, swish_slope 1 and up_offset 0 make the
    plain gated form down . (silu(gate . x) * (up . x))."""

    intermediate_size: int
    limit: float
    swish_slope: float
    up_offset: float = 1.0


@dataclass(frozen=True)
class RoutedFeedForwardSpec:
    """A mixture of `num_experts` feed-forwards of one shape (`expert`): router logits z = router . x in float32; every
    token uses the `top` experts with the largest logits (ties to the lower index) with the softmax over the chosen
    logits as weights.  `shared`: one more expert that every token uses, multiplied by sigmoid(shared_gate . x), one
    number per token.  `weights`: router, shared_gate, shared_{gate,up,down}, and expert_{gate,up,down} with `{expert}`
    in the name."""

    hidden_size: int
    num_experts: int
    top: int
    expert: ClampedExpertSpec
    shared: Optional[ClampedExpertSpec]
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "routed"
    # Variations.  `rule` "scored": the scores s = softmax(z) are taken over ALL router outputs; the choice runs on
    # s + correction (a tensor of one number per router output, `weights["correction"]`, when `correction` is set); the outputs
    # form `groups` equal groups of neighbours, a group counts by its largest choice score, and only outputs of the
    # `keep_groups` best groups can be chosen; the weights are `weight_scale` times the chosen outputs' s, not renormalised.
    # `identity_experts` n: the router has num_experts + n outputs, the last n of which stand for experts without tensors
    # whose result is their input.  `shared_gated` False: the shared expert is added as it is (no `shared_gate_score` tensor).
    rule: str = "top_logits"
    correction: bool = False
    groups: int = 1
    keep_groups: int = 1
    weight_scale: float = 1.0
    identity_experts: int = 0
    shared_gated: bool = True


@dataclass(frozen=True)
class HyperBlockSpec:
    """A pre-norm layer over `streams` copies of the residual stream (hyper-connections).  For the mixer and then, if
    the layer has one, the feed-forward: u = sum_s in[s] x_s; y = sublayer(norm(u)); then all copies at once from the old
    ones, x_t <- sum_s mix[s, t] x_s + out[t] y.  in, out [streams] and mix [streams, streams] are tensors
    (`weights`: mixer_in, mixer_out, mixer_mix, feed_forward_in, ...).  `streams` 0: one stream and no such tensors,
    x <- x + sublayer(norm(x))."""

    mixer: object
    feed_forward: Optional[object]
    mixer_norm: object
    feed_forward_norm: Optional[object]
    streams: int
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "prenorm_hyper"


@dataclass(frozen=True)
class ChunkedAttentionSpec:
    """Causal grouped-query softmax attention whose projections are normalised as a whole.  q, k and v have biases when
    `bias` is set; with `projection_norm` q (all heads side by side) passes ONE RMS norm with a gain of that size and eps `eps`,
    and so does k, before the heads are split and rotated (`position`, or None).  score = scale * q.k.  `chunk` n: query i sees
    key j <= i only if floor(i / n) = floor(j / n), chunks counted from position 0 of the sequence (None: every earlier key).
    Keys have `head_dim` coordinates, values `value_dim`."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    eps: float
    position: Optional[RopeSpec]
    chunk: Optional[int]
    bias: bool
    projection_norm: bool
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "chunked_attention"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule.  q and k (`num_kv_heads` heads of `head_dim`) and v (`num_heads` heads of `value_dim`) pass a short
    causal convolution over time per channel (`conv_taps` weights, the last one meeting the current token, zeros before the
    sequence's start) and a silu; q and k become unit vectors x / sqrt(sum x^2 + unit_eps), q times head_dim^-1/2;
    beta = sigmoid(b . xn) and g = exp(-exp(A_log) * softplus(a . xn + dt_bias)), one number per head; per head with a float32
    state S [head_dim, value_dim] that starts at zero: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Every
    head's o is divided by its root mean square (eps `eps`), multiplied by a gain of value_dim numbers the heads share and by
    silu(gate . xn); then the output matrix.  The last conv_taps - 1 inputs of the convolutions are part of the state."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    conv_taps: int
    unit_eps: float
    eps: float
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "gated_delta"


@dataclass(frozen=True)
class RglruSpec:
    """A recurrent block around a real-gated linear recurrent unit.  Two branches of `width` channels: y = gelu_tanh(Wy . xn + by)
    and u = conv(Wx . xn + bx), a short causal convolution per channel with a bias.  The channels form `blocks` equal blocks;
    in block b, r = sigmoid(Ra[b] u_b + ra_b) and i = sigmoid(Ri[b] u_b + ri_b) with square matrices; log a = -rate * r *
    softplus(lambda), S_t = a S_(t-1) + sqrt(1 - a^2) * i * u with a float32 state that starts at zero; result Wo . (S * y).
    The last conv_taps - 1 inputs of the convolution are part of the state."""

    hidden_size: int
    width: int
    blocks: int
    conv_taps: int
    rate: float
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "rglru"


@dataclass(frozen=True)
class NormedPairSpec:
    """Two mixers that read the same rows, each with an output matrix of its own; the result is the mean of the two results
    after an RMS norm each over the model's width (eps `eps`, gains `weights["left"]` and `weights["right"]`)."""

    left: object
    right: object
    hidden_size: int
    eps: float
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "normed_pair"


@dataclass(frozen=True)
class OutputNormBlockSpec:
    """A layer whose norms sit on the sublayers' RESULTS: x += mixer_scale * mixer_norm(mixer(x)); then, if the layer has a
    feed-forward, x += feed_forward_scale * feed_forward_norm(feed_forward(x)).  The sublayers read x itself; the scales are
    tensors of the model's width (`weights`: mixer_scale, feed_forward_scale), multiplied element by element."""

    mixer: object
    feed_forward: Optional[object]
    mixer_norm: object
    feed_forward_norm: Optional[object]
    weights: Mapping[str, str] = field(default_factory=dict, hash=False, compare=False)
    kind: str = "output_norm"

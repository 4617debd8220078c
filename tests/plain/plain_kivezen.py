"""A plain, slow statement of the Kivezen decoder: whole sequences, no cache, float64 on the CPU, one function
per mechanism, written from the design's equations and sharing nothing with the package.

The model keeps `streams` copies of the residual stream (hyper-connections; without the key there is one stream
and a plain residual sum).  A sublayer reads a mix of the copies, u = sum_s in[s] x_s, through an RMS norm, and its
result y goes back into all copies at once: x_t <- sum_s mix[s, t] x_s + out[t] y.  Mixers: `attention` (grouped
heads, rotated and unit-normed queries and keys, rotated values turned back after the sum, a temperature per head, a
tanh cap on the scores, a softmax with one more term of score 0 in its denominator) and `lightning` (a linear
recurrence with a fixed decay per head over silu'd projections, normed over all heads together and gated).  The
feed-forward is dense (gelu) or routed (a few experts per token and a shared one behind a gate).  A span of layers
may run several times in a row, each pass with its own cache.  Weights are a dict name -> tensor; a configuration is
the dict of the model's config.json.
"""

from __future__ import annotations

import math

import torch

from .plain_llama import read_model_folder  # noqa: F401  (reads config.json and the safetensors file)

F = torch.float64
SWISH_SLOPE = 1.702  # the expert's gate is g * sigmoid(1.702 g)


def rms_norm(x, weight=None, eps=1e-6):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def pair_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims) for pair i; with `scaling` (factor, original, fast, slow) the frequencies of slow pairs
    are divided by `factor`, those of fast pairs stay, and between them a ramp blends the two.  Returns the
    frequencies and the number that multiplies cosines and sines."""
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    if scaling is None:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, frequencies, magnitude=1.0, angle_dtype=F):
    """x [T, heads, n]: over the first 2 * len(frequencies) coordinates, coordinate 2i is paired with 2i + 1; the
    pair (u, v) at position p becomes (u c - v s, v c + u s) with c, s = magnitude * cos, sin(p * frequency_i).
    Negative positions turn the other way."""
    pairs = frequencies.numel()
    if pairs == 0:
        return x
    angle = (positions.to(angle_dtype)[:, None] * frequencies.to(angle_dtype)[None, :]).to(F)
    c, s = magnitude * torch.cos(angle)[:, None, :], magnitude * torch.sin(angle)[:, None, :]
    u, v = x[..., 0:2 * pairs:2], x[..., 1:2 * pairs:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).reshape(*x.shape[:-1], 2 * pairs)
    return torch.cat([turned, x[..., 2 * pairs:]], dim=-1)


def capped_scores(q, k, scale, temperature, cap):
    """q [T, D], k [T, D] of one head: cap * tanh(scale * temperature * q.k / cap) (cap None or 0: no cap)."""
    s = (q @ k.T) * scale * temperature
    return cap * torch.tanh(s / cap) if cap else s


def sink_softmax(scores):
    """Row i over the keys j <= i, with one more term of score 0 in the denominator that has no value:
    p_ij = exp(s_ij) / (1 + sum_j exp(s_ij))."""
    T = scores.shape[0]
    visible = torch.ones(T, T, dtype=torch.bool).tril()
    s = scores.masked_fill(~visible, -math.inf)
    top = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - top)
    return e / (torch.exp(-top) + e.sum(-1, keepdim=True))


def attention_mixer(h, w, prefix, m, eps, angle_dtype=F):
    """h [T, width] -> [T, width]."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T, dtype=F)
    q = (h @ w[prefix + "q"].to(F).T).reshape(T, H, D)
    k = (h @ w[prefix + "k"].to(F).T).reshape(T, G, D)
    v = (h @ w[prefix + "v"].to(F).T).reshape(T, G, Dv)
    rot = m.get("rot")
    if rot is not None and rot["dims"]:
        f, magnitude = pair_frequencies(rot["dims"], float(rot["base"]), rot.get("scaling"))
        q = rotate_interleaved(q, positions, f, magnitude, angle_dtype)
        k = rotate_interleaved(k, positions, f, magnitude, angle_dtype)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    value_f = None
    if rot is not None:
        value_f, _ = pair_frequencies(Dv, float(rot["base"]))
        v = rotate_interleaved(v, positions, value_f, 1.0, angle_dtype)
    temperature = w[prefix + "temp"].to(F)
    heads = []
    for head in range(H):
        g = head // (H // G)
        p = sink_softmax(capped_scores(q[:, head], k[:, g], m["scale"], temperature[head], m.get("softcap")))
        heads.append(p @ v[:, g])
    o = torch.stack(heads, dim=1)  # [T, H, Dv]
    if value_f is not None:
        o = rotate_interleaved(o, -positions, value_f, 1.0, angle_dtype)
    return o.reshape(T, H * Dv) @ w[prefix + "o"].to(F).T


def lightning_recurrence(q, k, v, decay, start=None):
    """One head, token by token: S_t = decay S_(t-1) + k_t v_t^T from `start` (zeros), o_t = S_t^T q_t."""
    S = torch.zeros(k.shape[1], v.shape[1], dtype=F) if start is None else start.clone()
    out = []
    for t in range(q.shape[0]):
        S = decay * S + torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out), S


def lightning_mixer(h, w, prefix, m, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[prefix + "q"].to(F).T).reshape(T, H, D)
    k = silu(h @ w[prefix + "k"].to(F).T).reshape(T, H, D)
    v = silu(h @ w[prefix + "v"].to(F).T).reshape(T, H, Dv)
    o = torch.stack([lightning_recurrence(q[:, i], k[:, i], v[:, i], float(m["decay"][i]))[0] for i in range(H)], dim=1)
    o = rms_norm(o.reshape(T, H * Dv), w[prefix + "norm"].to(F), eps)
    return (o * sigmoid(h @ w[prefix + "g"].to(F).T)) @ w[prefix + "o"].to(F).T


def dense_feed_forward(h, w, prefix):
    return gelu_tanh(h @ w[prefix + "up"].to(F).T) @ w[prefix + "down"].to(F).T


def expert(h, w, prefix, limit):
    """g = min(Wg h, limit), u = clamp(Wu h, -limit, limit), down(g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ w[prefix + "gate"].to(F).T, max=limit)
    u = torch.clamp(h @ w[prefix + "up"].to(F).T, min=-limit, max=limit)
    return (g * sigmoid(SWISH_SLOPE * g) * (u + 1.0)) @ w[prefix + "down"].to(F).T


def route(h, router, top):
    """The `top` experts with the largest logits per token (ties to the lower index) and the softmax over the
    chosen logits only: indices [T, top], weights [T, top]."""
    z = h @ router.to(F).T
    order = torch.sort(z, dim=-1, descending=True, stable=True)
    chosen, logits = order.indices[:, :top], order.values[:, :top]
    return chosen, torch.softmax(logits, dim=-1)


def route_margin(h, router, top):
    """Per token, how far the last chosen logit lies above the first one left out, in units of the logits' root mean
    square (infinite when every expert is chosen): a small number is a close call that roundings may turn."""
    z = torch.sort(h @ router.to(F).T, dim=-1, descending=True).values
    if top >= z.shape[1]:
        return torch.full((z.shape[0],), math.inf, dtype=F)
    return (z[:, top - 1] - z[:, top]) / torch.sqrt(torch.mean(z ** 2, dim=-1))


def routed_feed_forward(h, w, prefix, mlp, margins=None):
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    chosen, weights = route(h, w[prefix + "router"], top)
    if margins is not None:
        margins.append(route_margin(h, w[prefix + "router"], top))
    out = torch.zeros(h.shape[0], w[prefix + "e0.down"].shape[0], dtype=F)
    for e in range(n):
        rows, slot = (chosen == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += weights[rows, slot][:, None] * expert(h[rows], w, f"{prefix}e{e}.", float(mlp["expert"]["limit"]))
    shared = mlp.get("shared")
    if shared is not None:
        gate = sigmoid(h @ w[prefix + "shared.sg"].to(F).T)  # [T, 1]
        out = out + gate * expert(h, w, prefix + "shared.", float(shared["limit"]))
    return out


def feed_forward(h, w, prefix, mlp, margins=None):
    return dense_feed_forward(h, w, prefix) if mlp["kind"] == "dense" else routed_feed_forward(h, w, prefix, mlp, margins)


def schedule(config):
    """The order in which the layers run: layers start .. stop - 1 `times` times in a row."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def sublayer(streams, w, layer_prefix, which, eps, hyper, function):
    """streams [S, T, width].  With hyper-connections u = sum_s in[s] x_s and x_t <- sum_s mix[s, t] x_s + out[t] y;
    without, the one stream gets x + y."""
    norm = w[f"{layer_prefix}norm{which}"].to(F)
    if not hyper:
        return streams + function(rms_norm(streams[0], norm, eps))[None]
    hc = f"{layer_prefix}hc{which}."
    u = torch.einsum("s,std->td", w[hc + "in"].to(F), streams)
    y = function(rms_norm(u, norm, eps))
    return torch.einsum("sr,std->rtd", w[hc + "mix"].to(F), streams) + w[hc + "out"].to(F)[:, None, None] * y[None]


def forward(config, w, tokens, observe=None, angle_dtype=F, margins=None):
    """tokens: a list of ids -> logits [T, vocab] (float64).  `observe(run, x)` gets the sum of the streams after
    every run of a layer; `margins` (a list) gets, for every run of a mixture of experts, each token's `route_margin`."""
    eps = float(config["norm"]["eps"])
    hyper = "streams" in config
    S = int(config.get("streams", 1))
    x = w["embed"].to(F)[torch.tensor(tokens, dtype=torch.long)]
    streams = x[None].repeat(S, 1, 1)
    for run, index in enumerate(schedule(config)):
        layer, p = config["layers"][index], f"l{index}."
        if layer["type"] == "attention":
            mixer = lambda h: attention_mixer(h, w, p + "mix.", layer["mixer"], eps, angle_dtype)  # noqa: E731
        else:
            mixer = lambda h: lightning_mixer(h, w, p + "mix.", layer["mixer"], eps)  # noqa: E731
        streams = sublayer(streams, w, p, 1, eps, hyper, mixer)
        if layer.get("mlp") is not None:
            streams = sublayer(streams, w, p, 2, eps, hyper, lambda h: feed_forward(h, w, p + "mlp.", layer["mlp"], margins))
        if observe is not None:
            observe(run, streams.sum(0))
    x = rms_norm(streams.sum(0), w["final.norm"].to(F), eps)
    logits = x @ w["head"].to(F).T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits

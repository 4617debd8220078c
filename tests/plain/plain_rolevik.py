"""A plain, slow Rolevik in float64: whole sequences, no cache, one function per mechanism.

It shares nothing with the package: it reads a configuration dictionary (the keys of the design's config.json) and a
dictionary of tensors by their checkpoint names, and walks every recurrence token by token.

The design.  x_0 = E[token] * embedding.scale.  Layer i: x += ls1 * LN1(mixer(x)); x += ls2 * LN2(ff(x)) (the
sublayers read x itself; LN is a layer norm with a gain and no bias; a layer may have no feed-forward).  Mixers:
"parallel" = the mean of an attention over chunks and a gated delta rule, each RMS-normed over the width; "rglru" = a
gated linear recurrence behind a short convolution.  Feed-forwards: dense gated (gelu_tanh) or a mixture of experts with
a softmax router, a choice correction, groups, identity experts and a shared expert.  Logits = E LN(x) * logit_scale.
"""

from __future__ import annotations

import math

import torch

from .plain_llama import read_model_folder  # noqa: F401  (reads config.json and the safetensors file)

F = torch.float64
DELTA_UNIT_EPS = 1e-6  # the delta rule's unit vectors: x / sqrt(sum x^2 + 1e-6)
RGLRU_RATE = 8.0       # log a = -8 r softplus(lam)


def f64(t):
    return t.to(F)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.clamp(z, min=0.0) + torch.log1p(torch.exp(-z.abs()))


def rms_norm(x, gain, eps):
    """Over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def layer_norm(x, gain, eps):
    mean = x.mean(-1, keepdim=True)
    dev = x - mean
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * gain


def rotate_half(x, positions, dims, base):
    """x [T, heads, D]: the first `dims` coordinates of every head turn by position * base^(-2i/dims); coordinate i pairs
    with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = positions.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def chunk_visible(T, size, start=0):
    """[T, T] booleans: query i sees key j <= i when both lie in the same block of `size` positions counted from 0."""
    p = torch.arange(start, start + T)
    return (p[None, :] <= p[:, None]) & ((p[None, :] // size) == (p[:, None] // size))


def chunked_attention(h, w, name, c, eps):
    """The left mixer.  h [T, W]; tensors name + 'q', ...; c the 'left' dictionary."""
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = h @ f64(w[name + "q"]).T + f64(w[name + "q.b"])
    k = h @ f64(w[name + "k"]).T + f64(w[name + "k.b"])
    v = h @ f64(w[name + "v"]).T + f64(w[name + "v.b"])
    q = rms_norm(q, f64(w[name + "q.norm"]), eps)  # over the whole projection, all heads at once
    k = rms_norm(k, f64(w[name + "k.norm"]), eps)
    positions = torch.arange(T)
    rot = c.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_half(q.view(T, H, D), positions, rot["dims"], rot["base"])
    k = rotate_half(k.view(T, G, D), positions, rot["dims"], rot["base"])
    v = v.view(T, G, Dv)
    seen = chunk_visible(T, c["mask"]["size"] if c.get("mask") else T)  # no mask: one chunk holds everything
    out = torch.zeros(T, H, Dv, dtype=F)
    for head in range(H):
        g = head // (H // G)
        score = (q[:, head] @ k[:, g].T) * c["scale"]
        score = score.masked_fill(~seen, float("-inf"))
        out[:, head] = torch.softmax(score, dim=-1) @ v[:, g]
    return out.reshape(T, H * Dv) @ f64(w[name + "o"]).T


def causal_conv(x, taps_w, bias=None):
    """x [T, C], taps_w [C, taps] whose last column meets the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], dim=0)
    out = torch.zeros(T, C, dtype=F)
    for i in range(taps):
        out += padded[i:i + T] * taps_w[:, i][None, :]
    return out if bias is None else out + bias


def gated_delta_rule(h, w, name, c, eps):
    """The right mixer.  Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = silu(causal_conv(h @ f64(w[name + "q"]).T, f64(w[name + "q.conv"]))).view(T, G, D)
    k = silu(causal_conv(h @ f64(w[name + "k"]).T, f64(w[name + "k.conv"]))).view(T, G, D)
    v = silu(causal_conv(h @ f64(w[name + "v"]).T, f64(w[name + "v.conv"]))).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + DELTA_UNIT_EPS) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + DELTA_UNIT_EPS)
    beta = torch.sigmoid(h @ f64(w[name + "b"]).T)
    decay = torch.exp(-torch.exp(f64(w[name + "A_log"])) * softplus(h @ f64(w[name + "a"]).T + f64(w[name + "dt_bias"])))
    gate = silu(h @ f64(w[name + "g"]).T).view(T, H, Dv)
    out = torch.zeros(T, H, Dv, dtype=F)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(D, Dv, dtype=F)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    out = rms_norm(out, f64(w[name + "norm"]), eps) * gate
    return out.reshape(T, H * Dv) @ f64(w[name + "o"]).T


def parallel_mixer(h, w, name, c, eps):
    left = chunked_attention(h, w, name + "left.", c["left"], eps)
    right = gated_delta_rule(h, w, name + "right.", c["right"], eps)
    return 0.5 * (rms_norm(left, f64(w[name + "left.out"]), eps) + rms_norm(right, f64(w[name + "right.out"]), eps))


def rglru_mixer(h, w, name, c):
    T = h.shape[0]
    width, blocks = c["width"], c["blocks"]
    y = gelu_tanh(h @ f64(w[name + "y"]).T + f64(w[name + "y.b"]))
    u = causal_conv(h @ f64(w[name + "x"]).T + f64(w[name + "x.b"]), f64(w[name + "conv"]), f64(w[name + "conv.b"]))
    per = width // blocks
    ub = u.view(T, blocks, per)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, f64(w[name + "ra"])) + f64(w[name + "ra.b"])).reshape(T, width)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, f64(w[name + "ri"])) + f64(w[name + "ri.b"])).reshape(T, width)
    a = torch.exp(-RGLRU_RATE * r * softplus(f64(w[name + "lam"])))
    S = torch.zeros(width, dtype=F)
    out = torch.zeros(T, width, dtype=F)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ f64(w[name + "o"]).T


def gated_ff(h, w, name, act):
    return (act(h @ f64(w[name + "gate"]).T) * (h @ f64(w[name + "up"]).T)) @ f64(w[name + "down"]).T


def route(h, w, name, c):
    """(chosen [T, top], weights [T, top], margin [T]): the experts every token uses, the weights of their results, and how
    clear the decision was: the smaller of (last chosen choice score - best one left out) and (last kept group's score - best
    group left out), as a fraction of the spread of the token's choice scores."""
    r = c["router"]
    experts, identity, top = r["experts"], r.get("identity", 0), r["top"]
    total = experts + identity
    z = h @ f64(w[name + "router"]).T
    s = torch.softmax(z, dim=-1)
    choice = s + f64(w[name + "correction"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = total // groups["count"]
    best = choice.view(-1, groups["count"], per).max(-1).values
    by_group = torch.sort(best, dim=-1, descending=True)
    kept = by_group.indices[:, :groups["keep"]]
    open_ = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
    masked = choice.masked_fill(~open_.repeat_interleave(per, dim=1), float("-inf"))
    ordered = torch.sort(masked, dim=-1, descending=True)
    chosen = ordered.indices[:, :top]
    far = torch.full((h.shape[0],), float("inf"), dtype=F)
    margin = ordered.values[:, top - 1] - ordered.values[:, top] if total > top else far
    margin = torch.where(torch.isfinite(margin), margin, far)  # (everything left out lies in a closed group)
    if groups["keep"] < groups["count"]:
        margin = torch.minimum(margin, by_group.values[:, groups["keep"] - 1] - by_group.values[:, groups["keep"]])
    spread = choice.std(-1).clamp_min(1e-30) if total > 1 else torch.ones_like(far)
    return chosen, torch.gather(s, 1, chosen) * r["scale"], margin / spread


def moe_ff(h, w, name, c):
    experts = c["router"]["experts"]
    chosen, weights, _ = route(h, w, name, c)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(chosen[t].tolist(), weights[t]):
            out[t] += p * (h[t] if e >= experts else gated_ff(h[t:t + 1], w, f"{name}e{e}.", silu)[0])
    if c.get("shared") is not None:
        out = out + gated_ff(h, w, name + "shared.", silu)
    return out


def feed_forward(h, w, name, c, margins=None):
    if c["kind"] == "dense":
        return gated_ff(h, w, name, gelu_tanh)
    if margins is not None:
        margins.append(route(h, w, name, c)[2])
    return moe_ff(h, w, name, c)


def forward(config, w, tokens, return_layers=False, margins=None):
    """Logits [T, vocab] of one sequence (and, if asked, the stream after every layer [layers, T, W]).  `margins` (a list)
    receives, per layer with experts, how clear every token's router decision was (see `route`)."""
    eps = config["norm"]["eps"]
    table = f64(w["embed"])
    x = table[torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    layers = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        if layer["type"] == "parallel":
            m = parallel_mixer(x, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "rglru":
            m = rglru_mixer(x, w, p + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        x = x + f64(w[p + "ls1"]) * layer_norm(m, f64(w[p + "norm1"]), eps)
        if layer.get("mlp") is not None:
            x = x + f64(w[p + "ls2"]) * layer_norm(feed_forward(x, w, p + "mlp.", layer["mlp"], margins), f64(w[p + "norm2"]), eps)
        layers.append(x.clone())
    logits = layer_norm(x, f64(w["final.norm"]), eps) @ table.T * config["logit_scale"]
    return (logits, torch.stack(layers)) if return_layers else logits

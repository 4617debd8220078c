"""Small Rolevik configurations for the tests.  They differ from one another in every size and constant, and between their
own layers: the order of the mixers, head counts (one head, one key/value head, as many as heads, other counts left and
right), key and value sizes (equal, unequal, no multiples of 8), chunks of 1, of 5, of 64, of 100 and none, rotation of part
of a head, of a whole head and none, 1 to 5 convolution weights, one block and several, dense feed-forwards, experts with and
without identity experts, groups, a shared expert, one expert per token and many, layers without a feed-forward, scales of 1
and others, and widths the tensor-core products do not take."""

from __future__ import annotations

from pathlib import Path

import torch

from plain import plain_rolevik


def moe(experts, identity, top, scale, groups, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "identity": identity, "top": top, "scale": scale, "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def dense(ff):
    return {"kind": "dense", "ff": ff}


def parallel(left, right, mlp):
    """left: (heads, kv_heads, dim, vdim, scale, chunk or None, rot or None); right: (heads, kv_heads, dim, vdim, taps)."""
    h, g, d, dv, scale, chunk, rot = left
    l = {"heads": h, "kv_heads": g, "dim": d, "vdim": dv, "scale": scale}
    if chunk is not None:
        l["mask"] = {"size": chunk}
    if rot is not None:
        l["rot"] = {"dims": rot[0], "base": rot[1]}
    h, g, d, dv, taps = right
    return {"type": "parallel", "mixer": {"left": l, "right": {"heads": h, "kv_heads": g, "dim": d, "vdim": dv, "conv": taps}}, "mlp": mlp}


def rglru(width, blocks, taps, mlp):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": taps}, "mlp": mlp}


def model(vocab, width, eps, embedding_scale, logit_scale, layers):
    return {"architecture": "Rolevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embedding_scale},
            "logit_scale": logit_scale, "layers": layers}


RLV_A = model(210, 64, 1e-5, 2.0, 0.25, [
    rglru(48, 3, 3, dense(96)),
    parallel((4, 2, 16, 8, 0.3, 5, (8, 10000.0)), (2, 1, 16, 24, 4), moe(6, 2, 2, 1.5, (4, 2), 40, 24)),
    parallel((2, 2, 24, 24, 0.2, 64, (24, 500.0)), (3, 3, 8, 8, 2), None),
    rglru(40, 1, 1, moe(4, 0, 1, 1.0, (1, 1), 20)),
])

RLV_B = model(150, 72, 1e-6, 1.0, 1.0, [
    parallel((3, 1, 20, 12, 0.22, 100, (10, 3000.0)), (4, 2, 12, 6, 5), moe(5, 3, 3, 2.5, (2, 2), 36, 16)),
    rglru(72, 6, 4, None),
    parallel((1, 1, 8, 40, 0.35, None, None), (1, 1, 32, 32, 1), dense(50)),
    parallel((3, 3, 16, 10, 0.3, 1, (0, 100.0)), (2, 2, 10, 20, 3), moe(3, 1, 4, 0.7, (1, 1), 20)),
])

# sizes at which the tensor-core products and the tensor-core attention run
RLV_C = model(512, 256, 1e-5, 0.7, 0.5, [
    parallel((8, 2, 64, 128, 0.125, 96, (32, 100000.0)), (4, 2, 64, 128, 4), moe(8, 4, 2, 2.0, (3, 2), 128, 64)),
    rglru(256, 2, 4, dense(512)),
    parallel((4, 4, 32, 64, 0.17, 48, (32, 10000.0)), (8, 4, 32, 32, 4), dense(256)),
])

# a width and head sizes that are no multiples of 8
RLV_D = model(131, 50, 3e-6, 1.3, 2.0, [
    parallel((6, 3, 18, 14, 0.24, 7, (6, 3000.0)), (6, 2, 18, 10, 4), moe(5, 2, 2, 1.0, (7, 3), 33, 7)),
    rglru(33, 3, 2, moe(7, 0, 3, 3.0, (7, 4), 12)),
    parallel((2, 1, 12, 6, 0.3, 33, (12, 50.0)), (1, 1, 6, 14, 3), dense(40)),
])

RLV = {"A": RLV_A, "B": RLV_B, "C": RLV_C, "D": RLV_D}


def make_folder(raw: dict, seed: int, root, std: float = 0.15) -> Path:
    """A folder with random weights.  Some tensors are then drawn anew so that they matter: convolution weights of both signs
    and of size one, recurrences that forget slowly and quickly (so that a lost state shows), decays and write strengths away
    from their ends, layer scales between 0.5 and 1.5, a router sharp enough to decide, corrections that change choices."""
    from models_b200.config import config_from_dict
    from models_b200.weights import write_random_model
    from models_b200.weights.safetensors_io import write_safetensors

    folder = Path(root) / f"rolevik_{seed}"
    write_random_model(folder, config_from_dict(raw), seed, std=std, gain_std=0.1, dtype=torch.bfloat16)
    _, weights = plain_rolevik.read_model_folder(folder)
    g = torch.Generator().manual_seed(seed)
    for name in list(weights):
        shape = weights[name].shape
        uniform = lambda lo, hi: torch.rand(shape, generator=g) * (hi - lo) + lo  # noqa: E731
        if name.endswith(".conv"):
            t = torch.randn(shape, generator=g) * 0.6
        elif name.endswith(".lam"):
            t = uniform(-6.0, 0.5)
        elif name.endswith(".A_log"):
            t = uniform(-3.0, 0.5)
        elif name.endswith(".dt_bias"):
            t = uniform(-2.0, 1.0)
        elif name.endswith(".ls1") or name.endswith(".ls2"):
            t = uniform(0.5, 1.5)
        elif name.endswith(".mlp.router") or name.endswith(".right.a") or name.endswith(".right.b"):
            t = torch.randn(shape, generator=g) * 0.5
        elif name.endswith(".correction"):
            t = torch.randn(shape, generator=g) * 0.05
        elif name.endswith(".b") and weights[name].dim() <= 2 and ".left." in name or name.endswith((".y.b", ".x.b", ".conv.b", ".ra.b", ".ri.b")):
            t = torch.randn(shape, generator=g) * 0.3
        else:
            continue
        weights[name] = t.to(torch.bfloat16)
    write_safetensors(folder / "model.safetensors", {n: t.contiguous() for n, t in weights.items()}, {"format": "pt"})
    return folder


CLOSE_CALL = 0.05  # of the spread of a token's choice scores


def plain_logits(folder, tokens, layers_out=None) -> torch.Tensor:
    config, weights = plain_rolevik.read_model_folder(folder)
    if layers_out is None:
        return plain_rolevik.forward(config, weights, list(tokens))
    logits, layers = plain_rolevik.forward(config, weights, list(tokens), return_layers=True)
    layers_out.extend(layers)
    return logits


def plain_logits_and_sure(folder, tokens):
    """The logits, and per position whether every router decision of that token and of all tokens before it was clear of a
    close call: in bfloat16 the roundings of the router's input may turn a close one; that token then runs through another
    expert, and every later token reads it through the cache and the recurrent state."""
    config, weights = plain_rolevik.read_model_folder(folder)
    margins = []
    logits = plain_rolevik.forward(config, weights, list(tokens), margins=margins)
    sure = torch.ones(len(tokens), dtype=torch.bool)
    for m in margins:
        sure &= m >= CLOSE_CALL
    return logits, torch.cumprod(sure.to(torch.int64), dim=0).bool()

"""Small Kivezen configurations for the tests.  They differ from one another in every size and constant, and between
their own layers: the order of the mixers, 3, 2, 1 and no residual streams, a looped span in the middle, at the start
and none, head counts (one head, one key/value head, as many key/value heads as heads), key and value sizes (equal,
unequal, no multiples of 8), rotation of part of a head, of a whole head, stretched and not, and none at all, a score
cap small enough to bend every score and none, decays of 1 and below, experts with and without a shared one, one expert
per token and all of them, layers without a feed-forward, and widths the tensor-core products do not take."""

from __future__ import annotations

from pathlib import Path

import torch

from plain import plain_kivezen


def moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def dense(ff):
    return {"kind": "dense", "ff": ff}


def lightning(heads, dim, vdim, decay, mlp):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, scale, rot, softcap, mlp):
    """rot: None, or (dims, base) or (dims, base, (factor, original, fast, slow))."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        mixer["softcap"] = softcap
    if rot is not None:
        mixer["rot"] = {"dims": rot[0], "base": rot[1]}
        if len(rot) > 2:
            mixer["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot[2]))
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


KVZ_A = {
    "architecture": "Kivezen", "vocab": 210, "width": 64, "norm": {"eps": 1e-5}, "streams": 3, "logit_softcap": 20.0,
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [lightning(2, 16, 24, [0.9, 0.995], dense(96)),
               attention(4, 2, 16, 8, 0.25, (8, 10000.0, (8.0, 64, 4.0, 1.0)), 30.0, moe(6, 2, 40, 3.0, (24, 1.5))),
               attention(2, 2, 24, 24, 0.2, (24, 500.0), None, dense(72)),
               lightning(1, 32, 32, [1.0], None)],
}

KVZ_B = {
    "architecture": "Kivezen", "vocab": 150, "width": 72, "norm": {"eps": 1e-6},
    "layers": [attention(3, 1, 20, 12, 0.22, (10, 3000.0, (2.0, 32, 8.0, 2.0)), 12.0, moe(4, 1, 36, 2.5)),
               lightning(3, 10, 6, [0.5, 0.25, 0.99], dense(50)),
               attention(1, 1, 8, 40, 0.35, None, 2.0, moe(3, 3, 20, 1.0, (16, 4.0))),
               attention(3, 3, 16, 10, 0.3, (0, 100.0), None, None)],
}

# sizes at which the tensor-core products and the tensor-core attention run
KVZ_C = {
    "architecture": "Kivezen", "vocab": 512, "width": 256, "norm": {"eps": 1e-5}, "streams": 2, "logit_softcap": 40.0,
    "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [attention(8, 2, 64, 128, 0.125, (32, 100000.0, (4.0, 128, 16.0, 1.0)), 25.0, moe(8, 2, 128, 2.0, (64, 2.0))),
               lightning(4, 64, 128, [0.97, 0.99, 0.999, 0.9], dense(512)),
               attention(4, 4, 64, 128, 0.125, (64, 10000.0), 50.0, dense(256))],
}

# a width and head sizes that are no multiples of 8, one stream with its connections, a loop that runs once
KVZ_D = {
    "architecture": "Kivezen", "vocab": 131, "width": 50, "norm": {"eps": 3e-6}, "streams": 1, "logit_softcap": 8.0,
    "loop": {"start": 0, "stop": 1, "times": 1},
    "layers": [attention(6, 3, 18, 14, 0.24, (6, 3000.0), 9.0, moe(5, 2, 33, 2.0, (7, 1.0))),
               lightning(2, 18, 10, [0.9, 0.97], moe(7, 3, 12, 5.0)),
               attention(2, 1, 12, 6, 0.3, (12, 50.0, (3.0, 16, 2.0, 0.5)), None, dense(40))],
}

KVZ = {"A": KVZ_A, "B": KVZ_B, "C": KVZ_C, "D": KVZ_D}


def make_folder(raw: dict, seed: int, root, std: float = 0.15) -> Path:
    """A folder with random weights.  The numbers of the hyper-connections and the heads' temperatures are then drawn
    anew so that they matter: reading weights of both signs, a mixing matrix that is far from the identity but does not
    blow the streams up, temperatures between 0.5 and 1.5."""
    from models_b200.config import config_from_dict
    from models_b200.weights import write_random_model
    from models_b200.weights.safetensors_io import write_safetensors

    folder = Path(root) / f"kivezen_{seed}"
    write_random_model(folder, config_from_dict(raw), seed, std=std, gain_std=0.1, dtype=torch.bfloat16)
    _, weights = plain_kivezen.read_model_folder(folder)
    g = torch.Generator().manual_seed(seed)
    S = raw.get("streams", 0)
    for name in list(weights):
        kind = name.rsplit(".", 1)[-1]
        if ".hc" in name:
            if kind == "mix":
                t = torch.eye(S) * 0.7 + (torch.rand(S, S, generator=g) - 0.3) * 0.5
            elif kind == "in":
                t = (torch.rand(S, generator=g) + 0.3) * (1.0 if S == 1 else torch.tensor([(1.0, -0.6, 0.8, 0.5)[i % 4] for i in range(S)]))
            else:
                t = torch.rand(S, generator=g) + 0.5
            weights[name] = t.to(torch.bfloat16)
        elif kind == "temp":
            weights[name] = (torch.rand(weights[name].shape, generator=g) + 0.5).to(torch.bfloat16)
    write_safetensors(folder / "model.safetensors", {n: t.contiguous() for n, t in weights.items()}, {"format": "pt"})
    return folder


def plain_logits(folder, tokens, hidden_out=None, margins=None) -> torch.Tensor:
    config, weights = plain_kivezen.read_model_folder(folder)
    observe = None if hidden_out is None else (lambda run, x: hidden_out.append(x.clone()))
    return plain_kivezen.forward(config, weights, list(tokens), observe, margins=margins)


CLOSE_CALL = 0.05  # of the router logits' root mean square


def plain_logits_and_sure(folder, tokens):
    """The logits, and per position whether every router decision of that token and of all tokens before it was clear of
    a close call: in bfloat16 the roundings of the router's input may turn a close one; that token then runs through
    another expert, and every later token reads it through the cache and the recurrent state."""
    margins = []
    logits = plain_logits(folder, tokens, margins=margins)
    sure = torch.ones(len(tokens), dtype=torch.bool)
    for m in margins:
        sure &= m >= CLOSE_CALL
    return logits, torch.cumprod(sure.to(torch.int64), dim=0).bool()

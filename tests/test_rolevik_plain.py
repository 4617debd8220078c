"""Rolevik without a GPU: the configuration reader (round trip, refusals, the tensors a model asks for), and the plain
implementation against cases worked out by hand and against itself (a prefix of a sequence gives the prefix of its logits)."""

import math

import pytest
import torch

from plain import plain_rolevik as pr
from tiny import random_tokens
from tiny_rolevik import RLV, dense, make_folder, model, moe, parallel, rglru

F = torch.float64


@pytest.mark.parametrize("name", sorted(RLV))
def test_configuration_round_trip_and_tensors(name):
    from models_b200.config import config_from_dict
    from models_b200.engine.model import parameter_requests

    raw = RLV[name]
    config = config_from_dict(raw)
    assert config.to_dict() == raw
    spec = config.model_spec()
    assert spec.head.tied and spec.head.logit_scale == raw["logit_scale"] and spec.embedding.scale == raw["embedding"]["scale"]
    requests = parameter_requests(spec)
    assert "embed" in requests and "final.norm" in requests and "head" not in requests
    for i, layer in enumerate(raw["layers"]):
        p = f"l{i}."
        assert requests[p + "norm1"].shape == (raw["width"],) and requests[p + "ls1"].shape == (raw["width"],)
        assert ((p + "norm2") in requests) == (layer["mlp"] is not None) == ((p + "ls2") in requests)
        if layer["type"] == "parallel":
            left, right = layer["mixer"]["left"], layer["mixer"]["right"]
            assert requests[p + "mix.left.q.norm"].shape == (left["heads"] * left["dim"],)
            assert requests[p + "mix.left.k.b"].shape == (left["kv_heads"] * left["dim"],)
            assert requests[p + "mix.left.o"].shape == (raw["width"], left["heads"] * left["vdim"])
            assert requests[p + "mix.right.k.conv"].shape == (right["kv_heads"] * right["dim"], right["conv"])
            assert requests[p + "mix.right.norm"].shape == (right["vdim"],)
            assert requests[p + "mix.right.A_log"].shape == (right["heads"],)
        else:
            m = layer["mixer"]
            assert requests[p + "mix.ra"].shape == (m["blocks"], m["width"] // m["blocks"], m["width"] // m["blocks"])
            assert requests[p + "mix.conv"].shape == (m["width"], m["conv"])
        if layer["mlp"] and layer["mlp"]["kind"] == "moe":
            r = layer["mlp"]["router"]
            assert requests[p + "mlp.router"].shape == (r["experts"] + r["identity"], raw["width"])
            assert requests[p + "mlp.correction"].shape == (r["experts"] + r["identity"],)
            assert (p + f"mlp.e{r['experts'] - 1}.down") in requests and (p + f"mlp.e{r['experts']}.down") not in requests
            assert ((p + "mlp.shared.up") in requests) == ("shared" in layer["mlp"])


def test_configurations_that_are_refused():
    from models_b200.config import ConfigError, config_from_dict

    good = model(50, 16, 1e-5, 1.0, 1.0, [parallel((2, 1, 8, 8, 0.3, 4, (4, 100.0)), (2, 1, 8, 8, 2), moe(4, 2, 2, 1.0, (3, 2), 8))])
    config_from_dict(good)
    for change in (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3, kv_heads=2),
                   lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=10),
                   lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4),     # 6 outputs in 4 groups
                   lambda c: c["layers"][0]["mlp"]["router"].update(top=5),                  # more than the kept groups hold
                   lambda c: c["layers"][0].update(type="other"),
                   lambda c: c["layers"].append(rglru(10, 3, 2, None)),                      # 10 channels in 3 blocks
                   lambda c: c.pop("vocab")):
        import copy
        bad = copy.deepcopy(good)
        change(bad)
        with pytest.raises(ConfigError):
            config_from_dict(bad)


def test_chunks_are_counted_from_position_zero():
    seen = pr.chunk_visible(7, 3)
    assert seen.tolist() == [[j <= i and j // 3 == i // 3 for j in range(7)] for i in range(7)]
    assert pr.chunk_visible(4, 3, start=2).tolist() == [[True, False, False, False], [False, True, False, False],
                                                        [False, True, True, False], [False, True, True, True]]


def test_convolution_meets_the_current_token_with_its_last_weight():
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=F)
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=F)
    assert pr.causal_conv(x, w).flatten().tolist() == [1.0, 12.0, 124.0]
    assert pr.causal_conv(x, w, torch.tensor([0.5], dtype=F)).flatten().tolist() == [1.5, 12.5, 124.5]


def test_router_by_hand():
    """Six outputs in three groups of which two are kept; a correction lifts output 5 into the choice but not into the weights;
    the last two outputs are identity experts."""
    c = {"kind": "moe", "expert": {"ff": 2}, "router": {"experts": 4, "identity": 2, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 2}}}
    z = torch.tensor([[2.0, 0.0, 1.9, 1.8, 0.0, 0.5]], dtype=F)
    w = {"f.router": torch.eye(6, dtype=F), "f.correction": torch.tensor([0, 0, 0, 0, 0, 0.3], dtype=F)}
    s = torch.softmax(z, -1)[0]
    chosen, weights, margin = pr.route(z, w, "f.", c)
    # groups' best choice scores: {0,1}: s0; {2,3}: s2; {4,5}: s5 + 0.3, the largest; kept: {4,5} and {0,1}; chosen: 5, then 0
    assert chosen.tolist() == [[5, 0]]
    assert torch.allclose(weights[0], torch.stack([s[5], s[0]]) * 2.0)
    assert float(margin) > 0
    # the identity expert returns its input: with zero expert matrices the result is weight_5 * h
    for e in range(4):
        w.update({f"f.e{e}.gate": torch.zeros(2, 6, dtype=F), f"f.e{e}.up": torch.zeros(2, 6, dtype=F), f"f.e{e}.down": torch.zeros(6, 2, dtype=F)})
    assert torch.allclose(pr.moe_ff(z, w, "f.", c), weights[0, 0] * z)


def test_recurrences_by_hand():
    # one channel, a = exp(-8 * sigmoid(0) * softplus(lam)); r and i gates see u through 1 x 1 matrices
    lam = math.log(math.e - 1.0)  # softplus(lam) = 1
    w = {"m.y": torch.zeros(1, 1, dtype=F), "m.y.b": torch.tensor([10.0], dtype=F), "m.x": torch.ones(1, 1, dtype=F), "m.x.b": torch.zeros(1, dtype=F),
         "m.conv": torch.ones(1, 1, dtype=F), "m.conv.b": torch.zeros(1, dtype=F), "m.ra": torch.zeros(1, 1, 1, dtype=F), "m.ra.b": torch.zeros(1, 1, dtype=F),
         "m.ri": torch.zeros(1, 1, 1, dtype=F), "m.ri.b": torch.full((1, 1), 50.0, dtype=F), "m.lam": torch.tensor([lam], dtype=F), "m.o": torch.ones(1, 1, dtype=F)}
    x = torch.tensor([[1.0], [0.0], [2.0]], dtype=F)
    a = math.exp(-4.0)
    g = math.sqrt(1 - a * a)
    want = [g * 1.0, a * g, a * a * g + 2 * g]
    got = pr.rglru_mixer(x, w, "m.", {"width": 1, "blocks": 1}).flatten()
    assert torch.allclose(got, torch.tensor(want, dtype=F) * float(pr.gelu_tanh(torch.tensor(10.0, dtype=F))), rtol=1e-12)
    # delta rule, one head of one key coordinate and one value: S is a number; k = 1 after the unit norm, q = 1
    big = 1e3
    w = {"m.q": torch.full((1, 1), big, dtype=F), "m.k": torch.full((1, 1), big, dtype=F), "m.v": torch.ones(1, 1, dtype=F),
         "m.q.conv": torch.ones(1, 1, dtype=F), "m.k.conv": torch.ones(1, 1, dtype=F), "m.v.conv": torch.ones(1, 1, dtype=F),
         "m.b": torch.zeros(1, 1, dtype=F), "m.a": torch.zeros(1, 1, dtype=F), "m.A_log": torch.zeros(1, dtype=F), "m.dt_bias": torch.tensor([lam], dtype=F),
         "m.g": torch.ones(1, 1, dtype=F), "m.norm": torch.ones(1, dtype=F), "m.o": torch.ones(1, 1, dtype=F)}
    x = torch.tensor([[1.0], [3.0]], dtype=F)
    v = pr.silu(x.flatten())
    decay, beta = math.exp(-1.0), 0.5
    s1 = beta * float(v[0])
    s2 = decay * s1 + beta * (float(v[1]) - decay * s1)
    got = pr.gated_delta_rule(x, w, "m.", {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1}, 0.0).flatten()
    # o / rms(o) is the sign of o; times silu(g)
    assert torch.allclose(got, torch.sign(torch.tensor([s1, s2], dtype=F)) * pr.silu(x.flatten()), rtol=1e-9)


@pytest.mark.parametrize("name", ["A", "B"])
def test_a_prefix_gives_the_prefix_of_the_logits(tmp_path, name):
    folder = make_folder(RLV[name], 5, tmp_path)
    config, weights = pr.read_model_folder(folder)
    tokens = random_tokens(RLV[name]["vocab"], 30, 3)
    whole = pr.forward(config, weights, tokens)
    assert torch.allclose(pr.forward(config, weights, tokens[:11]), whole[:11], rtol=1e-9, atol=1e-12)
    assert bool(torch.isfinite(whole).all())

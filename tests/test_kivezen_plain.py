"""Kivezen without a GPU: the configuration reader, the plain implementation against cases worked out by hand, the
cache and state a model of the design asks for (a looped layer once per pass), and a random model folder read back."""

import copy
import math

import pytest
import torch

from plain import plain_kivezen as pk
from tiny_kivezen import KVZ, attention, dense, lightning, moe

F = torch.float64


def test_the_configuration_reads_every_constant_and_round_trips():
    from models_b200.config import config_from_dict

    for raw in KVZ.values():
        config = config_from_dict(raw)
        assert config_from_dict(config.to_dict()) == config
        spec = config.model_spec()
        assert [e.layer for e in spec.schedule] == pk.schedule(raw)
        assert spec.residual_streams == max(1, raw.get("streams", 0)) and spec.head.softcap == raw.get("logit_softcap", 0.0)
        for layer, block in zip(raw["layers"], spec.layers):
            m = layer["mixer"]
            assert block.streams == raw.get("streams", 0)
            assert (block.feed_forward is None) == (layer["mlp"] is None) == (block.feed_forward_norm is None)
            if layer["type"] == "lightning":
                assert block.mixer.kind == "retention" and block.mixer.decay == tuple(m["decay"]) and block.mixer.key_scale == 1.0
                assert block.mixer.position is None and block.mixer.input_activation == "silu" and block.mixer.norm == "all"
            else:
                a = block.mixer
                assert a.kind == "capped_attention" and a.sink and a.unit_norm and a.head_temperature
                assert (a.scale, a.softcap, a.value_dim) == (m["scale"], m.get("softcap", 0.0), m["vdim"])
                rot = m.get("rot")
                assert (a.value_position is None) == (rot is None)
                assert (a.position is None) == (rot is None or rot["dims"] == 0)
                if rot is not None:
                    assert (a.value_position.rotary_dim, a.value_position.theta, a.value_position.scaling) == (m["vdim"], rot["base"], None)
                if a.position is not None:
                    assert (a.position.rotary_dim, a.position.theta, a.position.pairing) == (rot["dims"], rot["base"], "interleaved")
                    assert (a.position.scaling is None) == ("scaling" not in rot)
                    if "scaling" in rot:
                        assert a.position.scaling.magnitude == pytest.approx(0.1 * math.log(rot["scaling"]["factor"]) + 1.0)
            f = layer["mlp"]
            if f is not None and f["kind"] == "moe":
                ff = block.feed_forward
                assert (ff.num_experts, ff.top, ff.expert.limit) == (f["router"]["experts"], f["router"]["top"], f["expert"]["limit"])
                assert (ff.shared is None) == ("shared" not in f) and ff.expert.swish_slope == pk.SWISH_SLOPE


def test_the_configuration_names_what_is_wrong():
    from models_b200.config import ConfigError, config_from_dict

    def changed(edit):
        raw = copy.deepcopy(KVZ["A"])
        edit(raw)
        return raw

    for edit, message in (
            (lambda r: r["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
            (lambda r: r["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
            (lambda r: r["layers"][2].update(type="convolution"), "not built"),
            (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
            (lambda r: r["layers"][1]["mlp"]["router"].update(top=9), "top"),
            (lambda r: r["layers"][1]["mlp"].update(kind="sparse"), "not built"),
            (lambda r: r["loop"].update(stop=9), "loop"),
            (lambda r: r["layers"][1]["mixer"].pop("scale"), "scale"),
            (lambda r: r["norm"].pop("eps"), "eps")):
        with pytest.raises(ConfigError, match=message):
            config_from_dict(changed(edit))


def test_stretched_frequencies_by_hand():
    """8 pairs over base 10000, made for 64 positions, fast 4, slow 1: pair(t) = 16 ln(64 / (2 pi t)) / (2 ln 10000), so
    lo = floor(pair(4)) = 0 and hi = ceil(pair(1)) = 3: pair 0 keeps its frequency, pairs 3.. are divided by the factor."""
    f, magnitude = pk.pair_frequencies(16, 10000.0, {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 1.0})
    plain = torch.tensor([10000.0 ** (-2 * i / 16) for i in range(8)], dtype=F)
    ramp = torch.tensor([0.0, 1 / 3, 2 / 3] + [1.0] * 5, dtype=F)
    assert torch.allclose(f, plain / 8.0 * ramp + plain * (1 - ramp), rtol=1e-12)
    assert magnitude == pytest.approx(0.1 * math.log(8.0) + 1.0)
    f, magnitude = pk.pair_frequencies(16, 10000.0)
    assert torch.allclose(f, plain) and magnitude == 1.0


def test_rotation_by_hand_and_back():
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0]]], dtype=F)  # pairs (1, 0) and (0, 2); the fifth coordinate passes
    f = torch.tensor([math.pi / 2, math.pi], dtype=F)
    y = pk.rotate_interleaved(x, torch.tensor([1.0], dtype=F), f, 2.0)
    assert torch.allclose(y, torch.tensor([[[0.0, 2.0, 0.0, -4.0, 5.0]]], dtype=F), atol=1e-12)
    g = torch.Generator().manual_seed(0)
    v = torch.randn(5, 2, 6, generator=g, dtype=F)
    p = torch.arange(5, dtype=F) + 3
    f = pk.pair_frequencies(6, 50.0)[0]
    assert torch.allclose(pk.rotate_interleaved(pk.rotate_interleaved(v, p, f), -p, f), v, atol=1e-12)


def test_sink_and_cap_by_hand():
    s = torch.tensor([[0.0, 9.0], [math.log(3.0), math.log(4.0)]], dtype=F)
    p = pk.sink_softmax(s)
    assert torch.allclose(p, torch.tensor([[0.5, 0.0], [3 / 8, 4 / 8]], dtype=F), atol=1e-12)
    big = pk.sink_softmax(torch.tensor([[-800.0]], dtype=F))  # the sink takes everything, nothing overflows
    assert float(big) == 0.0
    q, k = torch.tensor([[100.0, 0.0]], dtype=F), torch.tensor([[1.0, 0.0]], dtype=F)
    assert float(pk.capped_scores(q, k, 0.5, 2.0, 5.0)) == pytest.approx(5.0 * math.tanh(20.0))
    assert float(pk.capped_scores(q, k, 0.5, 2.0, None)) == 100.0


def test_a_value_reaches_the_result_turned_by_its_distance():
    """Values cached turned by j and sums turned back by i: o_i = sum_j p_ij R((j - i) f) v_j, with the weights of the
    rotated, normed queries and keys; at position 0 nothing is turned."""
    g = torch.Generator().manual_seed(3)
    m = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 6, "scale": 0.4, "softcap": 6.0, "rot": {"dims": 4, "base": 30.0}}
    w = {"q": torch.randn(16, 12, generator=g, dtype=F), "k": torch.randn(8, 12, generator=g, dtype=F),
         "v": torch.randn(6, 12, generator=g, dtype=F), "o": torch.eye(12, dtype=F), "temp": torch.tensor([0.7, 1.3], dtype=F)}
    T = 9
    h = torch.randn(T, 12, generator=g, dtype=F)
    whole = pk.attention_mixer(h, w, "", m, 1e-5).reshape(T, 2, 6)
    positions = torch.arange(T, dtype=F)
    f = pk.pair_frequencies(4, 30.0)[0]
    q = pk.rms_norm(pk.rotate_interleaved((h @ w["q"].T).reshape(T, 2, 8), positions, f), None, 1e-5)
    k = pk.rms_norm(pk.rotate_interleaved((h @ w["k"].T).reshape(T, 1, 8), positions, f), None, 1e-5)
    v = (h @ w["v"].T).reshape(T, 1, 6)
    vf = pk.pair_frequencies(6, 30.0)[0]
    for head in range(2):
        weights = pk.sink_softmax(pk.capped_scores(q[:, head], k[:, 0], 0.4, w["temp"][head], 6.0))
        for i in range(T):
            turned = pk.rotate_interleaved(v, positions - i, vf)[:, 0]  # row j turned by j - i
            assert torch.allclose(whole[i, head], weights[i] @ turned, atol=1e-12)
    no_rot = {key: value for key, value in m.items() if key != "rot"}
    assert torch.allclose(whole[0].reshape(-1), pk.attention_mixer(h[:1], w, "", no_rot, 1e-5)[0], atol=1e-12)


def test_the_lightning_recurrence_in_closed_form_and_carried():
    g = torch.Generator().manual_seed(1)
    q, k, v = torch.randn(7, 4, generator=g, dtype=F), torch.randn(7, 4, generator=g, dtype=F), torch.randn(7, 3, generator=g, dtype=F)
    out, state = pk.lightning_recurrence(q, k, v, 0.8)
    for t in range(7):
        want = sum(0.8 ** (t - j) * float(q[t] @ k[j]) * v[j] for j in range(t + 1))
        assert torch.allclose(out[t], want, atol=1e-12)
    first, mid = pk.lightning_recurrence(q[:3], k[:3], v[:3], 0.8)
    rest, last = pk.lightning_recurrence(q[3:], k[3:], v[3:], 0.8, mid)
    assert torch.allclose(torch.cat([first, rest]), out, atol=1e-12) and torch.allclose(last, state, atol=1e-12)


def test_routing_by_hand():
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F)
    router = torch.tensor([[1.0, 5.0], [3.0, 5.0], [2.0, 0.0], [3.0, -1.0]], dtype=F)
    chosen, weights = pk.route(h, router, 2)
    assert chosen.tolist() == [[1, 3], [0, 1]]  # ties go to the lower index
    assert torch.allclose(weights, torch.tensor([[0.5, 0.5], [0.5, 0.5]], dtype=F))
    chosen, weights = pk.route(h, router, 3)
    e = torch.tensor([math.exp(3.0), math.exp(3.0), math.exp(2.0)], dtype=F)
    assert chosen[0].tolist() == [1, 3, 2] and torch.allclose(weights[0], e / e.sum())
    margins = pk.route_margin(h, router, 2)
    assert float(margins[0]) == pytest.approx(1.0 / math.sqrt((1 + 9 + 4 + 9) / 4)) and math.isinf(float(pk.route_margin(h, router, 4)[0]))


def test_an_expert_by_hand():
    w = {"gate": torch.tensor([[1.0], [1.0]], dtype=F), "up": torch.tensor([[1.0], [-1.0]], dtype=F), "down": torch.tensor([[1.0, 10.0]], dtype=F)}
    y = pk.expert(torch.tensor([[3.0]], dtype=F), w, "", 2.0)  # g = min(3, 2) = 2 twice, u = 2 and -2
    s = 2.0 / (1.0 + math.exp(-pk.SWISH_SLOPE * 2.0))
    assert float(y) == pytest.approx(s * 3.0 + 10.0 * s * -1.0)


def test_one_stream_with_unit_connections_is_the_plain_residual_sum():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1, 5, 8, generator=g, dtype=F)
    w = {"l0.norm1": torch.rand(8, generator=g, dtype=F), "l0.hc1.in": torch.ones(1, dtype=F), "l0.hc1.out": torch.ones(1, dtype=F),
         "l0.hc1.mix": torch.ones(1, 1, dtype=F)}
    function = lambda h: h * 3.0 + 1.0  # noqa: E731
    assert torch.allclose(pk.sublayer(x, w, "l0.", 1, 1e-5, True, function), pk.sublayer(x, w, "l0.", 1, 1e-5, False, function))
    # two streams: all copies at once from the old ones, the mixing matrix indexed [from, to]
    x2 = torch.randn(2, 5, 8, generator=g, dtype=F)
    w.update({"l0.hc1.in": torch.tensor([1.0, 0.0], dtype=F), "l0.hc1.out": torch.tensor([0.0, 1.0], dtype=F),
              "l0.hc1.mix": torch.tensor([[0.0, 1.0], [0.0, 0.0]], dtype=F)})
    got = pk.sublayer(x2, w, "l0.", 1, 1e-5, True, function)
    assert float(got[0].abs().max()) == 0.0
    assert torch.allclose(got[1], x2[0] + function(pk.rms_norm(x2[0], w["l0.norm1"], 1e-5)))


def test_the_cache_and_state_a_model_asks_for():
    """Every pass of a looped layer has a cache or a state of its own; attention runs of equal shape share a group of
    pools; a lightning run keeps no pages and a float32 state [heads, dim, vdim] per sequence."""
    from models_b200.cache import KvCache
    from models_b200.config import config_from_dict
    from models_b200.engine.model import DecoderModel
    from models_b200.parts import Runtime

    raw = {"architecture": "Kivezen", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "streams": 2,
           "loop": {"start": 1, "stop": 3, "times": 2},
           "layers": [attention(2, 1, 8, 16, 0.3, (8, 100.0), 9.0, dense(40)), lightning(2, 8, 4, [0.5, 0.9], None),
                      attention(2, 1, 8, 16, 0.2, None, None, moe(4, 2, 12, 1.0, (8, 1.0)))]}
    model = DecoderModel(config_from_dict(raw).model_spec(), Runtime(torch.device("meta"), "float32", max_positions=1))
    requests, states = model.kv_requests(), model.state_requests()
    assert [r is None for r in requests] == [False, True, False, True, False]
    assert requests[0] == requests[2] == requests[4] and (requests[0].head_dim, requests[0].value_head_dim) == (8, 16)
    assert [s is not None for s in states] == [False, True, False, True, False] and states[1].shape == (2, 8, 4)
    cache = KvCache(requests, [None] * 5, max_tokens=256, max_slots=3)
    assert [g.runs for g in cache.groups] == [[0, 2, 4]]


def test_random_model_folder_loads_by_name_and_reports_what_is_wrong(tmp_path):
    import json

    from models_b200.config import load_config
    from models_b200.engine.model import parameter_requests
    from models_b200.weights import WeightsError, load_tensors
    from tiny_kivezen import make_folder

    folder = make_folder(KVZ["B"], 5, tmp_path)
    requests = parameter_requests(load_config(folder).model_spec())
    tensors = load_tensors(folder, requests)
    assert set(tensors) == set(requests)
    assert tensors["l0.mix.temp"].shape == (3,) and tensors["l2.mlp.shared.sg"].shape == (1, 72) and tensors["l1.mix.norm"].shape == (18,)
    assert "l3.norm2" not in tensors and "l0.hc1.in" not in tensors  # no feed-forward in the last layer, one plain stream
    logits = pk.forward(*pk.read_model_folder(folder), [1, 2, 3, 4, 5])
    assert logits.shape == (5, KVZ["B"]["vocab"]) and bool(torch.isfinite(logits).all())
    raw = json.loads((folder / "config.json").read_text())
    raw["layers"][0]["mixer"]["heads"] = 6
    (folder / "config.json").write_text(json.dumps(raw))
    with pytest.raises(WeightsError, match="l0.mix"):
        load_tensors(folder, parameter_requests(load_config(folder).model_spec()))

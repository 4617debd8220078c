"""The Kivezen decoder in the engine against the plain implementation (tests/plain/plain_kivezen.py): each kernel alone
with inputs made so that one key, the sink, the cap, one expert or one stream decides the result, whole prompts, prompts
cut into portions, token-by-token decoding across cache pages, unequal batches, slots, pages and states used again, long
decoding from CUDA graphs, and greedy generation through the public entry point."""

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from plain import plain_kivezen as pk
from tiny import TOLERANCE, random_tokens, scaled_error
from tiny_kivezen import KVZ, attention, dense, lightning, make_folder, moe, plain_logits_and_sure
from tiny_kivezen import plain_logits as plain_logits_alone

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
F = torch.float64


def _engine(folder, dtype, max_tokens=2048, **more):
    from models_b200.engine.loading import engine_from_folder

    return engine_from_folder(folder, dtype, max_tokens, **more)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("kivezen")
    return {name: make_folder(raw, seed=41 + i, root=root) for i, (name, raw) in enumerate(KVZ.items())}


def plain_logits(folder, tokens):
    """The plain logits [T, vocab + 1]: the last column says (1 or 0) whether every router decision up to and with that
    token was clear of a close call.  It rides along through the tests' slicing and stacking; `_close` takes it off."""
    logits, sure = plain_logits_and_sure(folder, tokens)
    return torch.cat([logits, sure.to(logits.dtype)[:, None]], dim=-1)


def _close(got, want, dtype):
    """float32: every position within the common bound.  bfloat16: a router logit that is a close call in the plain
    implementation may fall the other way after 8-bit roundings; that token then differs by a whole expert, and the later
    ones of its sequence, which read it through the cache and the recurrent state, by a good part of that.  So the positions
    before a sequence's first close call stay within five times the bound, at most one in eight of them beyond the bound
    itself; over all positions the median stays within the bound and every position is sane.  (The kernels alone are held
    to tight bounds in bfloat16 above, and every schedule to the float32 bound at every position.)"""
    got, want = torch.as_tensor(got, dtype=F).cpu(), torch.as_tensor(want, dtype=F).cpu()
    if got.dim() == 1:
        got, want = got[None], want[None]
    sure = torch.ones(want.shape[0], dtype=torch.bool)
    if want.shape[-1] == got.shape[-1] + 1:
        want, sure = want[:, :-1], want[:, -1] > 0.5
    assert got.shape == want.shape, (got.shape, want.shape)
    errors = (got - want).abs().amax(-1) / want.abs().max().clamp_min(1e-30)
    bound = TOLERANCE[dtype]
    if dtype == "float32":
        return bool((errors < bound).all())
    ok = bool((errors[sure] < 5 * bound).all()) and int((errors[sure] >= bound).sum()) <= max(1, int(sure.sum()) // 8) \
        and bool((errors < 1.0).all()) and float(errors.median()) < bound
    if not ok:
        print("positions", errors.numel(), "sure", int(sure.sum()), "beyond the bound among the sure", int((errors[sure] >= bound).sum()),
              "median", round(float(errors.median()), 4),
              "largest", [(int(i), round(float(errors[i]), 3), bool(sure[i])) for i in errors.argsort(descending=True)[:12]])
    return ok


def _rounded(t, dtype):
    return t.to(dtype).to(F)


# ----------------------------------------------------------------------------------- kernels alone

def _pools(T, G, D, Dv, page_size, device, dtype, shuffle_seed=0):
    """Fresh pools with the sequence's pages in a shuffled order: pools, page table, slot mapping, positions."""
    pages = -(-T // page_size)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(shuffle_seed)) + 1
    k_pool = torch.full((pages + 1, G, page_size, D), float("nan"), dtype=dtype, device=device)
    v_pool = torch.full((pages + 1, G, page_size, Dv), float("nan"), dtype=dtype, device=device)
    positions = torch.arange(T, dtype=torch.int32)
    mapping = (order[positions // page_size].to(torch.int32) * page_size + positions % page_size).to(torch.int32).to(device)
    return k_pool, v_pool, order.to(torch.int32)[None, :].contiguous().to(device), mapping, positions.to(device)


def _scaling(rot):
    """(dims, base[, (factor, original, fast, slow)]) -> the stretching as the plain frequencies take it."""
    if rot is None or len(rot) < 3:
        return None
    return dict(zip(("factor", "original", "fast", "slow"), rot[2]))


def _tables(dims, base, scaling, positions, device):
    """float32 cos / sin tables [positions, dims / 2] as the plain frequencies give them."""
    f, magnitude = pk.pair_frequencies(dims, base, scaling)
    angle = (torch.arange(positions, dtype=torch.float32)[:, None] * f.float()[None, :]).double()
    return ((torch.cos(angle) * magnitude).float().contiguous().to(device), (torch.sin(angle) * magnitude).float().contiguous().to(device),
            f, magnitude)


def _capped_attend(q, k, v, rot, vrot_base, temperature, scale, cap, sink, dtype, device, page_size=64, q_len=None, kernel=None,
                   eps=1e-5):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] (float64, already rounded to `dtype`) through rotate_norm_store and the
    attention kernel; the last `q_len` tokens are the step (the earlier ones are stored by a step of their own)."""
    from models_b200.kernels import ops

    T, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    q_len = T if q_len is None else q_len
    k_pool, v_pool, table, mapping, positions = _pools(T, G, D, Dv, page_size, device, dtype)
    cos = sin = vcos = vsin = None
    dims = 0
    if rot is not None:
        dims = rot[0]
        cos, sin, _, _ = _tables(dims, rot[1], _scaling(rot), T, device) if dims else (None, None, None, None)
    if vrot_base:
        vcos, vsin, _, _ = _tables(Dv, vrot_base, None, T, device)
    qd, kd, vd = (t.reshape(T, -1).to(dtype).to(device).contiguous() for t in (q, k, v))
    temp = None if temperature is None else temperature.float().to(device).contiguous()
    out = torch.empty((q_len, H * Dv), dtype=dtype, device=device)
    first = T - q_len
    if first:
        ops.rotate_norm_store(qd[:first].clone(), kd[:first], vd[:first], positions[:first], cos, sin, dims, True, True, eps, vcos, vsin,
                              Dv if vrot_base else 0, k_pool, v_pool, mapping[:first], H, G, D, Dv)
    qs = qd[first:].clone()
    ops.rotate_norm_store(qs, kd[first:], vd[first:], positions[first:], cos, sin, dims, True, True, eps, vcos, vsin,
                          Dv if vrot_base else 0, k_pool, v_pool, mapping[first:], H, G, D, Dv)
    cu_q = torch.tensor([0, q_len], dtype=torch.int32, device=device)
    kv_lens = torch.tensor([T], dtype=torch.int32, device=device)
    ops.gated_attention(qs, out, k_pool, v_pool, table, cu_q, kv_lens, q_len, H, G, D, Dv, "softmax", scale, head_scale=temp,
                        softcap=cap or 0.0, sink=sink, turn_cos=vcos, turn_sin=vsin, kernel=kernel)
    return out.double().cpu().reshape(q_len, H, Dv)


def _plain_capped_attend(q, k, v, rot, vrot_base, temperature, scale, cap, sink, eps=1e-5):
    T, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    positions = torch.arange(T, dtype=F)
    if rot is not None and rot[0]:
        f, magnitude = pk.pair_frequencies(rot[0], rot[1], _scaling(rot))
        q, k = pk.rotate_interleaved(q, positions, f, magnitude, torch.float32), pk.rotate_interleaved(k, positions, f, magnitude, torch.float32)
    q, k = pk.rms_norm(q, None, eps), pk.rms_norm(k, None, eps)
    if vrot_base:
        vf, _ = pk.pair_frequencies(Dv, vrot_base)
        v = pk.rotate_interleaved(v, positions, vf, 1.0, torch.float32)
    heads = []
    for h in range(H):
        g = h // (H // G)
        s = pk.capped_scores(q[:, h], k[:, g], scale, 1.0 if temperature is None else temperature[h], cap)
        if sink:
            p = pk.sink_softmax(s)
        else:
            p = torch.softmax(s.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), -math.inf), dim=-1)
        heads.append(p @ v[:, g])
    o = torch.stack(heads, dim=1)
    if vrot_base:
        o = pk.rotate_interleaved(o, -positions, vf, 1.0, torch.float32)
    return o


KERNEL_TOLERANCE = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot,page", [
    (1, 1, 8, 8, None, 32), (3, 1, 9, 6, None, 32), (6, 2, 20, 12, (10, 3000.0, (2.0, 32, 8.0, 2.0)), 64), (3, 3, 40, 72, (40, 50.0), 128),
    (4, 1, 64, 128, (32, 1e5, (4.0, 128, 16.0, 1.0)), 64), (2, 2, 18, 14, (0, 100.0), 64), (8, 4, 32, 160, (16, 1e4), 64)])
def test_capped_attention_sizes_rotation_cap_sink_in_every_form(cuda_device, heads, kv_heads, dim, vdim, rot, page, dtype):
    """Random heads: a whole prompt (the tensor-core form where it applies, and the form with a warp per row), a prompt's last
    portion, and one decoded token (keys cut into runs), with pages in a shuffled order."""
    g = torch.Generator().manual_seed(heads * 100 + dim)
    T = 203
    q, k, v = (_rounded(torch.randn(T, h, d, generator=g, dtype=F), dtype) for h, d in ((heads, dim), (kv_heads, dim), (kv_heads, vdim)))
    temperature = torch.rand(heads, generator=g, dtype=F) + 0.5
    base = rot[1] if rot is not None else 0.0
    for cap, sink in ((4.0, True), (None, False), (40.0, True)):
        want = _plain_capped_attend(q, k, v, rot, base, temperature, 0.3, cap, sink)
        scale = float(want.abs().max())
        for q_len, kernel in ((T, None), (T, "rows"), (75, None), (2, None), (1, None)):
            got = _capped_attend(q, k, v, rot, base, temperature, 0.3, cap, sink, dtype, cuda_device, page, q_len, kernel)
            assert float((got - want[T - q_len:]).abs().max()) / scale < KERNEL_TOLERANCE[dtype], (cap, sink, q_len, kernel)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,target", [(700, 3), (700, 0), (130, 63), (130, 64), (65, 64), (321, 255), (40, 39)])
def test_one_far_key_decides_and_the_sink_takes_the_rest(cuda_device, tokens, target, dtype):
    """Every key is orthogonal to the query except key `target`, whose score is large: the result is that key's value
    (turned back to the distance between the two positions) times exp(s) / (1 + (n - 1) + exp(s)) -- the sink and the
    other keys weigh 1 each.  Without the sink the denominator is one less.  Prompt and decoded token."""
    D, Dv = 16, 8
    q = torch.zeros(tokens, 1, D, dtype=F)
    k = torch.zeros(tokens, 1, D, dtype=F)
    q[:, 0, 0] = 1.0
    k[:, 0, 1] = 1.0
    k[target, 0, 0], k[target, 0, 1] = 1.0, 0.0
    g = torch.Generator().manual_seed(tokens + target)
    v = _rounded(torch.randn(tokens, 1, Dv, generator=g, dtype=F), dtype)
    # unit norm makes q.k = D for the target and 0 for the others; scale 0.5 -> score 8, cap 6 -> 6 tanh(8/6)
    for sink in (True, False):
        want = _plain_capped_attend(q, k, v, None, 77.0, None, 0.5, 6.0, sink)
        s = 6.0 * math.tanh(8.0 / 6.0)
        n = tokens  # the last query sees all keys
        share = math.exp(s) / ((1.0 if sink else 0.0) + (n - 1) + math.exp(s)) if target < tokens else 0.0
        assert want[-1, 0].norm() > 0.5 * share * v[target, 0].norm()  # the plain result is indeed that key's value, mostly
        for q_len in (tokens, 1):
            got = _capped_attend(q, k, v, None, 77.0, None, 0.5, 6.0, sink, dtype, cuda_device, 64, q_len)
            assert float((got[-1] - want[-1]).abs().max()) / float(want[-1].abs().max()) < KERNEL_TOLERANCE[dtype], (sink, q_len)
    # and the sink alone: with every score at -cap the weights are tiny and the result nearly vanishes
    q2 = q.clone()
    q2[:, 0, 0] = -1.0
    k2 = torch.zeros_like(k)
    k2[:, 0, 0] = 1.0
    with_sink = _capped_attend(q2, k2, v, None, 0.0, None, 0.5, 6.0, True, dtype, cuda_device, 64, 1)
    without = _capped_attend(q2, k2, v, None, 0.0, None, 0.5, 6.0, False, dtype, cuda_device, 64, 1)
    mean = v[:, 0].mean(0)
    weight = tokens * math.exp(-s) / (1.0 + tokens * math.exp(-s))
    assert float((with_sink[0, 0] - weight * mean).abs().max()) < 2e-2 * float(mean.abs().max()) + 1e-4
    assert float((without[0, 0] - mean).abs().max()) < 2e-2 * float(mean.abs().max()) + 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotated_values_come_back_by_the_distance(cuda_device, dtype):
    """A query that sees one key only (its own, by a huge score): the value goes in rotated by j and comes out turned back by
    i = j, so the result is the value itself; and one far key: the value comes out turned by j - i."""
    D, Dv, T = 8, 12, 150
    q = torch.zeros(T, 1, D, dtype=F)
    k = torch.zeros(T, 1, D, dtype=F)
    for t in range(T):  # key t points along coordinate t % D with a sign pattern that makes only q_t . k_t large
        q[t, 0, t % D] = 1.0
        k[t, 0, t % D] = 1.0 if t % (2 * D) < D else -1.0
        q[t, 0, t % D] = k[t, 0, t % D]
    g = torch.Generator().manual_seed(3)
    v = _rounded(torch.randn(T, 1, Dv, generator=g, dtype=F), dtype)
    want = _plain_capped_attend(q, k, v, None, 20.0, None, 4.0, None, False)
    for q_len in (T, 1):
        got = _capped_attend(q, k, v, None, 20.0, None, 4.0, None, False, dtype, cuda_device, 64, q_len)
        assert float((got - want[T - q_len:]).abs().max()) / float(want.abs().max()) < KERNEL_TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams,width,tokens", [(1, 50, 3), (2, 256, 70), (3, 64, 1), (8, 72, 33)])
def test_reading_and_writing_the_streams(cuda_device, streams, width, tokens, dtype):
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(streams * 7 + width)
    x = torch.randn(tokens, streams, width, generator=g, dtype=F)
    read, out = torch.randn(streams, generator=g, dtype=F), torch.randn(streams, generator=g, dtype=F)
    mix = torch.randn(streams, streams, generator=g, dtype=F)
    gain = 1.0 + 0.1 * torch.randn(width, generator=g, dtype=F)
    y = _rounded(torch.randn(tokens, width, generator=g, dtype=F), dtype)
    dev = lambda t: t.float().contiguous().to(cuda_device)  # noqa: E731
    xd = dev(x.reshape(tokens, streams * width))
    u = torch.einsum("s,tsd->td", read, x.float().double())
    got = ops.hyper_read_norm(xd, dev(read), dev(gain), 1e-5, dtype)
    assert scaled_error(got, pk.rms_norm(u, gain, 1e-5)) < KERNEL_TOLERANCE[dtype]
    wide = torch.zeros(tokens, width + 8, dtype=dtype, device=cuda_device)
    wide[:, 8:] = y.to(dtype).to(cuda_device)
    ops.hyper_write(xd, wide[:, 8:], dev(out), dev(mix))
    want = torch.einsum("sr,tsd->trd", mix.float().double(), x.float().double()) + out.float().double()[None, :, None] * y[:, None, :]
    assert scaled_error(xd.reshape(tokens, streams, width), want) < 2e-6
    assert scaled_error(ops.stream_sum(xd, width), want.sum(1)) < 2e-6
    copies = ops.stream_copies(dev(y), streams).reshape(tokens, streams, width)
    assert all(torch.equal(copies[:, s], dev(y)) for s in range(streams))
    # writing and the next reading in one pass: the oracle's numbers, and the same bits as the two kernels one after the other
    read2 = torch.randn(streams, generator=g, dtype=F)
    y32 = dev(torch.randn(tokens, width, generator=g, dtype=F))
    one, two = dev(x.reshape(tokens, streams * width)), dev(x.reshape(tokens, streams * width))
    got = ops.hyper_write_read_norm(one, y32, dev(out), dev(mix), dev(read2), dev(gain), 1e-5, dtype)
    ops.hyper_write(two, y32, dev(out), dev(mix))
    assert torch.equal(one, two) and torch.equal(got, ops.hyper_read_norm(two, dev(read2), dev(gain), 1e-5, dtype))
    want = torch.einsum("sr,tsd->trd", mix.float().double(), x.float().double()) + out.float().double()[None, :, None] * y32.double().cpu()[:, None, :]
    assert scaled_error(one.reshape(tokens, streams, width), want) < 2e-6
    assert scaled_error(got, pk.rms_norm(torch.einsum("s,tsd->td", read2.float().double(), want), gain, 1e-5)) < KERNEL_TOLERANCE[dtype]


@pytest.mark.parametrize("experts,top,width,ff,tokens", [(4, 2, 64, 40, 70), (7, 3, 200, 136, 333), (16, 1, 128, 264, 500), (3, 3, 72, 8, 129),
                                                         (33, 4, 96, 48, 64)])
def test_routed_experts_on_padded_tiles(cuda_device, experts, top, width, ff, tokens):
    """The prompt form: every expert's rows padded to tiles of 128 (experts with no row, with a few and with more than a tile),
    both products grouped on the tensor cores (widths and hidden sizes that are no multiples of the tile among them), and the
    combination through each entry's row."""
    from models_b200.kernels import ops

    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(experts * 7 + top)
    x = _rounded(torch.randn(tokens, width, generator=g, dtype=F), dtype)
    router = _rounded(torch.randn(experts, width, generator=g, dtype=F) * 0.3, dtype)
    if experts > 3:
        router[2] = 0.0
        router[2, 0] = -50.0  # an expert that only tokens with a very negative first element pick
        router[0] = router[0] * 4  # one expert with many rows
        router = _rounded(router, dtype)
    names = {"router": router}
    for e in range(experts):
        names[f"e{e}.gate"], names[f"e{e}.up"] = (_rounded(torch.randn(ff, width, generator=g, dtype=F) * 0.4, dtype) for _ in range(2))
        names[f"e{e}.down"] = _rounded(torch.randn(width, ff, generator=g, dtype=F) * 0.2, dtype)
    dev = lambda t: t.to(dtype).contiguous().to(cuda_device)  # noqa: E731
    xd = dev(x)
    chosen, weights = ops.router_topk(xd, dev(router), top)
    want_chosen, _ = pk.route(x, router, top)
    assert torch.equal(chosen.cpu().long(), want_chosen)
    stack = lambda role: torch.stack([names[f"e{e}.{role}"] for e in range(experts)])  # noqa: E731
    gate_up, down = dev(torch.stack([stack("gate"), stack("up")])), dev(stack("down"))
    assert ops.grouped_product_takes(gate_up, down)
    plan = ops.route_pad(chosen, experts)
    position, order, groups = plan.position.cpu().long(), plan.sorted.cpu().long(), plan.tile_group.cpu().long()
    assert torch.equal(order[position], torch.arange(tokens * top))  # every entry lies at its row
    assert int((order >= 0).sum()) == tokens * top
    assert torch.equal(groups[position // plan.tile], want_chosen.reshape(-1))  # in a tile of its expert
    used = groups[groups >= 0]
    assert torch.equal(used, used.sort().values) and bool((groups[len(used):] < 0).all())
    limit = 0.8
    mid = ops.grouped_first_product(ops.gather_rows(xd, plan), gate_up, plan, limit, pk.SWISH_SLOPE)
    got = ops.expert_combine(ops.grouped_second_product(mid, down, plan), weights, position=plan.position)
    want = pk.routed_feed_forward(x, names, "", {"router": {"experts": experts, "top": top}, "expert": {"limit": limit}})
    assert scaled_error(got, want) < KERNEL_TOLERANCE[dtype]
    assert ops.gemm_tcgen05_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,width,ff,tokens", [(6, 2, 64, 40, 1), (12, 4, 256, 80, 300), (3, 3, 50, 33, 77), (5, 1, 72, 36, 130),
                                                         (40, 8, 128, 64, 9), (300, 2, 64, 16, 70)])
def test_routed_experts(cuda_device, experts, top, width, ff, tokens, dtype):
    """Router choices (ties to the lower index), the softmax over the chosen logits, the grouped products with few and many
    rows per expert (experts nobody chose among them), the clamps, and the shared expert behind its gate."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(experts * 10 + top)
    x = _rounded(torch.randn(tokens, width, generator=g, dtype=F), dtype)
    router = _rounded(torch.randn(experts, width, generator=g, dtype=F) * 0.3, dtype)
    if experts > 3:
        router[experts - 1] = router[1]  # a tie: the lower index is chosen first
        router[2] = -3.0 * x[0] if tokens > 1 else router[2]  # an expert the first token never picks
        router = _rounded(router, dtype)
    names = {}
    for e in range(experts):
        names[f"e{e}.gate"], names[f"e{e}.up"] = (_rounded(torch.randn(ff, width, generator=g, dtype=F) * 0.4, dtype) for _ in range(2))
        names[f"e{e}.down"] = _rounded(torch.randn(width, ff, generator=g, dtype=F) * 0.2, dtype)
    names["router"] = router
    dev = lambda t: t.to(dtype).contiguous().to(cuda_device)  # noqa: E731
    xd = dev(x)
    chosen, weights = ops.router_topk(xd, dev(router), top)
    want_chosen, want_weights = pk.route(x, router, top)
    assert torch.equal(chosen.cpu().long(), want_chosen)
    assert scaled_error(weights, want_weights) < 1e-5
    limit = 0.8
    plan = ops.route_sort(chosen, experts)
    stack = lambda role: dev(torch.stack([names[f"e{e}.{role}"] for e in range(experts)]))  # noqa: E731
    for tensor_cores in (True, False):
        mid = ops.expert_first_product(xd, stack("gate"), stack("up"), plan, limit, pk.SWISH_SLOPE, tensor_cores)
        slot_out = ops.expert_second_product(mid, stack("down"), plan, tensor_cores)
        got = ops.expert_combine(slot_out, weights)
        mlp = {"router": {"experts": experts, "top": top}, "expert": {"limit": limit}}
        want = pk.routed_feed_forward(x, names, "", mlp)
        assert scaled_error(got, want) < KERNEL_TOLERANCE[dtype], tensor_cores
    # the form for few entries (entry by entry, nothing sorted); here with any number of them, also on rows of a wider tensor
    wide = torch.zeros((tokens, width + 8), dtype=dtype, device=cuda_device)
    wide[:, :width] = xd
    for rows in (xd, wide[:, :width]):
        by_entry = ops.expert_rows_second(ops.expert_rows_first(rows, stack("gate"), stack("up"), chosen, limit, pk.SWISH_SLOPE),
                                          stack("down"), chosen)
        assert scaled_error(ops.expert_combine(by_entry, weights), want) < KERNEL_TOLERANCE[dtype]
    shared = torch.randn(tokens, width, generator=g, dtype=F)
    score = _rounded(torch.randn(tokens, 1, generator=g, dtype=F), dtype)
    got = ops.expert_combine(slot_out, weights, shared.float().contiguous().to(cuda_device), dev(score))
    assert scaled_error(got, want + pk.sigmoid(score) * shared.float().double()) < KERNEL_TOLERANCE[dtype]
    gate, up = (_rounded(torch.randn(tokens, ff, generator=g, dtype=F) * 2, dtype) for _ in range(2))
    both = dev(torch.cat([gate, up], dim=1))
    out = torch.empty((tokens, ff), dtype=dtype, device=cuda_device)
    ops.clamped_swish(both[:, :ff], both[:, ff:], out, limit, pk.SWISH_SLOPE)
    gl, ul = torch.clamp(gate, max=limit), torch.clamp(up, -limit, limit)
    assert scaled_error(out, gl * pk.sigmoid(pk.SWISH_SLOPE * gl) * (ul + 1.0)) < KERNEL_TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("run_length", [0, 16, 7])
@pytest.mark.parametrize("heads,dim,vdim,decay", [(2, 16, 24, [0.9, 0.999]), (1, 32, 32, [1.0]), (3, 10, 6, [0.5, 0.0, 0.99]),
                                                  (4, 64, 128, [0.97, 0.99, 0.999, 0.9])])
def test_lightning_ragged_and_carried(cuda_device, heads, dim, vdim, decay, run_length, dtype):
    """The retention kernel in its lightning form (silu on q, k, v; raw results; one norm over all heads; sigmoid gate): three
    sequences of unequal lengths in one step, the second continuing from a stored state."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(heads + dim)
    lengths = [37, 1, 90]
    T = sum(lengths)
    W = heads * (2 * dim + 2 * vdim)
    proj = _rounded(torch.randn(T, W, generator=g, dtype=F), dtype)
    gain = 1.0 + 0.1 * torch.randn(heads * vdim, generator=g, dtype=F)
    start = torch.randn(heads, dim, vdim, generator=g, dtype=F).float().double()
    at = [0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim]
    pd = proj.to(dtype).contiguous().to(cuda_device)
    q, k = pd[:, at[0]:at[1]], pd[:, at[1]:at[2]]
    v, gate = pd[:, at[2]:at[3]], pd[:, at[3]:]
    state = torch.zeros(5, heads, dim, vdim, dtype=torch.float32, device=cuda_device)
    state[3] = start.float().to(cuda_device)
    slots = torch.tensor([1, 3, 0], dtype=torch.int32, device=cuda_device)
    cu = torch.tensor([0, 37, 38, 128], dtype=torch.int32, device=cuda_device)
    positions = torch.cat([torch.arange(n) for n in lengths]).to(torch.int32).to(cuda_device)
    raw = torch.empty(T, heads * vdim, dtype=torch.float32, device=cuda_device)
    out = torch.empty(T, heads * vdim, dtype=dtype, device=cuda_device)
    ops.retention_scan(q, k, v, None, positions, None, None, 0, torch.tensor(decay, dtype=torch.float32, device=cuda_device), 1.0, 1e-5,
                       state, slots, cu, heads, dim, vdim, None, 1.0, max(lengths), run_length=run_length, input_activation="silu",
                       raw_out=raw)
    ops.group_norm_gate(raw, gain.float().to(cuda_device), gate, out, 1e-5, "sigmoid")
    row = 0
    for n, slot, begin in zip(lengths, (1, 3, 0), (None, start, None)):
        part = proj[row:row + n]
        qs, ks = (pk.silu(part[:, a:b]).reshape(n, heads, dim) for a, b in ((at[0], at[1]), (at[1], at[2])))
        vs = pk.silu(part[:, at[2]:at[3]]).reshape(n, heads, vdim)
        heads_out, finals = zip(*[pk.lightning_recurrence(qs[:, h], ks[:, h], vs[:, h], decay[h], None if begin is None else begin[h])
                                  for h in range(heads)])
        o = torch.stack(heads_out, dim=1).reshape(n, heads * vdim)
        want = pk.rms_norm(o, gain, 1e-5) * pk.sigmoid(part[:, at[3]:])
        assert scaled_error(out[row:row + n], want) < KERNEL_TOLERANCE[dtype], slot
        assert scaled_error(state[slot], torch.stack(finals)) < 2e-5, slot
        row += n


# ----------------------------------------------------------------------------------- the model in the engine

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(KVZ))
def test_whole_prompt_every_position(cuda_device, folders, name, dtype):
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    for n, seed in ((1, 1), (2, 5), (7, 2), (70, 3), (200, 4)):
        tokens = random_tokens(KVZ[name]["vocab"], n, seed)
        slot = engine.open_slot()
        logits = engine.step([StepEntry(slot, tokens, list(range(n)))])
        engine.release_slot(slot)
        assert _close(logits, plain_logits(folders[name], tokens), dtype), (name, dtype, n)
    engine.cache.check()


@pytest.mark.parametrize("name", sorted(KVZ))
def test_residual_stream_after_every_run_of_a_layer(cuda_device, folders, name):
    """The sum of the streams after every run of the schedule (a looped layer counts each time), in float32."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], "float32")
    tokens = random_tokens(KVZ[name]["vocab"], 90, 6)
    seen = []
    engine.model.observer = lambda run, x: seen.append(x.double().cpu())
    slot = engine.open_slot()
    engine.step([StepEntry(slot, tokens, [89])])
    expected = []
    plain_logits_alone(folders[name], tokens, expected)
    raw = KVZ[name]
    loop = raw.get("loop") or {"start": 0, "stop": 0, "times": 1}
    assert len(expected) == len(raw["layers"]) + (loop["stop"] - loop["start"]) * (loop["times"] - 1)
    assert len(seen) == len(expected)
    for run, (got, want) in enumerate(zip(seen, expected)):
        assert scaled_error(got, want) < 1e-5, run


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(KVZ))
def test_prompt_then_token_by_token(cuda_device, folders, name, dtype):
    """A short prompt, then 130 tokens one by one: the decode form of the attention crosses cache pages, every pass of a
    looped layer reads the cache and the state of its own, and the lightning state is carried through every step."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    n, head = 150, 20
    tokens = random_tokens(KVZ[name]["vocab"], n, 7)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, tokens[:head], [head - 1])])]
    for i in range(head, n):
        rows.append(engine.step([StepEntry(slot, [tokens[i]], [0])]))
    assert _close(torch.cat(rows), expected[head - 1:], dtype)
    engine.cache.check()
    engine.release_slot(slot)
    assert all(g.pages.held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "D"])
def test_token_by_token_from_the_first_token(cuda_device, folders, name, dtype):
    """No prompt step at all: the first tokens of a sequence go through the decode kernels (one key and the sink; a state
    that starts at zero)."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    tokens = random_tokens(KVZ[name]["vocab"], 70, 17)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, [t], [0])]) for t in tokens]
    assert _close(torch.cat(rows), expected, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,portions", [("A", [2, 3, 17, 64, 1, 2, 90, 21]), ("B", [64, 64, 2, 70]), ("C", [130, 2, 68]),
                                           ("D", [5, 2, 2, 129, 62])])
def test_prompt_in_portions(cuda_device, folders, name, portions, dtype):
    """A portion starts inside a sequence: its recurrence goes on from the stored state, its queries see the keys and the
    rotated values of earlier portions, and its positions go on from where it stands."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    tokens = random_tokens(KVZ[name]["vocab"], sum(portions), 8)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    at, rows = 0, []
    for count in portions:
        rows.append(engine.step([StepEntry(slot, tokens[at:at + count], list(range(count)))]).clone())
        if dtype == "float32":
            assert _close(rows[-1], expected[at:at + count], dtype), (at, count)
        at += count
    assert _close(torch.cat(rows), expected, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(KVZ))
def test_unequal_batches_and_slots_used_again(cuda_device, folders, name, dtype):
    """Four prompts of unequal lengths in one step, decoded together while the shorter ones end; then new requests take the
    freed slots and pages (their states must start at zero, their pages hold old keys and values)."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype, max_tokens=1024)
    vocab = KVZ[name]["vocab"]
    for round_index in range(2):
        lengths, prompts = [1, 33, 140, 70], [1, 20, 131, 66]
        full = [random_tokens(vocab, n + 12, 10 * round_index + i) for i, n in enumerate(lengths)]
        expected = [plain_logits(folders[name], t) for t in full]
        slots = [engine.open_slot() for _ in full]
        out = engine.step([StepEntry(s, t[:p], [0, p - 1]) for s, t, p in zip(slots, full, prompts)])
        want = torch.stack([expected[i][r] for i, p in enumerate(prompts) for r in (0, p - 1)])
        assert _close(out, want, dtype), round_index
        live = list(range(4))
        at = list(prompts)
        got_rows, want_rows = [], []
        while live:
            out = engine.step([StepEntry(slots[i], [full[i][at[i]]], [0]) for i in live])
            for row, i in enumerate(live):
                got_rows.append(out[row].clone())
                want_rows.append(expected[i][at[i]])
                at[i] += 1
            for i in [i for i in live if at[i] == len(full[i])]:
                engine.release_slot(slots[i])
                live.remove(i)
        assert _close(torch.stack(got_rows), torch.stack(want_rows), dtype), round_index
        engine.cache.check()
    assert engine.cache.slots.held == 0 and all(g.pages.held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_from_graphs(cuda_device, folders, name, dtype):
    """Three sequences decoded for 330 steps from captured steps, over several pages; one sequence ends on the way and
    another takes its slot (and must not inherit its state or its keys)."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype, max_tokens=4096)
    engine.enable_decode_graphs(4)
    vocab = KVZ[name]["vocab"]
    full = [random_tokens(vocab, n, 20 + i) for i, n in enumerate((340, 200, 150, 120))]
    expected = [plain_logits(folders[name], t) for t in full]
    prompts = [5, 70, 1, 30]
    slots = {i: engine.open_slot() for i in range(3)}
    engine.step([StepEntry(slots[i], full[i][:prompts[i]], []) for i in range(3)])
    at = {i: prompts[i] for i in range(3)}
    got_rows, want_rows = [], []
    while at:
        live = sorted(at)
        out = engine.decode([slots[i] for i in live], [full[i][at[i]] for i in live])
        for row, i in enumerate(live):
            if at[i] % 7 == 0 or at[i] > len(full[i]) - 3:
                got_rows.append(out[row].clone())
                want_rows.append(expected[i][at[i]])
            at[i] += 1
            if at[i] == len(full[i]):
                engine.release_slot(slots.pop(i))
                del at[i]
                if i == 2:  # a new request in the freed slot, from its prompt
                    slots[3] = engine.open_slot()
                    engine.step([StepEntry(slots[3], full[3][:prompts[3]], [])])
                    at[3] = prompts[3]
    assert _close(torch.stack(got_rows), torch.stack(want_rows), dtype)
    assert engine.decode_graphs.captured  # the steps did come from captures
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["lightning", "attention"])
def test_models_of_one_kind_of_layer(cuda_device, tmp_path, kind, dtype):
    """Only lightning layers (no cache group at all, state alone) or only attention layers (no state): prompts of one length
    class four times over, then tokens one by one from captured decode steps; the whole model looped three times."""
    from models_b200.engine import StepEntry

    layers = {"lightning": [lightning(2, 16, 24, [0.9, 0.99], dense(48)), lightning(1, 32, 16, [0.95], None)],
              "attention": [attention(4, 2, 16, 8, 0.25, (16, 1e4), 9.0, moe(4, 2, 24, 2.0)),
                            attention(2, 1, 32, 32, 0.2, (8, 300.0, (2.0, 48, 6.0, 1.5)), None, None)]}[kind]
    raw = {"architecture": "Kivezen", "vocab": 120, "width": 64, "norm": {"eps": 1e-5}, "streams": 4, "layers": layers,
           "loop": {"start": 0, "stop": 2, "times": 3}}
    folder = make_folder(raw, 90, tmp_path)
    engine = _engine(folder, dtype, 1024)
    engine.enable_decode_graphs(4)
    assert (len(engine.cache.groups) == 0) == (kind == "lightning")
    for seed in range(4):
        tokens = random_tokens(120, 140, seed)
        want = plain_logits(folder, tokens)
        slot = engine.open_slot()
        rows = [engine.step([StepEntry(slot, tokens[:100], [99])])]
        for t in tokens[100:]:
            rows.append(engine.decode([slot], [t]).clone())
        assert _close(torch.cat(rows), want[99:], dtype), seed
        engine.release_slot(slot)
    engine.cache.check()


def test_every_pass_of_a_looped_layer_has_a_cache_and_a_state_of_its_own(cuda_device, folders):
    from models_b200.engine import StepEntry

    engine = _engine(folders["A"], "float32")
    raw = KVZ["A"]
    loop = raw["loop"]
    runs = len(raw["layers"]) + (loop["stop"] - loop["start"]) * (loop["times"] - 1)
    order = list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], len(raw["layers"])))
    assert [entry.layer for entry in engine.model.spec.schedule] == order and len(order) == runs
    attention_runs = sum(raw["layers"][i]["type"] == "attention" for i in order)
    lightning_runs = runs - attention_runs
    assert sum(len(g.runs) for g in engine.cache.groups) == attention_runs
    assert len(engine.state.tensors) == lightning_runs
    slot = engine.open_slot()
    engine.step([StepEntry(slot, random_tokens(raw["vocab"], 40, 3), [])])
    states = [t[slot].clone() for t in engine.state.tensors.values()]
    assert all(float(s.abs().max()) > 0 for s in states)


def test_logits_do_not_depend_on_the_batch_or_the_cut(cuda_device, folders):
    """float32: the same position through a whole prompt, through portions, and inside a batch differs by rounding only."""
    from models_b200.engine import StepEntry

    for name in ("A", "C"):
        engine = _engine(folders[name], "float32")
        vocab = KVZ[name]["vocab"]
        a, b = random_tokens(vocab, 100, 31), random_tokens(vocab, 37, 32)
        slot = engine.open_slot()
        whole = engine.step([StepEntry(slot, a, [99])])
        engine.release_slot(slot)
        s1, s2 = engine.open_slot(), engine.open_slot()
        engine.step([StepEntry(s2, b[:30], []), StepEntry(s1, a[:64], [])])
        engine.step([StepEntry(s1, a[64:99], []), StepEntry(s2, b[30:], [])])
        cut = engine.step([StepEntry(s1, a[99:], [0])])
        assert scaled_error(cut, whole) < 5e-6, name


def test_greedy_generation_through_the_entry_point(cuda_device, folders):
    import models_b200

    folder = folders["A"]
    prompts = [random_tokens(KVZ["A"]["vocab"], n, 50 + n) for n in (3, 40, 11)]
    steps = 40
    config, weights = pk.read_model_folder(folder)
    expected, margins = [], []
    for prompt in prompts:
        tokens, out, margin = list(prompt), [], []
        for _ in range(steps):
            logits = pk.forward(config, weights, tokens)[-1]
            top = torch.topk(logits, 2).values
            margin.append(float(top[0] - top[1]))
            out.append(int(torch.argmax(logits)))
            tokens.append(out[-1])
        expected.append(out)
        margins.append(margin)
    for dtype in DTYPES:
        model = models_b200.load_model(folder, dtype=dtype, max_batch=4, context=256)
        results = model.generate_batch(prompts, models_b200.SamplingOptions(temperature=0.0, max_tokens=steps))
        for result, want, margin in zip(results, expected, margins):
            for i, (a, b) in enumerate(zip(result.tokens, want)):
                if a != b:
                    assert dtype == "bfloat16" and margin[i] < 0.05, (dtype, i, result.tokens, want)
                    break
        model.close()


def test_trace_replay_program(cuda_device, folders, tmp_path):
    """bin/trace_run on a Kivezen folder: two prompts in one step, then decoded together from captured steps."""
    name = "D"
    vocab = KVZ[name]["vocab"]
    a, b = random_tokens(vocab, 90, 1), random_tokens(vocab, 12, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for i in range(20):
        entries = [{"id": "a", "tokens": [a[70 + i]], "want": [0]}]
        if i < 7:
            entries.append({"id": "b", "tokens": [b[5 + i]], "want": [0]})
        steps.append({"step": i + 1, "entries": entries, "end": (["b"] if i == 6 else []) + (["a"] if i == 19 else [])})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ea, eb = plain_logits(folders[name], a), plain_logits(folders[name], b)
    for dtype in DTYPES:
        proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folders[name]), "--dtype", dtype,
                               "--out", str(out), "--max-tokens", "102"],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        first = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, vocab)
        got = [first[0], first[1], first[2]]
        want = [ea[0], ea[69], eb[4]]
        for i in range(20):
            rows = np.fromfile(out / f"{i + 1}.f32", dtype="<f4").reshape(-1, vocab)
            got.append(rows[0])
            want.append(ea[70 + i])
            if i < 7:
                got.append(rows[1])
                want.append(eb[5 + i])
        assert _close(np.stack(got), torch.stack(want), dtype), dtype
